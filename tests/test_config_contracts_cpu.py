"""Switches that are accepted on the command line must either do something or be refused with a clear message; none may
parse and vanish.  Also the engine actor's control surface (sleep / wake_up / reset_prefix_cache / set_model_step and the
two-phase weight update that keeps a forward pass from running on half-written weights)."""

import threading
import time

import pytest
import torch


def test_quantised_loading_is_refused():
    from open_instruct_b200.config.schemas import ModelConfig

    ModelConfig(model_name_or_path="tiny", lora_target_modules=["q_proj", "v_proj"])
    for kw in (dict(load_in_4bit=True), dict(load_in_8bit=True), dict(use_bnb_nested_quant=True)):
        with pytest.raises(ValueError, match="quantised base weights"):
            ModelConfig(model_name_or_path="tiny", **kw)
    with pytest.raises(ValueError, match="lora_target_modules"):
        ModelConfig(model_name_or_path="tiny", lora_target_modules=["router"])
    assert ModelConfig(model_name_or_path="tiny", gradient_checkpointing=True, use_cache=True).use_cache is False


def test_context_parallel_maps_to_ulysses_or_is_refused():
    from open_instruct_b200.config.schemas import check_context_parallel

    assert check_context_parallel(None, "llama3") == 1 and check_context_parallel(1, "zig_zag") == 1
    assert check_context_parallel(2, "ulysses", world=8) == 2
    for strategy in ("llama3", "zig_zag"):
        with pytest.raises(ValueError, match="ring attention"):
            check_context_parallel(2, strategy)
    with pytest.raises(ValueError, match="must divide"):
        check_context_parallel(3, "ulysses", world=8)


def test_dpo_and_sft_refuse_switches_they_cannot_honour(tmp_path):
    from open_instruct_b200.dpo_utils import DPOExperimentConfig
    from open_instruct_b200.finetune import FlatArguments

    base = dict(model_name_or_path="tiny", mixer_list=["x.jsonl", "1.0"])
    DPOExperimentConfig(**base)
    with pytest.raises(ValueError, match="context-parallel"):
        DPOExperimentConfig(**base, cp_degree=2, cp_strategy="ulysses")
    with pytest.raises(ValueError, match="ring attention"):
        DPOExperimentConfig(**base, cp_degree=2, cp_strategy="llama3")
    with pytest.raises(ValueError, match="mixture-of-experts"):
        DPOExperimentConfig(**base, load_balancing_loss=True)
    with pytest.raises(ValueError, match="quantised"):
        DPOExperimentConfig(**base, load_in_4bit=True)
    with pytest.raises(ValueError, match="offload_param is not built"):
        DPOExperimentConfig(**base, zero_stage=3, offload_param=True)
    FlatArguments(model_name_or_path="tiny", dataset_mixer_list=["x.jsonl", "1.0"], load_balancing_loss=True)  # accepted; a dense model refuses at start
    assert FlatArguments(model_name_or_path="tiny", dataset_mixer_list=["x.jsonl", "1.0"], use_qlora=True).use_lora  # QLoRA is built for SFT
    with pytest.raises(ValueError):
        FlatArguments(model_name_or_path="tiny", dataset_mixer_list=["x.jsonl", "1.0"], use_8bit_optimizer=True)


def test_grpo_eval_on_step_0_needs_local_eval():
    from open_instruct_b200.grpo_utils import GRPOExperimentConfig

    assert GRPOExperimentConfig(eval_on_step_0=True, local_eval_every=5).eval_on_step_0
    with pytest.raises(ValueError, match="eval_on_step_0"):
        GRPOExperimentConfig(eval_on_step_0=True, local_eval_every=0)
    assert GRPOExperimentConfig(sequence_parallel_size=2, deepspeed_stage=2).sequence_parallel_size == 2
    with pytest.raises(ValueError):
        GRPOExperimentConfig(sequence_parallel_size=0)
    with pytest.raises(ValueError, match="deepspeed_offload_param is not built"):
        GRPOExperimentConfig(deepspeed_offload_param=True)


def _engine_worker():
    import queue

    from open_instruct_b200.grpo_fast import EngineWorker
    from open_instruct_b200.models import get_spec

    return EngineWorker(get_spec("tiny"), queue.Queue(), queue.Queue(), queue.Queue(), None, device="cpu", ops="ref", max_model_len=64,
                        num_blocks=32)


def test_engine_control_rpcs():
    w = _engine_worker()
    try:
        w.set_model_step(7)
        assert w.engine.model_step == 7
        assert w.reset_prefix_cache() is True
        w.sleep()
        assert w.should_stop.is_set()
        w.wake_up()
        assert not w.should_stop.is_set()
        w.check_background_threads()
    finally:
        w.shutdown()


def test_control_calls_go_ahead_of_the_decode_loop():
    """A weight update is served after the step that is running, not after however many steps the loop manages to start while the
    caller waits for an unfair lock (measured before the fix: 4 to 20 seconds of engine steps per sync)."""
    w = _engine_worker()
    try:
        steps = []

        def quick_step():
            steps.append(time.perf_counter())
            time.sleep(0.002)
            return []

        w.engine.step = quick_step
        w.engine.has_unfinished = lambda: True
        time.sleep(0.1)
        assert len(steps) > 5  # the loop is spinning
        worst = 0
        for _ in range(20):
            n0 = len(steps)
            w.begin_weight_update()
            worst = max(worst, len(steps) - n0)
            w.abort_weight_update()
            time.sleep(0.005)
        assert worst <= 2, worst
    finally:
        w.engine.has_unfinished = lambda: False
        w.shutdown()


def test_weight_update_cannot_overlap_an_engine_step():
    """begin_weight_update waits for the running step and holds the next one back until update_weights ends the update."""
    w = _engine_worker()
    try:
        in_step, release, order = threading.Event(), threading.Event(), []
        real_step = w.engine.step

        def slow_step():
            in_step.set()
            order.append("step-start")
            release.wait(5)
            order.append("step-end")
            return real_step()

        w.engine.step = slow_step
        w.engine.has_unfinished = lambda: True  # make the loop step continuously
        assert in_step.wait(5)
        t = threading.Thread(target=lambda: (w.begin_weight_update(), order.append("update-open")))
        t.start()
        time.sleep(0.1)
        assert "update-open" not in order  # the step is still running: the update has to wait
        release.set()
        t.join(5)
        assert order.index("step-end") < order.index("update-open")
        n_before = order.count("step-start")
        time.sleep(0.1)
        assert order.count("step-start") == n_before  # no new step while the update is open
        new = torch.zeros_like(w.engine.model.flat)
        w.update_weights(new, 3)
        assert w.engine.model_step == 3 and float(w.engine.model.flat.abs().sum()) == 0.0
        time.sleep(0.1)
        assert order.count("step-start") > n_before  # the loop runs again
        w.begin_weight_update()
        w.abort_weight_update()  # a failed push releases the engine too
        assert w.lock.acquire(timeout=2)
        w.lock.release()
    finally:
        w.engine.has_unfinished = lambda: False
        release.set()
        w.shutdown()


def test_rope_scaling_flags_become_a_yarn_rule():
    from open_instruct_b200.config.schemas import ModelConfig, spec_with_rope_flags
    from open_instruct_b200.models import get_spec

    spec = get_spec("tiny")
    assert spec_with_rope_flags(spec, ModelConfig(model_name_or_path="tiny")) is spec
    out = spec_with_rope_flags(spec, ModelConfig(model_name_or_path="tiny", rope_scaling_factor=8.0, rope_scaling_old_context_len=4096))
    assert out.rope_scaling == {"rope_type": "yarn", "factor": 8.0, "beta_fast": 32.0, "beta_slow": 1.0, "original_max_position_embeddings": 4096}
    assert out.max_position_embeddings == 32768 and out.attn_scale > spec.attn_scale
