"""GRPO end to end on CPU in single-process mode: prompts -> engine -> rewards -> packing -> learner -> sync."""

import json
import os

import pytest

import torch

from helpers import make_rlvr_jsonl, make_tokenizer


def test_grpo_single_process(tmp_path):
    from open_instruct_b200.config.schemas import ModelConfig
    from open_instruct_b200.data.tokenize import TokenizerConfig
    from open_instruct_b200.grpo_fast import main
    from open_instruct_b200.grpo_utils import GRPOExperimentConfig
    from open_instruct_b200.streaming import StreamingDataLoaderConfig, VLLMConfig

    tmp = str(tmp_path)
    tok = make_tokenizer(os.path.join(tmp, "tok"))
    data = make_rlvr_jsonl(os.path.join(tmp, "rl.jsonl"), n=12)
    args = GRPOExperimentConfig(total_episodes=3 * 4 * 4, learning_rate=1e-3, beta=0.0, load_ref_policy=False, output_dir=os.path.join(tmp, "out"),
                                single_gpu_mode=True, ops="ref", seed=3, save_freq=-1, checkpoint_state_freq=2,
                                checkpoint_state_dir=os.path.join(tmp, "state"), lr_scheduler_type="constant", record_entropy=True,
                                local_eval_every=2, eval_pass_at_k=2)
    eval_data = make_rlvr_jsonl(os.path.join(tmp, "eval.jsonl"), n=3)
    streaming = StreamingDataLoaderConfig(max_prompt_token_length=64, response_length=12, pack_length=256, async_steps=1,
                                          num_samples_per_prompt_rollout=4, num_unique_prompts_rollout=4, dataset_mixer_list=[data, "1.0"],
                                          dataset_mixer_eval_list=[eval_data, "1.0"], dataset_mixer_eval_list_splits=["train"],
                                          dataset_local_cache_dir=os.path.join(tmp, "cache"), filter_zero_std_samples=False, temperature=1.0,
                                          save_traces=True, rollouts_save_path=os.path.join(tmp, "rollouts"))
    out = main(args, TokenizerConfig(tokenizer_name_or_path=tok, chat_template_name="tulu"), ModelConfig(model_name_or_path="tiny"), streaming,
               VLLMConfig())
    assert out["num_training_steps"] == 3 and out["training_step"] == 3
    # save_traces: every rollout of the three steps (4 prompts x 4 samples each) with reward, advantage, tokens and log-probs
    files = sorted(os.listdir(os.path.join(tmp, "rollouts")))
    assert any(f.endswith("_metadata.jsonl") for f in files) and any("_rollouts_000000.jsonl" in f for f in files)
    recs = [json.loads(l) for f in files if "_rollouts_" in f for l in open(os.path.join(tmp, "rollouts", f))]
    assert len(recs) >= 3 * 16 and {r["step"] for r in recs} >= {1, 2, 3}
    r0 = recs[0]
    assert len(r0["response_tokens"]) == len(r0["logprobs"]) > 0 and r0["ground_truth"] is not None and r0["finish_reason"] in ("stop", "length")
    with pytest.raises(ValueError, match="rollouts_save_path"):
        StreamingDataLoaderConfig(save_traces=True, rollouts_save_path="")
    lines = [json.loads(l) for l in open(os.path.join(args.output_dir, "metrics.jsonl"))]
    assert len(lines) == 3
    for l in lines:
        assert abs(l["val/ratio"] - 1.0) < 1e-4          # single pass: ratio is exactly one
        assert l["debug/vllm_vs_local_logprob_diff_mean"] < 1e-3 or l["training_step"] > 1   # engine == learner at step 1
        assert "policy/entropy_avg" in l and l["time/weight_sync"] >= 0
    assert os.path.exists(os.path.join(args.output_dir, "model.safetensors"))
    assert os.path.exists(os.path.join(tmp, "state", "step_2", "COMPLETED"))
    # evaluation prompts were submitted at step 2 and at the last step; the last step waits for its results
    assert lines[-1]["eval/num_prompts"] == 3 and "eval/pass_at_2" in lines[-1] and lines[-1]["eval/sequence_lengths"] > 0


def test_grpo_train_step_moves_policy_toward_advantage():
    from open_instruct_b200.data_types import CollatedBatchData
    from open_instruct_b200.grpo_fast import grpo_train_step
    from open_instruct_b200.grpo_utils import GRPOExperimentConfig
    from open_instruct_b200.learner import Learner, LearnerConfig
    from open_instruct_b200.models import get_spec
    from open_instruct_b200.rl_utils import pack_sequences

    spec = get_spec("tiny")
    learner = Learner(spec, LearnerConfig(ops="ref", learning_rate=5e-3, lr_scheduler_type="constant"))
    q = [[5, 6, 7]] * 2
    r = [[10, 11, 12], [20, 21, 22]]
    lp = [[-1.0] * 3] * 2
    p = pack_sequences(q, r, [[1] * 3] * 2, 64, 0, lp)
    adv = torch.tensor([0.0, 1.0, -1.0])
    p.advantages = [adv[m.long()] for m in p.response_masks]
    data = CollatedBatchData(p.query_responses, p.attention_masks, p.position_ids, p.advantages, p.response_masks, p.vllm_logprobs, p.cu_seqlens)
    args = GRPOExperimentConfig(beta=0.0, load_ref_policy=False, use_rho_correction=False)

    def seq_logp(resp):
        ids = torch.tensor(q[0] + resp)
        logits = learner.model.logits(ids, torch.arange(6), torch.tensor([0, 6], dtype=torch.int32))
        return torch.log_softmax(logits[2:5].float(), -1).gather(-1, ids[3:, None]).sum().item()

    before = seq_logp(r[0]), seq_logp(r[1])
    for _ in range(3):
        grpo_train_step(learner, data, args)
    after = seq_logp(r[0]), seq_logp(r[1])
    assert after[0] > before[0] and after[1] < before[1]


def test_grpo_train_step_label_space_matches_token_space():
    """Sequence parallelism keeps per-token quantities at the position that predicts the token (so that a rank never needs
    its neighbour's log-prob) instead of shifting the log-probs after the forward pass.  On one rank both forms must give
    the same metrics and the same parameter update, with rho correction, several mini-batches and two epochs."""
    from open_instruct_b200.data_types import CollatedBatchData
    from open_instruct_b200.grpo_fast import grpo_train_step
    from open_instruct_b200.grpo_utils import GRPOExperimentConfig
    from open_instruct_b200.learner import Learner, LearnerConfig
    from open_instruct_b200.models import get_spec
    from open_instruct_b200.rl_utils import pack_sequences

    spec = get_spec("tiny")
    g = torch.Generator().manual_seed(0)
    q = [torch.randint(1, 100, (int(n),), generator=g).tolist() for n in (5, 9, 4, 7)]
    r = [torch.randint(1, 100, (int(n),), generator=g).tolist() for n in (6, 3, 8, 5)]
    lp = [(-torch.rand(len(x), generator=g) * 3).tolist() for x in r]
    p = pack_sequences(q, r, [[1] * len(x) for x in r], 24, 0, lp)
    adv = torch.tensor([0.0, 1.0, -0.5, 0.7, -1.2])
    p.advantages = [adv[m.long()] for m in p.response_masks]
    data = CollatedBatchData(p.query_responses, p.attention_masks, p.position_ids, p.advantages, p.response_masks, p.vllm_logprobs, p.cu_seqlens)
    outs = []
    for force in (False, True):
        learner = Learner(spec, LearnerConfig(ops="ref", learning_rate=5e-3, lr_scheduler_type="constant", seed=3))
        args = GRPOExperimentConfig(beta=0.0, load_ref_policy=False, use_rho_correction=True, num_mini_batches=2, num_epochs=2, record_entropy=True)
        args._force_label_space = force
        m = grpo_train_step(learner, data, args)
        outs.append((m, learner.model.flat.detach().clone()))
    (m0, w0), (m1, w1) = outs
    assert torch.allclose(w0, w1, atol=1e-7), (w0 - w1).abs().max()
    for k in ("loss/policy_avg", "policy/clipfrac_avg", "val/ratio", "optim/grad_norm", "policy/entropy_avg", "num_response_tokens",
              "debug/vllm_vs_local_logprob_diff_mean"):
        assert abs(m0[k] - m1[k]) < 1e-5 * max(1.0, abs(m0[k])), (k, m0[k], m1[k])


@pytest.mark.parametrize("init", ["by_value", "by_first_sync"])
def test_grpo_multi_process_actors(tmp_path, init, monkeypatch):
    """Two learner processes (gloo) + one engine process + cross-process queues, CPU.  ``by_first_sync``: the engine starts with
    random weights and gets the learners' through the first weight sync (the GPU default), checked against the learner's checksum."""
    if init == "by_first_sync":
        monkeypatch.setenv("B200_GRPO_INIT_BY_PUSH", "force")
    from open_instruct_b200.actors import ray_compat as ray
    from open_instruct_b200.config.schemas import ModelConfig
    from open_instruct_b200.data.tokenize import TokenizerConfig
    from open_instruct_b200.grpo_fast import main
    from open_instruct_b200.grpo_utils import GRPOExperimentConfig
    from open_instruct_b200.streaming import StreamingDataLoaderConfig, VLLMConfig
    import open_instruct_b200.grpo_fast as gf

    tmp = str(tmp_path)
    tok = make_tokenizer(os.path.join(tmp, "tok"))
    data = make_rlvr_jsonl(os.path.join(tmp, "rl.jsonl"), n=12)
    args = GRPOExperimentConfig(total_episodes=2 * 4 * 4, learning_rate=1e-3, beta=0.0, load_ref_policy=False, output_dir=os.path.join(tmp, "out"),
                                num_learners_per_node=[2], ops="ref", seed=3, save_freq=-1, lr_scheduler_type="constant",
                                verify_weight_sync=True)
    streaming = StreamingDataLoaderConfig(max_prompt_token_length=64, response_length=8, pack_length=128, async_steps=1,
                                          num_samples_per_prompt_rollout=4, num_unique_prompts_rollout=4, dataset_mixer_list=[data, "1.0"],
                                          dataset_local_cache_dir=os.path.join(tmp, "cache"), filter_zero_std_samples=False)
    try:
        out = main(args, TokenizerConfig(tokenizer_name_or_path=tok, chat_template_name="tulu"), ModelConfig(model_name_or_path="tiny"),
                   streaming, VLLMConfig())
    finally:
        ray.shutdown()
    assert out["training_step"] == 2
    assert os.path.exists(os.path.join(args.output_dir, "model.safetensors"))


def test_engine_worker_runs_tool_sessions(tmp_path):
    """An engine worker with a counter environment: every sample is a multi-turn session."""
    import queue
    import time

    from transformers import AutoTokenizer

    from open_instruct_b200.data_types import PromptRequest, SamplingConfig
    from open_instruct_b200.environments.tools.utils import EnvsConfig
    from open_instruct_b200.grpo_fast import EngineWorker
    from open_instruct_b200.models import get_spec

    tok = AutoTokenizer.from_pretrained(make_tokenizer(os.path.join(str(tmp_path), "tok")))
    pq, rq = queue.Queue(), queue.Queue()
    w = EngineWorker(get_spec("tiny"), pq, rq, None, None, tok, device="cpu", ops="ref", num_blocks=256,
                     envs_config=EnvsConfig(envs=["counter"], tool_parser_type="vllm_hermes", max_steps=2))
    try:
        pq.put(PromptRequest(prompt=[5, 6, 7], generation_config=SamplingConfig(max_tokens=24, n=2, seed=1), index=3, prompt_id="0_3"))
        res = rq.get(timeout=120)
        assert res.index == 3 and len(res.responses) == 2
        assert all(len(r) == len(m) == len(l) for r, m, l in zip(res.responses, res.masks, res.logprobs))
        assert len(res.request_info.rollout_states) == 2 and res.reward_scores == [0.0, 0.0]
        w.check_background_threads()
    finally:
        w.shutdown()


@pytest.mark.parametrize("family", ["olmo-hybrid", "olmo3-window-shorter-than-the-text"])
def test_grpo_on_hybrid_and_sliding_window_models(tmp_path, family):
    """The whole loop on an OLMo-Hybrid model (gated-DeltaNet layers: recurrent state in the engine, chunked rule in the learner)
    and on OLMo-3 with a window shorter than prompt + response: the engine's sampling log-probs equal the learner's at every
    step (also after a weight sync), and the export loads as the same transformers class."""
    transformers = pytest.importorskip("transformers")
    from open_instruct_b200.config.schemas import ModelConfig
    from open_instruct_b200.data.tokenize import TokenizerConfig
    from open_instruct_b200.grpo_fast import main
    from open_instruct_b200.grpo_utils import GRPOExperimentConfig
    from open_instruct_b200.streaming import StreamingDataLoaderConfig, VLLMConfig

    tmp = str(tmp_path)
    tok = make_tokenizer(os.path.join(tmp, "tok"))
    common = dict(vocab_size=600, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                  max_position_embeddings=256, pad_token_id=0, eos_token_id=1)
    torch.manual_seed(0)
    if family == "olmo-hybrid":
        hf = transformers.OlmoHybridForCausalLM(transformers.OlmoHybridConfig(**common))
    else:
        hf = transformers.Olmo3ForCausalLM(transformers.Olmo3Config(sliding_window=16, **common))
    src = os.path.join(tmp, "hf")
    hf.save_pretrained(src)
    data = make_rlvr_jsonl(os.path.join(tmp, "rl.jsonl"), n=12)
    args = GRPOExperimentConfig(total_episodes=2 * 4 * 4, learning_rate=1e-3, beta=0.0, load_ref_policy=False, output_dir=os.path.join(tmp, "out"),
                                single_gpu_mode=True, ops="ref", seed=3, save_freq=-1, lr_scheduler_type="constant")
    streaming = StreamingDataLoaderConfig(max_prompt_token_length=64, response_length=12, pack_length=256, async_steps=1,
                                          num_samples_per_prompt_rollout=4, num_unique_prompts_rollout=4, dataset_mixer_list=[data, "1.0"],
                                          dataset_local_cache_dir=os.path.join(tmp, "cache"), filter_zero_std_samples=False, temperature=1.0)
    main(args, TokenizerConfig(tokenizer_name_or_path=tok, chat_template_name="tulu"), ModelConfig(model_name_or_path=src), streaming, VLLMConfig())
    lines = [json.loads(l) for l in open(os.path.join(args.output_dir, "metrics.jsonl"))]
    assert len(lines) == 2
    for l in lines:
        assert l["debug/vllm_vs_local_logprob_diff_mean"] < 1e-5
    assert type(transformers.AutoModelForCausalLM.from_pretrained(args.output_dir)) is type(hf)


def test_grpo_recipe_topology_four_learners_two_tensor_parallel_engines(tmp_path, monkeypatch):
    """The process layout of the 8-GPU recipe - 4 learner ranks, 2 engines of tensor-parallel size 2 (each rank its own process:
    a leader that drives and a follower that mirrors its command stream) - as 8 CPU processes over gloo.  The engine ranks start
    with random weights and take the learners' through the first weight sync (every rank receives the model and cuts out its
    shard when the leader's command reaches it; verified per shard by checksum), the tensor-parallel engines' sampling log-probs
    equal the learners', two training steps complete."""
    monkeypatch.setenv("B200_GRPO_INIT_BY_PUSH", "force")
    from open_instruct_b200.actors import ray_compat as ray
    from open_instruct_b200.config.schemas import ModelConfig
    from open_instruct_b200.data.tokenize import TokenizerConfig
    from open_instruct_b200.grpo_fast import main
    from open_instruct_b200.grpo_utils import GRPOExperimentConfig
    from open_instruct_b200.streaming import StreamingDataLoaderConfig, VLLMConfig

    tmp = str(tmp_path)
    tok = make_tokenizer(os.path.join(tmp, "tok"))
    data = make_rlvr_jsonl(os.path.join(tmp, "rl.jsonl"), n=16)
    args = GRPOExperimentConfig(total_episodes=2 * 8 * 4, learning_rate=1e-3, beta=0.0, load_ref_policy=False, output_dir=os.path.join(tmp, "out"),
                                num_learners_per_node=[4], ops="ref", seed=3, save_freq=-1, lr_scheduler_type="constant", verify_weight_sync=True)
    streaming = StreamingDataLoaderConfig(max_prompt_token_length=64, response_length=8, pack_length=128, async_steps=1,
                                          num_samples_per_prompt_rollout=4, num_unique_prompts_rollout=8, dataset_mixer_list=[data, "1.0"],
                                          dataset_local_cache_dir=os.path.join(tmp, "cache"), filter_zero_std_samples=False)
    try:
        out = main(args, TokenizerConfig(tokenizer_name_or_path=tok, chat_template_name="tulu"), ModelConfig(model_name_or_path="tiny"),
                   streaming, VLLMConfig(vllm_num_engines=2, vllm_tensor_parallel_size=2))
    finally:
        ray.shutdown()
    assert out["training_step"] == 2
    lines = [json.loads(l) for l in open(os.path.join(args.output_dir, "metrics.jsonl"))]
    assert len(lines) == 2 and lines[0]["debug/vllm_vs_local_logprob_diff_mean"] < 1e-4   # the engines sampled with the learners' weights
