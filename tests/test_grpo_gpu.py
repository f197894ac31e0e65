"""GRPO on GPUs: single-GPU mode through the fused kernels; learner + engine in separate processes
with the weight push through a CUDA-IPC mapping (2 GPUs)."""

import json
import os

import pytest
import torch

from helpers import make_rlvr_jsonl, make_tokenizer

pytestmark = pytest.mark.gpu


def _run(tmp, single, tp=1, model="tiny128", verify=False, shard=None):
    from open_instruct_b200.actors import ray_compat as ray
    from open_instruct_b200.config.schemas import ModelConfig
    from open_instruct_b200.data.tokenize import TokenizerConfig
    from open_instruct_b200.grpo_fast import main
    from open_instruct_b200.grpo_utils import GRPOExperimentConfig
    from open_instruct_b200.streaming import StreamingDataLoaderConfig, VLLMConfig

    tok = make_tokenizer(os.path.join(tmp, "tok"))
    data = make_rlvr_jsonl(os.path.join(tmp, "rl.jsonl"), n=12)
    args = GRPOExperimentConfig(total_episodes=3 * 4 * 4, learning_rate=1e-4, beta=0.0, load_ref_policy=False, output_dir=os.path.join(tmp, "out"),
                                single_gpu_mode=single, ops="fused", seed=3, save_freq=-1, lr_scheduler_type="constant", verify_weight_sync=verify, shard_parameters=shard)
    streaming = StreamingDataLoaderConfig(max_prompt_token_length=64, response_length=16, pack_length=256, async_steps=1,
                                          num_samples_per_prompt_rollout=4, num_unique_prompts_rollout=4, dataset_mixer_list=[data, "1.0"],
                                          dataset_local_cache_dir=os.path.join(tmp, "cache"), filter_zero_std_samples=False)
    try:
        out = main(args, TokenizerConfig(tokenizer_name_or_path=tok, chat_template_name="tulu"), ModelConfig(model_name_or_path=model),
                   streaming, VLLMConfig(vllm_gpu_memory_utilization=0.3, vllm_tensor_parallel_size=tp))
    finally:
        ray.shutdown()
    lines = [json.loads(l) for l in open(os.path.join(args.output_dir, "metrics.jsonl"))]
    assert out["training_step"] == 3 and len(lines) == 3
    # the engine and the learner run the same weights through the same kernels: their log-probs agree
    assert lines[0]["debug/vllm_vs_local_logprob_diff_mean"] < 0.05
    if verify:  # the engines compute with exactly the learner's weights after every sync
        assert all(l["debug/weight_sync_checksum_diff"] == 0.0 for l in lines)
    else:
        assert lines[-1]["debug/vllm_vs_local_logprob_diff_mean"] < 0.05  # still true after two weight syncs
    return lines


def test_grpo_single_gpu_mode(tmp_path):
    _run(str(tmp_path), single=True)


def test_grpo_single_gpu_mode_sharded_parameters(tmp_path):
    """The learner keeps parameter slices only (one rank: the gather is a copy); the engine gets the gathered weights."""
    _run(str(tmp_path), single=True, shard=True)


@pytest.mark.parametrize("shard", [None, True])
def test_grpo_learner_and_engine_processes_ipc_push(tmp_path, shard):
    """``shard``: the learner pushes its parameter slices unit by unit straight from the shard buffer."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    lines = _run(str(tmp_path), single=False, verify=True, shard=shard)
    assert all(l["time/weight_sync"] < 30 for l in lines)


def test_grpo_tensor_parallel_engine(tmp_path):
    """One learner + one rollout engine split over two GPUs (three processes, three GPUs)."""
    if torch.cuda.device_count() < 3:
        pytest.skip("needs 3 GPUs")
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    lines = _run(str(tmp_path), single=False, tp=2, model="tiny128-tp", verify=True)
    assert all(l["time/weight_sync"] < 30 for l in lines)
