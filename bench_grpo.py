"""GRPO step-time benchmark: learner processes + rollout-engine processes on one node, synthetic arithmetic prompts.

    python bench_grpo.py --learners 2 --engines 2 --steps 4 --model llama3.1-8b --prompts 64 --samples 8 --response_length 512

Runs ``open_instruct_b200.grpo_fast.main`` in its multi-process topology (one process per GPU: ``--learners`` learner
ranks with the sharded optimizer, ``--engines`` rollout engines, a full weight sync after every step) and prints one JSON
line: median seconds per training step after the first (warm-up) step, time inside the learner step, weight-sync time,
time the trainer waited for rollouts, and generated tokens per step.  Step 1 includes cold starts and is reported apart.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import tempfile


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--learners", type=int, default=1)
    ap.add_argument("--engines", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--model", default="llama3.1-8b")
    ap.add_argument("--prompts", type=int, default=64)
    ap.add_argument("--samples", type=int, default=8)
    ap.add_argument("--response_length", type=int, default=512)
    ap.add_argument("--pack_length", type=int, default=4096)
    ap.add_argument("--async_steps", type=int, default=1)
    ap.add_argument("--single_gpu_mode", action="store_true")
    ap.add_argument("--ops", default="fused")
    ap.add_argument("--engine_tp", type=int, default=1, help="tensor-parallel size of every rollout engine (one process and GPU per rank)")
    ap.add_argument("--warmup", type=int, default=1, help="steps left out of the medians (step 1 includes every cold start)")
    a = ap.parse_args(argv)

    from open_instruct_b200.actors import ray_compat as ray
    from open_instruct_b200.config.schemas import ModelConfig
    from open_instruct_b200.data.synthetic import arithmetic_rlvr_jsonl, make_byte_tokenizer
    from open_instruct_b200.data.tokenize import TokenizerConfig
    from open_instruct_b200.grpo_fast import main as grpo_main
    from open_instruct_b200.grpo_utils import GRPOExperimentConfig
    from open_instruct_b200.streaming import StreamingDataLoaderConfig, VLLMConfig

    tmp = tempfile.mkdtemp(prefix="grpo_bench_")
    tok = make_byte_tokenizer(os.path.join(tmp, "tok"))
    data = arithmetic_rlvr_jsonl(os.path.join(tmp, "rl.jsonl"), n=a.prompts * (a.steps + a.async_steps + 2), seed=0)
    per_step = a.prompts * a.samples
    args = GRPOExperimentConfig(total_episodes=a.steps * per_step, learning_rate=1e-6, beta=0.0, load_ref_policy=False, clip_lower=0.2, clip_higher=0.2,
                                output_dir=os.path.join(tmp, "out"), num_learners_per_node=[a.learners], single_gpu_mode=a.single_gpu_mode,
                                ops=a.ops, seed=1, save_freq=-1, save_final_model=False, lr_scheduler_type="constant")
    streaming = StreamingDataLoaderConfig(max_prompt_token_length=128, response_length=a.response_length, pack_length=a.pack_length,
                                          async_steps=a.async_steps, num_samples_per_prompt_rollout=a.samples, num_unique_prompts_rollout=a.prompts,
                                          temperature=1.0, dataset_mixer_list=[data, "1.0"], dataset_local_cache_dir=os.path.join(tmp, "cache"),
                                          filter_zero_std_samples=False)
    try:
        grpo_main(args, TokenizerConfig(tokenizer_name_or_path=tok, chat_template_name="tulu"), ModelConfig(model_name_or_path=a.model), streaming,
                  VLLMConfig(vllm_num_engines=a.engines, vllm_gpu_memory_utilization=0.85, vllm_tensor_parallel_size=a.engine_tp))
    finally:
        ray.shutdown()
    lines = [json.loads(line) for line in open(os.path.join(args.output_dir, "metrics.jsonl"))]
    steady = lines[a.warmup:] or lines
    med = lambda k: statistics.median(float(x.get(k, 0.0)) for x in steady)
    out = {"metric": "grpo_step_seconds", "value": med("time/total"), "unit": "s", "higher_is_better": False, "n_gpus": 1 if a.single_gpu_mode else a.learners + a.engines * a.engine_tp,
           "steps": len(steady), "warmup": a.warmup, "scaling": "strong", "first_step_s": float(lines[0].get("time/total", 0.0)), "learner_step_s": med("time/training"),
           "weight_sync_s": med("time/weight_sync"), "waiting_for_rollouts_s": med("time/trainer_waiting_for_data"),
           "response_tokens_per_step": med("val/total_response_tokens"), "mean_response_length": med("val/sequence_lengths"),
           "dtype": "bf16", "data": "synthetic arithmetic prompts, random-init weights",
           "config": {"model": a.model, "learners": a.learners, "engines": a.engines, "engine_tp": a.engine_tp, "prompts_per_step": a.prompts,
                      "samples_per_prompt": a.samples, "max_response": a.response_length, "async_steps": a.async_steps,
                      "weight_sync": "every step, multi-destination push kernel through CUDA-IPC mappings"}}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
