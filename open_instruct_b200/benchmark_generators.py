"""Rollout-engine benchmark: new tokens/s, MFU and MBU of generation, and the measured weight-sync time.

Protocol of ``open_instruct/benchmark_generators.py:351-546``: one warm-up batch, then ``num_batches - 1`` timed batches of
``num_unique_prompts_rollout`` prompts x ``num_samples_per_prompt_rollout`` samples with ``response_length`` new tokens each
(``min_tokens = response_length`` unless stop strings are given, so every batch does the same work); after every batch the
engine receives the weights again.  Where the reference assumes 1.0 s for that sync (``:303-304``), this benchmark runs the
real multi-destination push kernel from a learner-side buffer and reports its device time.  Results go to stdout as one JSON
line per batch plus a summary, and optionally to a CSV file.

    python -m open_instruct_b200.benchmark_generators --model llama3.1-8b --num_unique_prompts_rollout 32 \
        --num_samples_per_prompt_rollout 16 --response_length 512 --prompt_length 512 --num_batches 4
"""

from __future__ import annotations

import argparse
import collections
import csv
import json
import os
import time

import torch

from .data_types import SamplingConfig
from .models.spec import get_spec
from .utils.model_dims import ModelDims


def synthetic_prompts(n: int, length: int, vocab: int, seed: int) -> list[list[int]]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(10, vocab - 10, (n, length), generator=g).tolist()


def run_batch(engine, prompts, cfg: SamplingConfig) -> dict:
    dev = engine.device
    if dev.type == "cuda":
        torch.cuda.synchronize(dev)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
    t0 = time.perf_counter()
    results = engine.generate(prompts, cfg)
    if dev.type == "cuda":
        ev1.record()
        torch.cuda.synchronize(dev)
        seconds = ev0.elapsed_time(ev1) / 1e3
    else:
        seconds = time.perf_counter() - t0
    resp = [len(r) for res in results for r in res.responses]
    return {"generation_time": seconds, "num_new_tokens": sum(resp), "response_lengths": resp, "prompt_lengths": [len(p) for p in prompts],
            "finish_reasons": dict(collections.Counter(fr for res in results for fr in res.finish_reasons)),
            "tokens_per_second": sum(resp) / max(seconds, 1e-9)}


def measure_weight_sync(engine, learner_flat: torch.Tensor) -> float:
    from .parallel.weight_sync import push_slice

    dev = engine.device
    n = engine.model.layout.total
    if dev.type != "cuda":
        t0 = time.perf_counter()
        push_slice(learner_flat, [engine.model.flat.detach()], 0, n)
        return time.perf_counter() - t0
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    ev0.record()
    push_slice(learner_flat, [engine.model.flat.detach()], 0, n)
    ev1.record()
    torch.cuda.synchronize(dev)
    return ev0.elapsed_time(ev1) / 1e3


def run_vllm(a) -> dict:
    """The same batches through ``vllm.LLM.generate`` offline (TP 1, in-process engine core, random weights of the same
    architecture): the library the reference's rollout actors wrap (``open_instruct/vllm_utils.py:1188-1313``), measured
    on the same box as a bar for this package's engine.  None of this package's kernels run here."""
    import tempfile

    os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")
    os.environ.setdefault("VLLM_LOGGING_LEVEL", "WARNING")
    import vllm

    spec = get_spec(a.model)
    d = tempfile.mkdtemp(prefix="b200_vllm_cfg_")
    cfg = spec.to_hf_config()
    cfg.update({"max_position_embeddings": max(4096, a.prompt_length + a.response_length + 16), "rope_scaling": None,
                "bos_token_id": 1, "eos_token_id": 2, "pad_token_id": 0})
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    llm = vllm.LLM(model=d, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16", tensor_parallel_size=1,
                   gpu_memory_utilization=a.gpu_memory_utilization, max_model_len=a.prompt_length + a.response_length + 16,
                   seed=a.seed, enable_prefix_caching=True, max_num_seqs=a.max_running, logprobs_mode="processed_logprobs")
    sp = vllm.SamplingParams(n=a.num_samples_per_prompt_rollout, temperature=a.temperature, top_p=a.top_p, max_tokens=a.response_length,
                             min_tokens=a.response_length, ignore_eos=True, logprobs=0, detokenize=False, seed=a.seed)
    dims = ModelDims.from_spec(spec)
    results = []
    for b in range(a.num_batches):
        prompts = synthetic_prompts(a.num_unique_prompts_rollout, a.prompt_length, spec.vocab_size, a.seed + b)
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        t0 = time.perf_counter()
        outs = llm.generate([{"prompt_token_ids": p} for p in prompts], sp, use_tqdm=False)
        ev1.record()
        torch.cuda.synchronize()
        seconds = max(ev0.elapsed_time(ev1) / 1e3, time.perf_counter() - t0)
        resp = [len(c.token_ids) for o in outs for c in o.outputs]
        r = {"generation_time": seconds, "num_new_tokens": sum(resp), "tokens_per_second": sum(resp) / seconds, "weight_sync_time": 0.0,
             "finish_reasons": dict(collections.Counter(c.finish_reason for o in outs for c in o.outputs)), "batch": b, "warmup": b == 0}
        r.update(dims.calculate_actor_utilization([len(p) for p in prompts], resp, seconds, a.num_samples_per_prompt_rollout, 1, 1))
        print(json.dumps(r))
        if b > 0:
            results.append(r)
    summary = aggregate(results) if results else {}
    summary.update({"impl": f"vllm {vllm.__version__}", "model": a.model, "batch_size": a.num_unique_prompts_rollout,
                    "samples_per_prompt": a.num_samples_per_prompt_rollout, "response_length": a.response_length, "prompt_length": a.prompt_length})
    print(json.dumps({"summary": summary}))
    return summary


def aggregate(results: list[dict]) -> dict:
    t = sum(r["generation_time"] for r in results)
    n = sum(r["num_new_tokens"] for r in results)
    k = max(1, len(results))
    fr = collections.Counter()
    for r in results:
        fr.update(r["finish_reasons"])
    return {"avg_tokens_per_second": n / max(t, 1e-9), "avg_mfu": sum(r["mfu"] for r in results) / k, "avg_mbu": sum(r["mbu"] for r in results) / k,
            "avg_generation_time": t / k, "avg_weight_sync_time": sum(r["weight_sync_time"] for r in results) / k, "total_num_new_tokens": n,
            "total_generation_time": t, "finish_reasons": dict(fr)}


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny128")
    ap.add_argument("--num_unique_prompts_rollout", type=int, default=8)
    ap.add_argument("--num_samples_per_prompt_rollout", type=int, default=4)
    ap.add_argument("--prompt_length", type=int, default=128)
    ap.add_argument("--response_length", type=int, default=128)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top_p", type=float, default=1.0)
    ap.add_argument("--num_batches", type=int, default=4, help="including the warm-up batch")
    ap.add_argument("--gpu_memory_utilization", type=float, default=0.85)
    ap.add_argument("--max_running", type=int, default=256)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--csv", default="")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--impl", default="ours", choices=["ours", "vllm"],
                    help="vllm: the same batches through vllm.LLM.generate (library bar on the same box; not this package's engine)")
    a = ap.parse_args(argv)
    if a.impl == "vllm":
        return run_vllm(a)

    from .rollout.engine import RolloutEngine

    spec = get_spec(a.model)
    engine = RolloutEngine(spec, device=a.device, gpu_memory_utilization=a.gpu_memory_utilization, max_running=a.max_running,
                           max_model_len=a.prompt_length + a.response_length + 16, seed=a.seed, eos_token_ids=[])
    learner_flat = engine.model.flat.detach().clone()
    dims = ModelDims.from_spec(spec)
    cfg = SamplingConfig(temperature=a.temperature, top_p=a.top_p, max_tokens=a.response_length, min_tokens=a.response_length,
                         n=a.num_samples_per_prompt_rollout, seed=a.seed)
    results = []
    for b in range(a.num_batches):
        prompts = synthetic_prompts(a.num_unique_prompts_rollout, a.prompt_length, spec.vocab_size, a.seed + b)
        r = run_batch(engine, prompts, cfg)
        r["weight_sync_time"] = measure_weight_sync(engine, learner_flat)
        u = dims.calculate_actor_utilization(r["prompt_lengths"], r["response_lengths"], r["generation_time"],
                                             a.num_samples_per_prompt_rollout, 1, 1)
        r.update(u)
        r["batch"] = b
        r["warmup"] = b == 0
        print(json.dumps({k: v for k, v in r.items() if k not in ("response_lengths", "prompt_lengths")}))
        if b > 0:
            results.append(r)
    summary = aggregate(results) if results else {}
    summary.update({"model": a.model, "batch_size": a.num_unique_prompts_rollout, "samples_per_prompt": a.num_samples_per_prompt_rollout,
                    "response_length": a.response_length, "prompt_length": a.prompt_length, "kv_blocks": engine.num_blocks})
    st = engine.stats
    if st.get("decode_steps"):  # where a graph-replayed decode step's wall time goes, in ms per step
        k = 1e3 / st["decode_steps"]
        summary["decode_step_ms"] = {"host_pack": st["host_pack_s"] * k, "device_wait": st["device_wait_s"] * k, "host_accept": st["host_accept_s"] * k,
                                     "host_schedule": st["host_sched_s"] * 1e3 / max(1, st["steps"]), "steps": st["decode_steps"]}
    print(json.dumps({"summary": summary}))
    if a.csv:
        new = not os.path.exists(a.csv)
        with open(a.csv, "a", newline="") as f:
            w = csv.DictWriter(f, fieldnames=sorted(k for k in summary if k != "finish_reasons"))
            if new:
                w.writeheader()
            w.writerow({k: v for k, v in summary.items() if k != "finish_reasons"})
    return summary


if __name__ == "__main__":
    main()
