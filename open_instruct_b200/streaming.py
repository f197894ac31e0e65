"""GRPO data path: prompts -> rollout results -> advantages -> packed, per-rank micro-batches.

Follows the reference's streaming design (``open_instruct/data_loader.py:393-1647``):
``StreamingDataLoaderConfig`` / ``VLLMConfig`` flags; a data-preparation worker that keeps
``async_steps`` batches of prompts in flight, replenishes one prompt for every consumed result, drops
results older than ``async_steps`` policy versions, filters zero-variance groups, computes group
advantages (``centered`` = score - group mean, ``standard`` = additionally / (std + 1e-8)), packs with
``pack_sequences(min_num_batches = dp_world)``, scatters advantages into the packed layout and splits
the rows contiguously across data-parallel ranks; learners pull ``get_data(rank, step)``.

The worker runs as a thread in single-process mode and inside an actor otherwise; the queues may be
``ray_compat.Queue`` (cross-process) or any object with ``put/get``.
"""

from __future__ import annotations

import json
import logging
import os
import threading
import time
from dataclasses import dataclass, field
from typing import Literal

import numpy as np
import torch

from .data_types import CollatedBatchData, GenerationResult, PromptRequest, SamplingConfig, ShutdownSentinel
from .rl_utils import pack_sequences

logger = logging.getLogger(__name__)


@dataclass
class VLLMConfig:
    """Rollout-engine placement (names kept from the reference so recipes carry over)."""

    vllm_num_engines: int = 1
    vllm_tensor_parallel_size: int = 1
    vllm_enforce_eager: bool = False
    vllm_attention_backend: str | None = None
    vllm_sync_backend: str = "nccl"
    vllm_gpu_memory_utilization: float = 0.9
    vllm_enable_prefix_caching: bool = False
    vllm_top_p: float = 1.0


@dataclass
class StreamingDataLoaderConfig:
    max_prompt_token_length: int = 256
    response_length: int = 256
    pack_length: int = 512
    async_steps: int = 8
    num_samples_per_prompt_rollout: int = 4
    num_unique_prompts_rollout: int = 16
    active_sampling: bool = False
    filter_zero_std_samples: bool = True
    no_resampling_pass_rate: float | None = None
    advantage_normalization_type: str = "centered"
    mask_truncated_completions: bool = False
    mask_tool_use: bool = True
    dataset_mixer_list: list[str] = field(default_factory=lambda: ["ai2-adapt-dev/rlvr_gsm8k_zs", "1.0"])
    dataset_mixer_eval_list: list[str] = field(default_factory=list)
    dataset_mixer_list_splits: list[str] = field(default_factory=lambda: ["train"])
    dataset_mixer_eval_list_splits: list[str] = field(default_factory=lambda: ["test"])
    dataset_transform_fn: list[str] = field(default_factory=lambda: ["rlvr_tokenize_v1", "rlvr_max_length_filter_v1"])
    dataset_cache_mode: Literal["hf", "local"] = "local"
    dataset_local_cache_dir: str = "local_dataset_cache"
    dataset_config_hash: str | None = None
    dataset_config_eval_hash: str | None = None
    dataset_skip_cache: bool = False
    system_prompt_override_file: str | None = None
    temperature: float = 1.0
    stop_strings: list[str] | None = None
    inflight_updates: bool = True
    eval_response_length: int | None = None
    additive_format_reward: bool = False
    apply_r1_style_format_reward: bool = False
    r1_style_format_reward: float = 1.0
    apply_verifiable_reward: bool = True
    verification_reward: float = 10.0
    remap_verifier: str | None = None
    reward_aggregator: Literal["last", "sum"] = "last"
    llm_judge_model: str = "gpt-4o-mini"
    llm_judge_max_tokens: int = 2048
    llm_judge_max_context_length: int = 8192
    llm_judge_temperature: float = 1.0
    llm_judge_timeout: int = 60
    code_api_url: str = "http://127.0.0.1:1234/test_program"
    code_max_execution_time: float = 1.0
    code_pass_rate_reward_threshold: float = 0.0
    code_apply_perf_penalty: bool = False
    max_length_verifier_max_length: int = 32768
    non_stop_penalty: bool = False
    non_stop_penalty_value: float = 0.0
    apply_evolving_rubric_reward: bool = False
    max_active_rubrics: int = 5
    cache_evolving_rubric_data_dir: str | None = None
    save_traces: bool = False
    rollouts_save_path: str = "rollouts/"
    max_possible_score: float = 1.0

    def __post_init__(self):
        if self.pack_length < self.max_prompt_token_length + self.response_length:
            raise ValueError("pack_length must be at least max_prompt_token_length + response_length")
        if self.num_samples_per_prompt_rollout < 1 or self.num_unique_prompts_rollout < 1:
            raise ValueError("rollout counts must be positive")
        if self.num_samples_per_prompt_rollout == 1 and self.filter_zero_std_samples:
            logger.warning("one sample per prompt: every group has zero reward variance; disabling filter_zero_std_samples")
            self.filter_zero_std_samples = False
        if self.advantage_normalization_type not in ("centered", "standard"):
            raise ValueError("advantage_normalization_type must be 'centered' or 'standard'")
        if self.async_steps < 1:
            raise ValueError("async_steps must be >= 1")
        if self.save_traces and not self.rollouts_save_path:
            raise ValueError("`rollouts_save_path` must be provided when `save_traces` is True.")
        if self.active_sampling and not self.filter_zero_std_samples:
            raise ValueError("active_sampling only makes sense with filter_zero_std_samples")
        if self.no_resampling_pass_rate is not None and not (0 < self.no_resampling_pass_rate <= 1):
            raise ValueError("no_resampling_pass_rate must lie in (0, 1]")
        if self.eval_response_length is None:
            self.eval_response_length = self.response_length


def compute_advantages(scores: np.ndarray, k: int, kind: str = "centered") -> np.ndarray:
    """Group-relative advantages for ``scores`` laid out as consecutive groups of ``k`` samples."""
    per_prompt = scores.reshape(-1, k)
    adv = per_prompt - per_prompt.mean(axis=-1, keepdims=True)
    if kind == "standard":
        adv = adv / (per_prompt.std(axis=-1, keepdims=True) + 1e-8)
    return adv.reshape(-1)


def maybe_mask_truncated_completions(masks: list[list[int]], finish_reasons: list[str], enabled: bool) -> list[list[int]]:
    """Responses that ran into the length limit contribute no loss when ``enabled``."""
    if not enabled:
        return masks
    return [m if fr == "stop" else [0] * len(m) for m, fr in zip(masks, finish_reasons)]


def prepare_collated_data_for_workers(packed, dp_world: int, per_device_train_batch_size: int, pad_token_id: int,
                                      seed: int | None = None, pin: bool = False) -> list[CollatedBatchData]:
    """Split packed rows contiguously over ranks (equal counts, leftovers dropped), shuffle inside a
    rank, group ``per_device_train_batch_size`` rows per micro-batch (rows are concatenated into one
    longer packed row with merged ``cu_seqlens`` - no padding)."""
    n = len(packed.query_responses)
    per_rank = n // dp_world
    if per_rank == 0:
        raise ValueError(f"{n} packed rows cannot feed {dp_world} ranks")
    rng = np.random.default_rng(seed)
    out = []
    for r in range(dp_world):
        idx = np.arange(r * per_rank, (r + 1) * per_rank)
        rng.shuffle(idx)
        fields = {k: [] for k in ("query_responses", "attention_masks", "position_ids", "advantages", "response_masks", "vllm_logprobs", "cu_seqlens")}
        for s in range(0, per_rank, per_device_train_batch_size):
            rows = idx[s : s + per_device_train_batch_size]
            cat = lambda lst: torch.cat([lst[i] for i in rows])
            fields["query_responses"].append(cat(packed.query_responses))
            fields["position_ids"].append(cat(packed.position_ids))
            fields["advantages"].append(cat(packed.advantages))
            fields["response_masks"].append(cat(packed.response_masks))
            fields["vllm_logprobs"].append(cat(packed.vllm_logprobs))
            off, docs, cus = 0, 0, [torch.zeros(1, dtype=torch.int32)]
            ams = []
            for i in rows:
                cu = packed.cu_seqlens[i]
                cus.append(cu[1:] + off)
                ams.append(packed.attention_masks[i] + docs)
                off += int(cu[-1])
                docs += cu.numel() - 1
            fields["cu_seqlens"].append(torch.cat(cus).to(torch.int32))
            fields["attention_masks"].append(torch.cat(ams))
        batch = CollatedBatchData(**fields)
        out.append(batch.pin_memory() if pin else batch)
    return out


# ---------------------------------------------------------------------------------- data preparation
class PromptIterator:
    """Endless, seeded, epoch-reshuffled stream over the prompt dataset with resumable state."""

    def __init__(self, dataset, seed: int):
        self.dataset, self.seed = dataset, seed
        self.epoch, self.pos = 0, 0
        self._order = self._perm()
        self.excluded: set[int] = set()

    def _perm(self):
        return torch.randperm(len(self.dataset), generator=torch.Generator().manual_seed(self.seed + self.epoch)).tolist()

    def __next__(self):
        for _ in range(2 * len(self.dataset) + 2):
            if self.pos >= len(self._order):
                self.epoch += 1
                self.pos = 0
                self._order = self._perm()
            i = self._order[self.pos]
            self.pos += 1
            row = self.dataset[i]
            if int(row.get("index", i)) in self.excluded:
                continue
            return row, self.epoch
        raise RuntimeError("every prompt is excluded")

    def exclude(self, index: int):
        self.excluded.add(int(index))

    def state_dict(self):
        return {"epoch": self.epoch, "pos": self.pos, "excluded": sorted(self.excluded)}

    def load_state_dict(self, sd):
        self.epoch, self.pos = sd["epoch"], sd["pos"]
        self.excluded = set(sd.get("excluded", []))
        self._order = self._perm()


ROLLOUT_SHARD_SIZE = 10000   # samples per JSONL shard of saved rollouts


def _at(seq, i):
    """``seq[i]`` when there is such an entry (made JSON-friendly), else None."""
    try:
        v = seq[i]
    except (TypeError, IndexError, KeyError):
        return None
    return v if isinstance(v, (str, int, float, bool, list, dict, type(None))) else str(v)


def save_rollout_metadata(save_path: str, run_name: str, model_name: str | None) -> None:
    """``<run>_metadata.jsonl``: which run, model, code revision and when (``open_instruct/rl_utils.py:46-67``)."""
    import datetime
    import subprocess

    try:
        commit = subprocess.run(["git", "rev-parse", "HEAD"], capture_output=True, text=True, timeout=5,
                                cwd=os.path.dirname(os.path.abspath(__file__))).stdout.strip() or "unknown"
    except Exception:  # noqa: BLE001
        commit = "unknown"
    os.makedirs(save_path, exist_ok=True)
    with open(os.path.join(save_path, f"{run_name}_metadata.jsonl"), "w") as fh:
        fh.write(json.dumps({"run_name": run_name, "git_commit": commit, "model_name": model_name or "unknown",
                             "timestamp": datetime.datetime.now(datetime.timezone.utc).isoformat()}) + "\n")


def save_rollouts(save_path: str, run_name: str, shard: int, records: list[dict]) -> None:
    """Append ``records`` to ``<run>_rollouts_<shard>.jsonl`` (``open_instruct/rl_utils.py:88-128``)."""
    os.makedirs(save_path, exist_ok=True)
    with open(os.path.join(save_path, f"{run_name}_rollouts_{shard:06d}.jsonl"), "a") as fh:
        for r in records:
            fh.write(json.dumps(r) + "\n")


class DataPreparation:
    """Producer of per-step training data (the role of ``DataPreparationActor``, ``data_loader.py:1292-1647``).

    ``prompt_queue``: where ``PromptRequest``s go (engines consume); ``results_queue``: where engines put
    ``GenerationResult``s with ``reward_scores`` already filled.  ``get_data(rank, step)`` blocks until
    the batch of ``step`` is ready.
    """

    def __init__(self, dataset, config: StreamingDataLoaderConfig, prompt_queue, results_queue, tokenizer, dp_world: int,
                 per_device_train_batch_size: int, seed: int, num_training_steps: int, eval_queue=None, top_p: float = 1.0,
                 rubric_judge=None, run_name: str = "run", model_name: str | None = None):
        self.cfg, self.tok = config, tokenizer
        # ``save_traces``: every rollout of every step goes to JSONL shards under ``rollouts_save_path``
        # (``open_instruct/rl_utils.py:46-159``), written by a background thread so that batch building does not wait for the disk
        self.run_name, self.model_name = run_name, model_name
        self._trace_samples, self._trace_pool = 0, None
        if config.save_traces:
            from concurrent.futures import ThreadPoolExecutor

            self._trace_pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="rollout-traces")
            save_rollout_metadata(config.rollouts_save_path, run_name, model_name)
        # evolving rubrics (``open_instruct/data_loader.py:1366-1370, 1462-1470``): after every step the judge proposes new
        # rubric items from the step's answers; prompts queued afterwards carry the updated rubric set as their ground truth
        self.rubric_manager = None
        self.ground_truth_overrides: dict[int, object] = {}
        if config.apply_evolving_rubric_reward:
            from .rubrics import RubricManager

            if rubric_judge is None:
                from .ground_truth_utils import LMJudgeVerifier, LMJudgeVerifierConfig

                judge = LMJudgeVerifier("quality", LMJudgeVerifierConfig(llm_judge_model=config.llm_judge_model, llm_judge_max_tokens=config.llm_judge_max_tokens,
                                                                         llm_judge_temperature=config.llm_judge_temperature,
                                                                         llm_judge_timeout=config.llm_judge_timeout,
                                                                         llm_judge_base_url=os.environ.get("LLM_JUDGE_BASE_URL")))
                rubric_judge = judge._ask
            self.rubric_manager = RubricManager(rubric_judge, max_active_rubrics=config.max_active_rubrics,
                                                cache_dir=config.cache_evolving_rubric_data_dir)
        self.prompt_q, self.results_q, self.eval_q = prompt_queue, results_queue, eval_queue
        self.dp_world, self.pdbs, self.seed = dp_world, per_device_train_batch_size, seed
        self.num_steps = num_training_steps
        self.prompts = PromptIterator(dataset, seed)
        self.prepared: dict[int, list[CollatedBatchData]] = {}
        self.metrics: dict[int, dict] = {}
        self.lock = threading.Condition()
        self.trainer_step = 0      # last step the learners asked for
        self.model_step = 0        # policy version prompts are tagged with
        self.stop = threading.Event()
        self.error: BaseException | None = None
        self.thread: threading.Thread | None = None
        self.pad = tokenizer.pad_token_id if tokenizer is not None and tokenizer.pad_token_id is not None else 0
        self.top_p = top_p
        self.total_prompts = 0
        self.next_step = 1

    # ------------------------------------------------------------------ prompts
    def _sampling(self) -> SamplingConfig:
        c = self.cfg
        return SamplingConfig(temperature=c.temperature, top_p=self.top_p, max_tokens=c.response_length,
                              n=c.num_samples_per_prompt_rollout, stop=c.stop_strings, logprobs=1)

    def add_prompt(self) -> None:
        row, epoch = next(self.prompts)
        index = int(row.get("index", 0))
        req = PromptRequest(prompt=list(row["input_ids_prompt"]), generation_config=self._sampling(), index=index,
                            prompt_id=f"{epoch}_{row.get('index', 0)}", raw_query=row.get("prompt"),
                            ground_truth=self.ground_truth_overrides.get(index, row.get("ground_truth")),
                            dataset=row.get("dataset"), epoch_number=epoch, training_step=self.model_step)
        self.prompt_q.put(req)
        self.total_prompts += 1

    # ------------------------------------------------------------------ accumulation
    def accumulate(self) -> tuple[list[GenerationResult], dict]:
        """Collect ``num_unique_prompts_rollout`` usable groups: stale results (older than
        ``async_steps`` policy versions) and zero-variance groups are dropped; every consumed result
        is replaced by a fresh prompt; with ``active_sampling`` keep pulling until the batch is full."""
        c = self.cfg
        want = c.num_unique_prompts_rollout
        kept: list[GenerationResult] = []
        stats = {"stale": 0, "zero_std": 0, "solved": 0, "pulled": 0}
        pulled_target = want
        while len(kept) < want and not self.stop.is_set():
            if stats["pulled"] >= pulled_target and not c.active_sampling:
                break
            try:
                res = self.results_q.get(timeout=0.2)
            except Exception:  # noqa: BLE001 - queue.Empty of either queue flavour
                continue
            if isinstance(res, ShutdownSentinel):
                self.stop.set()
                break
            stats["pulled"] += 1
            self.add_prompt()  # keep the number of prompts in flight constant
            if res.model_step is not None and self.trainer_step - res.model_step > c.async_steps:
                stats["stale"] += 1
                pulled_target += 1  # a stale result does not count against the batch
                continue
            scores = np.asarray(res.reward_scores, dtype=np.float64)
            if c.filter_zero_std_samples and scores.std() == 0:
                stats["zero_std"] += 1
                if c.no_resampling_pass_rate is not None and scores.mean() >= c.no_resampling_pass_rate * c.max_possible_score and res.index is not None:
                    self.prompts.exclude(res.index)
                    stats["solved"] += 1
                continue
            kept.append(res)
        return kept, stats

    def build_step(self, step: int) -> bool:
        c = self.cfg
        t0 = time.perf_counter()
        results, stats = self.accumulate()
        if self.stop.is_set():
            return False
        if not results:
            logger.warning("step %d: every group was filtered out; resampling without advancing", step)
            return self.build_step(step)
        k = c.num_samples_per_prompt_rollout
        queries, responses, masks, logps, scores, finish = [], [], [], [], [], []
        for r in results:
            for j in range(len(r.responses)):
                queries.append(list(r.queries[j]) if r.queries else [])
                responses.append(list(r.responses[j]))
                masks.append(list(r.masks[j]))
                logps.append(list(r.logprobs[j]))
                finish.append(r.finish_reasons[j])
            scores += list(r.reward_scores)
        scores_np = np.asarray(scores, dtype=np.float64)
        adv = compute_advantages(scores_np, k, c.advantage_normalization_type)
        if self._trace_pool is not None:
            owner = [(pi, r) for pi, r in enumerate(results) for _ in r.responses]
            records = [{"step": step, "sample_idx": i, "prompt_idx": owner[i][0], "prompt_tokens": queries[i], "response_tokens": responses[i],
                        "reward": float(scores_np[i]), "advantage": float(adv[i]), "finish_reason": finish[i], "logprobs": logps[i],
                        "dataset": _at([owner[i][1].dataset], 0), "ground_truth": _at([owner[i][1].ground_truth], 0)}
                       for i in range(len(responses))]
            shard = self._trace_samples // ROLLOUT_SHARD_SIZE
            self._trace_samples += len(records)
            self._trace_pool.submit(save_rollouts, c.rollouts_save_path, self.run_name, shard, records)
        masks = maybe_mask_truncated_completions(masks, finish, c.mask_truncated_completions)
        packed = pack_sequences(queries, responses, masks, c.pack_length, self.pad, logps, min_num_batches=self.dp_world,
                                mask_tool_use=c.mask_tool_use)
        lookup = torch.cat([torch.zeros(1), torch.tensor(adv, dtype=torch.float32)])
        packed.advantages = [lookup[m.long()] for m in packed.response_masks]
        per_rank = prepare_collated_data_for_workers(packed, self.dp_world, self.pdbs, self.pad, seed=self.seed + step,
                                                     pin=torch.cuda.is_available())
        lens = np.array([len(x) for x in responses])
        stop_rate = float(np.mean([f == "stop" for f in finish]))
        gen_times = [r.token_statistics.generation_time for r in results if r.token_statistics]
        m = {"scores": float(scores_np.mean()), "val/sequence_lengths": float(lens.mean()), "val/sequence_lengths_max": int(lens.max()),
             "val/sequence_lengths_min": int(lens.min()), "val/stop_rate": stop_rate, "val/advantages_abs_mean": float(np.abs(adv).mean()),
             "batch/filtered_zero_std": stats["zero_std"], "batch/stale_dropped": stats["stale"], "batch/prompts_solved": stats["solved"],
             "batch/num_groups": len(results), "batch/packed_rows": len(packed.query_responses),
             "time/getting_response": time.perf_counter() - t0, "time/group_generation_mean": float(np.mean(gen_times)) if gen_times else 0.0,
             "val/total_response_tokens": int(lens.sum()),
             "val/total_prompt_tokens": int(sum(len(q) for q in queries[::k]))}
        for r in results:
            for kk, v in (r.reward_metrics or {}).items():
                m.setdefault(kk, []).append(v)
        m = {kk: (float(np.mean(v)) if isinstance(v, list) else v) for kk, v in m.items()}
        if self.rubric_manager is not None:
            m.update(self._evolve_rubrics(results, responses, step))
        with self.lock:
            self.prepared[step] = per_rank
            self.metrics[step] = m
            self.lock.notify_all()
        return True

    def _evolve_rubrics(self, results: list[GenerationResult], responses: list[list[int]], step: int) -> dict:
        """One evolving-rubric step over this batch's groups; rubric ground truths are JSON specs (``{"query", "rubrics"}``)."""
        import json

        k = self.cfg.num_samples_per_prompt_rollout
        decoded, gts, idx, pos = [], [], [], 0
        for r in results:
            n = len(r.responses)
            texts = r.decoded_responses or ([self.tok.decode(x, skip_special_tokens=True) for x in responses[pos:pos + n]] if self.tok is not None else [""] * n)
            pos += n
            gt = r.ground_truth[0] if isinstance(r.ground_truth, list) and r.ground_truth else r.ground_truth
            if isinstance(gt, str):
                try:
                    gt = json.loads(gt)
                except json.JSONDecodeError:
                    gt = None
            if not isinstance(gt, dict) or n != k:
                continue  # not a rubric-scored prompt (mixed datasets), or an incomplete group
            decoded += list(texts)
            gts += [gt] * n
            idx += [int(r.index or 0)] * n
        if not decoded:
            return {}
        metrics, overrides = self.rubric_manager.step(decoded, gts, idx, k, training_step=step)
        self.ground_truth_overrides.update({i: json.dumps(o) for i, o in overrides.items()})
        return metrics

    # ------------------------------------------------------------------ loop / API
    def _run(self):
        try:
            for _ in range(self.cfg.async_steps * self.cfg.num_unique_prompts_rollout):
                self.add_prompt()
            while self.next_step <= self.num_steps and not self.stop.is_set():
                with self.lock:  # never run more than async_steps ahead of the trainer
                    while self.next_step - self.trainer_step > self.cfg.async_steps and not self.stop.is_set():
                        self.lock.wait(timeout=0.2)
                if not self.build_step(self.next_step):
                    break
                self.next_step += 1
        except BaseException as e:  # noqa: BLE001
            self.error = e
            with self.lock:
                self.lock.notify_all()

    def start(self):
        self.thread = threading.Thread(target=self._run, name="data-prep", daemon=True)
        self.thread.start()

    def get_data(self, rank: int, step: int, timeout: float = 3600.0):
        deadline = time.time() + timeout
        with self.lock:
            self.trainer_step = max(self.trainer_step, step - 1)
            self.lock.notify_all()
            while step not in self.prepared:
                if self.error is not None:
                    raise RuntimeError(f"data preparation failed: {self.error!r}")
                if time.time() > deadline:
                    raise TimeoutError(f"no data for step {step}")
                self.lock.wait(timeout=0.2)
            data = self.prepared[step][rank]
            metrics = self.metrics[step]
            # a step can be dropped once every rank fetched it; keep a small window instead of counting
            for old in [s for s in self.prepared if s < step - 2]:
                self.prepared.pop(old, None)
                self.metrics.pop(old, None)
        return data, metrics

    def set_model_step(self, step: int):
        self.model_step = step

    def get_state(self) -> dict:
        sd = {"prompts": self.prompts.state_dict(), "next_step": self.next_step, "total_prompts": self.total_prompts}
        if self.rubric_manager is not None:
            sd["rubric_buffer"] = self.rubric_manager.buffer.state_dict()
            sd["ground_truth_overrides"] = dict(self.ground_truth_overrides)
        return sd

    def set_state(self, sd: dict):
        self.prompts.load_state_dict(sd["prompts"])
        self.next_step = sd.get("next_step", 1)
        self.total_prompts = sd.get("total_prompts", 0)
        if self.rubric_manager is not None and "rubric_buffer" in sd:
            self.rubric_manager.buffer.load_state_dict(sd["rubric_buffer"])
            self.ground_truth_overrides = {int(k): v for k, v in sd.get("ground_truth_overrides", {}).items()}

    def shutdown(self):
        self.stop.set()
        with self.lock:
            self.lock.notify_all()
        if self.thread is not None:
            self.thread.join(timeout=5)
        if self._trace_pool is not None:
            self._trace_pool.shutdown(wait=True)   # rollouts still queued for the disk
            self._trace_pool = None
