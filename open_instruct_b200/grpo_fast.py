"""RLVR / GRPO entry point (the ``grpo_fast`` API).

    python -m open_instruct_b200.grpo_fast config.yaml [--flag value ...]

Process topology follows the reference (``open_instruct/grpo_fast.py:1245-1432``, ``:1796-2052``): learner
workers (one per GPU, sharded optimizer among them), rollout-engine workers, one data-preparation
worker, an actor manager, three queues (prompts, results, eval results); the driver loop steps the
learners, triggers the weight sync and logs.  Differences: the engines are this package's
``RolloutEngine`` (called in process, no HTTP server); weights reach the engines by direct stores
into their parameter buffers (CUDA IPC mapping + one multi-destination copy kernel over NVLink, or
a plain copy when learner and engine share a process) instead of 291 NCCL broadcasts.

``--single_gpu_mode`` (or a machine without several GPUs) runs learner, engine and data
preparation as threads of one process on one device.

The learner step implements the reference semantics (``grpo_fast.py:586-765``): per packed micro-batch,
new log-probs at ``temperature``; old log-probs = detached new ones on the first pass (or precomputed
with several mini-batches, or the engine's); rho correction; DAPO / CISPO loss (+ beta * KL to the
reference policy when loaded); token-normalised over the accumulation group with the denominator
all-reduced over data-parallel ranks.
"""

from __future__ import annotations

import asyncio
import json
import logging
import math
import os
import contextlib
import threading
import time
from dataclasses import asdict

import numpy as np
import torch

from .ckpt.hf_io import load_hf_checkpoint, save_hf_checkpoint
from .ckpt.train_state import load_train_state, save_train_state
from .config.argparser import ArgumentParserPlus
from .config.schemas import ModelConfig
from .data.tokenize import TokenizerConfig
from .data_types import CollatedBatchData, GenerationResult, PromptRequest, ShutdownSentinel
from .ground_truth_utils import RewardConfig, build_all_verifiers
from .grpo_utils import (
    GRPOExperimentConfig,
    calculate_token_counts,
    compute_grpo_loss,
    compute_rho_correction,
    compute_vllm_local_debug_metrics,
    mask_logprobs,
    masked_mean,
    resolve_old_logprob,
)
from .learner import Learner, LearnerConfig
from .models import get_spec
from .parallel import dist as pdist
from .streaming import DataPreparation, StreamingDataLoaderConfig, VLLMConfig
from .utils.common import INVALID_LOGPROB, Tracker, set_seed, setup_logger
from .utils.model_dims import ModelDims

logger = setup_logger(__name__)
WEIGHT_SYNC_TIMEOUT_S = 120


# ======================================================================================= learner step
def _packed_batch(data: CollatedBatchData, i: int, device, pad_multiple: int = 1, pad_token_id: int = 0) -> dict:
    """Model inputs of packed micro-batch ``i``.  ``pad_multiple`` > 1 (sequence parallelism) appends one fully masked
    document so that the token count divides evenly over the ranks of the group."""
    qr = data.query_responses[i].to(device, non_blocking=True)
    pos = data.position_ids[i].to(device, non_blocking=True)
    cu = data.cu_seqlens[i].to(device, non_blocking=True)
    T = qr.numel()
    labels = torch.full_like(qr, -100)
    labels[:-1] = qr[1:]
    labels[cu[1:].long() - 1] = -100  # the last token of a document has no target
    extra = (-T) % pad_multiple
    if extra:
        qr = torch.cat([qr, qr.new_full((extra,), pad_token_id)])
        pos = torch.cat([pos, torch.arange(extra, device=device, dtype=pos.dtype)])
        labels = torch.cat([labels, labels.new_full((extra,), -100)])
        cu = torch.cat([cu, cu.new_tensor([T + extra])])
    return {"input_ids": qr, "position_ids": pos, "cu_seq_lens_q": cu, "labels_shifted": labels}


def _to_label_space(x: torch.Tensor, fill, total: int) -> torch.Tensor:
    """``y[t] = x[t + 1]``: a per-token quantity moved to the position that PREDICTS the token (where the model's
    log-prob of it lives), padded with ``fill`` up to ``total`` entries."""
    y = x.new_full((total,), fill)
    y[: x.numel() - 1] = x[1:]
    return y


def forward_for_logprobs(learner: Learner, batch: dict, temperature: float, want_entropy: bool = False):
    """Per-token log-prob of the NEXT token at ``temperature`` (position t scores token t+1), shifted so
    that entry t is the log-prob OF token t; invalid entries hold ``INVALID_LOGPROB``."""
    lp, ent = learner.token_logprobs(batch, temperature, want_entropy)
    valid = batch["labels_shifted"] >= 0
    lp = torch.where(valid, lp, torch.full_like(lp, INVALID_LOGPROB))
    out = torch.full_like(lp, INVALID_LOGPROB)
    out[1:] = lp[:-1]
    e = None
    if ent is not None:
        e = torch.zeros_like(ent)
        e[1:] = ent[:-1]
    return out, e


def grpo_train_step(learner: Learner, data: CollatedBatchData, args: GRPOExperimentConfig, ref_learner: Learner | None = None,
                    group=None) -> dict:
    """All epochs / mini-batches of one training step on this rank's packed micro-batches."""
    dev = learner.device
    n = len(data)
    if n == 0:
        return {}
    accumulation_steps = max(1, math.ceil(n / args.num_mini_batches - 0.5))
    usable = (n // accumulation_steps) * accumulation_steps
    # Sequence parallelism: every rank of a group sees the same packs and computes log-probs for its chunk of the positions.
    # The per-token quantities are therefore kept in LABEL space (entry t belongs to the token at t + 1, scored at position
    # t) instead of being shifted after the forward pass, which would need the neighbour's last entry; then each is cut to
    # this rank's chunk.  Response tokens never open a document, so no response entry is lost by the shift.
    sp = getattr(learner, "sp", 1)
    label_space = sp > 1 or getattr(args, "_force_label_space", False)
    if label_space and (args.rho_mask_sequence_level or args.rho_mask_tv_divergence):
        raise NotImplementedError("sequence-level rho masking needs whole sequences on one rank: not available with sequence parallelism")
    batches = [_packed_batch(data, i, dev, pad_multiple=sp) for i in range(usable)]

    def per_token(col, i, fill):
        t = col[i].to(dev)
        if not label_space:
            return t
        return learner.local_slice(_to_label_space(t, fill, batches[i]["input_ids"].numel()))

    def logprobs_of(lrn, i, want_entropy=False):
        if not label_space:
            return forward_for_logprobs(lrn, batches[i], args.temperature, want_entropy)
        lp, ent = lrn.token_logprobs(batches[i], args.temperature, want_entropy)
        valid = learner.local_slice(batches[i]["labels_shifted"] >= 0)
        return torch.where(valid, lp, torch.full_like(lp, INVALID_LOGPROB)), ent

    resp_masks = [per_token(data.response_masks, i, 0) for i in range(usable)]
    resp_bool = [m > 0 for m in resp_masks]
    advantages = [per_token(data.advantages, i, 0.0) for i in range(usable)]
    vllm_raw = [per_token(data.vllm_logprobs, i, float("nan")) for i in range(usable)]
    vllm_lp = [mask_logprobs(vllm_raw[i], resp_bool[i]) for i in range(usable)]
    ref_lp = [None] * usable
    if ref_learner is not None:
        with torch.no_grad():
            for i in range(usable):
                ref_lp[i], _ = logprobs_of(ref_learner, i)
    old_cache: list = [None] * usable
    if args.num_mini_batches > 1:
        with torch.no_grad():
            for i in range(usable):
                old_cache[i] = vllm_lp[i] if args.use_vllm_logprobs else logprobs_of(learner, i)[0]
    if args.loss_denominator == "token":
        denoms = calculate_token_counts(accumulation_steps, resp_bool, dev, group)
    else:
        denoms = {s: float(args.loss_denominator) for s in range(0, usable, accumulation_steps)}
    world = pdist.world_size(group)
    stats = {k: [] for k in ("pg", "kl", "loss", "clipfrac", "ratio", "entropy", "lpdiff")}
    rho_stats: dict[str, list] = {}
    grad_norms = []
    for epoch in range(args.num_epochs):
        for i in range(usable):
            new_lp, ent = logprobs_of(learner, i, args.record_entropy)
            mask = resp_bool[i]
            new_lp = torch.where(mask, new_lp, torch.full_like(new_lp, INVALID_LOGPROB))
            old = resolve_old_logprob(old_cache, i, epoch, args.num_mini_batches, args.use_vllm_logprobs, vllm_lp[i], new_lp)
            ratio = torch.exp(new_lp - old)
            rho = compute_rho_correction(old, vllm_lp[i], mask, advantages[i], args, segment_ids=resp_masks[i])
            pg, clipfrac, kl = compute_grpo_loss(new_lp, ratio, advantages[i], ref_lp[i], args, rho.weights)
            group_start = (i // accumulation_steps) * accumulation_steps
            denom = max(denoms[group_start], 1.0)
            # summed over the group's tokens on ALL ranks / global token count; the optimizer averages over
            # ranks, hence the factor world (same convention as the reference with DeepSpeed)
            loss = masked_mean(pg + args.beta * kl, mask, None, denom) * world
            learner.backward(loss, last=(i + 1) % accumulation_steps == 0)
            with torch.no_grad():
                stats["pg"].append(masked_mean(pg, mask))
                stats["kl"].append(masked_mean(kl, mask))
                stats["loss"].append(masked_mean(pg + args.beta * kl, mask))
                stats["clipfrac"].append(masked_mean(clipfrac, mask))
                stats["ratio"].append(masked_mean(ratio, mask))
                if ent is not None:
                    stats["entropy"].append(masked_mean(ent, mask))
                if epoch == 0:
                    stats["lpdiff"].append(compute_vllm_local_debug_metrics(new_lp.detach(), vllm_raw[i], mask))
                for k, v in rho.metrics.items():
                    rho_stats.setdefault(k, []).append(masked_mean(v, mask))
            if (i + 1) % accumulation_steps == 0:
                # the loss already carries 1/denominator and the factor world: undo only the rank average
                grad_norms.append(learner.optimizer_step(grad_scale=1.0 / world))
    mean = lambda xs: float(torch.stack(xs).mean()) if xs else 0.0
    out = {"loss/policy_avg": mean(stats["pg"]), "loss/kl_avg": mean(stats["kl"]), "loss/total_avg": mean(stats["loss"]),
           "policy/clipfrac_avg": mean(stats["clipfrac"]), "val/ratio": mean(stats["ratio"]),
           "val/ratio_var": float(torch.stack(stats["ratio"]).var()) if len(stats["ratio"]) > 1 else 0.0,
           "optim/grad_norm": mean([g.reshape(()) for g in grad_norms]), "lr": learner.lr(max(0, learner.global_step - 1)),
           "num_response_tokens": float(sum(int(m.sum()) for m in resp_bool))}
    if stats["entropy"]:
        out["policy/entropy_avg"] = mean(stats["entropy"])
    for k, v in rho_stats.items():
        out[k] = mean(v)
    if stats["lpdiff"]:
        for k in stats["lpdiff"][0]:
            out[k] = float(np.mean([d[k] for d in stats["lpdiff"]]))
    return out


# ======================================================================================= engine worker
class _TPLeader:
    """Rank 0 of a tensor-parallel engine: forwards every state-changing engine call to the other ranks before running it
    itself.  Calls are batched: ``add_request`` only records; ``step`` (or ``send``) broadcasts the batch."""

    def __init__(self, engine, group):
        self._e, self._g, self._cmds = engine, group, []

    def __getattr__(self, name):
        return getattr(self._e, name)

    def __setattr__(self, name, value):
        if name.startswith("_"):
            object.__setattr__(self, name, value)
        else:
            setattr(self._e, name, value)

    def add_request(self, prompt, sampling, **meta):
        self._cmds.append(("add", list(prompt), sampling))
        return self._e.add_request(prompt, sampling, **meta)

    def send(self, extra: list) -> None:
        import torch.distributed as dist

        batch, self._cmds = self._cmds + list(extra), []
        dist.broadcast_object_list([batch], src=0, group=self._g)

    def step(self):
        self.send([("step",)])
        return self._e.step()


class EngineWorker:
    """Rollout engine + its request loop (the role of ``LLMRayActor``, ``open_instruct/vllm_utils.py:553-843``).

    A background thread pulls ``PromptRequest``s while the engine has room, steps the engine, computes
    rewards for finished requests and pushes ``GenerationResult``s to the results queue (eval requests
    go to the eval queue)."""

    def __init__(self, spec, prompt_queue, results_queue, eval_queue, reward_config: RewardConfig | None, tokenizer=None,
                 device="cuda", ops: str = "auto", seed: int = 0, max_model_len: int = 8192, num_blocks: int | None = None,
                 gpu_memory_utilization: float = 0.85, flat: torch.Tensor | None = None, inflight_updates: bool = True,
                 max_running: int = 256, envs_config=None, tp_rank: int = 0, tp_size: int = 1, tp_addr: str = "127.0.0.1", tp_port: int = 0,
                 enable_prefix_caching: bool = False):
        from .rollout.engine import RolloutEngine

        self.tp_rank, self.tp_size = tp_rank, tp_size
        self._prefix_caching = bool(enable_prefix_caching)
        if isinstance(tokenizer, TokenizerConfig):  # built in the worker's own process
            tokenizer = tokenizer.tokenizer
        if device == "auto":
            ids = os.environ.get("B200_GPU_IDS")
            device = f"cuda:{ids.split(',')[0]}" if ids and torch.cuda.is_available() else ("cuda:0" if torch.cuda.is_available() else "cpu")
        if str(device).startswith("cuda"):
            torch.cuda.set_device(torch.device(device))
            from .utils.numa import bind_to_gpu

            bind_to_gpu(device)

        if flat is not None:
            want = torch.bfloat16 if str(device).startswith("cuda") else torch.float32
            flat = flat.detach().to(device=device, dtype=want).clone()
        if ops == "fused" and ((spec.min_window and max_model_len > spec.min_window) or spec.has_gdn or spec.num_experts):
            # ``ops`` is one switch for learners and engines: a model the learner's kernel path serves (windowed layers through the
            # library fallback, experts GEMM by GEMM) may still need the engine's PyTorch path (no window in the paged kernels, no
            # recurrent-state or expert kernels there)
            logger.warning("rollout engine: this model runs on the engine's PyTorch path (ops='ref'); the learner keeps ops='fused'")
            ops = "ref"
        self.full_flat = None  # tensor parallel: staging copy of the whole model that the learners push into
        self._full_cv, self._full_step = threading.Condition(), None   # which version a follower's staging copy holds
        if tp_size > 1:
            self.engine = self._build_tp_engine(spec, device, ops, seed, max_model_len, num_blocks, gpu_memory_utilization, flat, tokenizer,
                                                max_running, tp_addr, tp_port)
        else:
            self.engine = RolloutEngine(spec, device=device, ops=ops, seed=seed, max_model_len=max_model_len, num_blocks=num_blocks,
                                        gpu_memory_utilization=gpu_memory_utilization, flat=flat, tokenizer=tokenizer,
                                        max_running=max_running, enable_prefix_caching=self._prefix_caching)
        self.prompt_q, self.results_q, self.eval_q = prompt_queue, results_queue, eval_queue
        self.reward_fn = reward_config.build() if reward_config is not None else None
        self.tokenizer = tokenizer
        self.inflight_updates = inflight_updates
        self.should_stop = threading.Event()
        self.shutdown_flag = threading.Event()
        self.lock = threading.Lock()  # engine state is touched by the loop thread and by update_weights
        # ``threading.Lock`` is not fair: the loop releases and re-takes it every few milliseconds and a control call could
        # wait through many engine steps.  Control calls announce themselves here and the loop stands back until they hold it.
        self._control_waiting = 0
        self._control_mutex = threading.Lock()
        self.error: BaseException | None = None
        self.pending: dict[int, PromptRequest] = {}
        # multi-turn tool / environment rollouts: engine request id -> (group key, sample index)
        self.tool_runner = None
        self.sessions: dict[int, tuple[int, int]] = {}
        self.groups: dict[int, dict] = {}
        self._group_ids = 0
        if envs_config is not None and envs_config.enabled:
            from .environments.base import TextRLEnvironment
            from .environments.tools.parsers import create_tool_parser
            from .environments.tools.tools import TOOL_REGISTRY, build_pools
            from .rollout.tool_session import ToolRunner

            pools = build_pools(envs_config, default_pool_size=max(8, max_running))
            text_env = next((n for n in envs_config.envs if isinstance(TOOL_REGISTRY[n], type) and issubclass(TOOL_REGISTRY[n], TextRLEnvironment)), None)
            names = [d["function"]["name"] for p in pools.values() for d in p.tool_definitions()] or list(pools)
            parser = create_tool_parser(envs_config.tool_parser_type, names)
            self.tool_runner = ToolRunner(pools, parser, tokenizer, envs_config.max_steps, envs_config.max_tool_calls, text_env)
            self.engine.tokenizer = tokenizer
        self.thread = threading.Thread(target=self._loop if tp_rank == 0 else self._follow, name="engine-loop", daemon=True)
        self.thread.start()

    # ------------------------------------------------------------------ tensor-parallel engines
    def _build_tp_engine(self, spec, device, ops, seed, max_model_len, num_blocks, util, flat, tokenizer, max_running, addr, port):
        """One rank of a tensor-parallel engine: own process group (NCCL for the symmetric-memory set-up, gloo for the
        command stream), this rank's weight shard, a KV cache for its heads.  Rank 0 drives; the others mirror every
        engine call it makes (``_TPLeader`` / ``_follow``), so all ranks run the same schedule on the same requests."""
        import datetime

        import torch.distributed as dist

        from .parallel.tp import TPContext, local_spec, shard_flat
        from .rollout.engine import KV_BLOCK, RolloutEngine

        dev = torch.device(device)
        on_gpu = dev.type == "cuda"
        dist.init_process_group(backend="cpu:gloo,cuda:nccl" if on_gpu else "gloo", init_method=f"tcp://{addr}:{port}", rank=self.tp_rank,
                                world_size=self.tp_size, timeout=datetime.timedelta(seconds=600), device_id=dev if on_gpu else None)
        self._tp_cmd_group = dist.new_group(backend="gloo")
        ls = local_spec(spec, self.tp_size)
        self.full_flat = None  # a full-size staging copy exists only while a host-supplied update is applied (CPU path)
        self._tp_spec = spec
        # without initial weights the shard starts random: the driver pushes the learners' weights before any prompt is queued
        local = shard_flat(flat, spec, self.tp_rank, self.tp_size) if flat is not None else None
        if on_gpu:
            tp = TPContext(spec.hidden_size, max(4096, max_model_len), dev)
        else:  # CPU processes: the PyTorch path with gloo all-reduces; same leader / follower command stream and weight updates
            from .parallel.tp import HostTPContext

            tp = HostTPContext(spec.hidden_size, max(4096, max_model_len), dev)
            ops = "ref"
        if num_blocks is None:
            free, total = torch.cuda.mem_get_info(dev)
            per_block = 2 * ls.num_layers * ls.num_kv_heads * KV_BLOCK * ls.head_dim * 2
            n = torch.tensor([max(16, int((free - (1 - util) * total) // per_block))], dtype=torch.int64, device=dev)
            dist.all_reduce(n, op=dist.ReduceOp.MIN)  # every rank must see the same number of KV blocks: same schedule
            num_blocks = int(n.item())
        eng = RolloutEngine(ls, device=dev, ops=ops, seed=seed, max_model_len=max_model_len, num_blocks=num_blocks, flat=local, tokenizer=tokenizer,
                            max_running=max_running, tp=tp, enable_prefix_caching=self._prefix_caching)
        return _TPLeader(eng, self._tp_cmd_group) if self.tp_rank == 0 else eng

    def _reshard(self, model_step: int) -> None:
        from .parallel.tp import shard_flat

        shard_flat(self.full_flat, self._tp_spec, self.tp_rank, self.tp_size, out=self.engine.model.flat.detach())
        self.engine.model_step = model_step
        self.engine.reset_prefix_cache()  # every rank, at the same point of the command stream: the schedules stay identical

    def _follow(self) -> None:
        """Ranks > 0 of a tensor-parallel engine: apply the leader's command batches in order."""
        import torch.distributed as dist

        try:
            if self.engine.device.type == "cuda":
                torch.cuda.set_device(self.engine.device)
            while not self.shutdown_flag.is_set():
                box = [None]
                dist.broadcast_object_list(box, src=0, group=self._tp_cmd_group)
                for cmd in box[0]:
                    if cmd[0] == "add":
                        self.engine.add_request(cmd[1], cmd[2])
                    elif cmd[0] == "step":
                        self.engine.step()
                    elif cmd[0] == "reshard":
                        # the whole model for this version arrives through this rank's own update call, which may still be copying
                        with self._full_cv:
                            if not self._full_cv.wait_for(lambda: self._full_step == cmd[1], timeout=600):
                                raise RuntimeError(f"tensor-parallel follower never received the weights of step {cmd[1]}")
                        self._reshard(cmd[1])
                    elif cmd[0] == "fence":
                        if self.engine.device.type == "cuda":
                            torch.cuda.synchronize(self.engine.device)
                        dist.barrier(group=self._tp_cmd_group)
                    elif cmd[0] == "set_step":
                        self.engine.model_step = cmd[1]
                        self.engine.reset_prefix_cache()
                    elif cmd[0] == "stop":
                        self.shutdown_flag.set()
        except BaseException as e:  # noqa: BLE001
            self.error = e
            logger.exception("tensor-parallel follower failed")

    def ready(self) -> bool:
        return True

    def get_kv_cache_info(self, seq_len: int) -> int:
        return self.engine.kv_cache_max_concurrency(seq_len)

    def set_should_stop(self, flag: bool) -> None:
        (self.should_stop.set if flag else self.should_stop.clear)()

    def check_background_threads(self) -> None:
        if self.error is not None:
            raise RuntimeError(f"engine loop died: {self.error!r}")
        if not self.thread.is_alive() and not self.shutdown_flag.is_set():
            raise RuntimeError("engine loop is not running")

    def _acquire_for_control(self) -> None:
        """Take the engine lock ahead of the loop's next step (the step that is running finishes first)."""
        with self._control_mutex:
            self._control_waiting += 1
        try:
            self.lock.acquire()
        finally:
            with self._control_mutex:
                self._control_waiting -= 1

    @contextlib.contextmanager
    def _control(self):
        self._acquire_for_control()
        try:
            yield
        finally:
            self.lock.release()

    # ---- control surface of the reference's engine actor (``open_instruct/vllm_utils.py:781-843``)
    def sleep(self) -> None:
        """Pause generation between engine steps and keep everything resident (the reference's ``sleep(level=0,
        mode="keep")``): returns once the step that was running has finished; no new step starts until ``wake_up``."""
        self.should_stop.set()
        self._paused = True
        with self._control():  # the loop holds the lock while it steps: taking it once means that step is over
            pass

    def wake_up(self) -> None:
        self._paused = False
        self.should_stop.clear()

    def reset_prefix_cache(self) -> bool:
        """Forget every cached prompt prefix (KV blocks shared between requests), as after a weight update: KV computed
        with older weights must not be reused for new requests."""
        with self._control():
            eng = self.engine._e if isinstance(self.engine, _TPLeader) else self.engine
            return bool(eng.reset_prefix_cache())

    def set_model_step(self, model_step: int) -> None:
        """Stamp the policy version that new results report (staleness accounting in the data-preparation actor)."""
        with self._control():
            (self.engine._e if isinstance(self.engine, _TPLeader) else self.engine).model_step = int(model_step)

    def begin_weight_update(self) -> None:
        """First half of a weight update whose data arrives from OUTSIDE this process (a learner storing through its
        CUDA-IPC mapping of the parameter buffer): waits for the engine step that is running and keeps the next one from
        starting until ``update_weights`` (or ``abort_weight_update``) ends the update, so no forward pass ever runs on
        half-old, half-new weights.  Requests in flight keep their KV cache (``inflight_updates`` semantics) and continue
        with the new weights at their next step; the reference likewise applies updates between engine steps."""
        self._acquire_for_control()
        self._update_open = True
        if self.tp_size > 1 and self.tp_rank == 0:
            # the followers mirror the leader's steps asynchronously: wait until every rank has finished what it was sent
            # (their last layers and sampling may still be in flight) before anyone's weights are written
            import torch.distributed as dist

            self.engine.send([("fence",)])
            if self.engine._e.device.type == "cuda":
                torch.cuda.synchronize(self.engine._e.device)
            dist.barrier(group=self._tp_cmd_group)

    def abort_weight_update(self) -> None:
        if getattr(self, "_update_open", False):
            self._update_open = False
            self.lock.release()

    def update_weights(self, flat, model_step: int) -> None:
        """In-process sync: copy ``flat`` into the engine's buffer (None: weights were already written
        into the buffer by a peer through its IPC mapping; only the version changes)."""
        if getattr(self, "_update_open", False):  # opened by begin_weight_update: the lock is already held
            try:
                self._apply_update(flat, model_step)
            finally:
                self._update_open = False
                self.lock.release()
            return
        if self.tp_size > 1 and self.tp_rank != 0:
            self._apply_update(flat, model_step)
            return
        with self._control():
            self._apply_update(flat, model_step)

    def _apply_update(self, flat, model_step: int) -> None:
        """The update itself; the caller holds ``self.lock`` (tensor-parallel followers have no loop to exclude)."""
        if self.tp_size > 1:
            if flat is None:
                # the learners already wrote this rank's shard in place (between engine steps, behind the fence of
                # ``begin_weight_update``): only the version stamp changes, on every rank
                if self.tp_rank == 0:
                    self.engine.send([("set_step", model_step)])
                    self.engine._e.model_step = model_step
                    self.engine._e.reset_prefix_cache()
                return
            if self.full_flat is None:
                self.full_flat = torch.empty(ParamLayoutTotal(self._tp_spec), dtype=self.engine.model.flat.dtype, device=self.engine.device)
            n = min(flat.numel(), self.full_flat.numel())  # the sender's buffer may carry padding for its world size
            if self.tp_rank == 0:  # followers reshard when the leader's command reaches them, at the same point of the schedule
                self.full_flat[:n].copy_(flat[:n].to(self.full_flat.dtype))
                self.engine.send([("reshard", model_step)])
                self._reshard(model_step)
            else:
                self.full_flat[:n].copy_(flat[:n].to(self.full_flat.dtype))
                with self._full_cv:   # the leader's "reshard" may reach the follower thread before this copy: it waits for it
                    self._full_step = model_step
                    self._full_cv.notify_all()
            return
        if flat is not None:
            self.engine.update_weights(flat, model_step)
        else:
            self.engine.model_step = model_step
            self.engine.reset_prefix_cache()  # K/V cached for later requests belong to the old weights

    def weights_checksum(self, expect_step: int | None = None) -> tuple[float, int, int]:
        """(sum of the weights this rank computes with, tp rank, tp size) - compared with the learner's after a sync.
        A tensor-parallel follower applies the reshard when the leader's command reaches it: wait (bounded) for that."""
        deadline = time.time() + 10.0
        while expect_step is not None and self.engine.model_step != expect_step and time.time() < deadline:
            time.sleep(0.002)
        with self._control():
            w = self.engine.model.flat.detach()
            n = self.engine.model.layout.total
            return float(w[:n].double().sum().item()), self.tp_rank, self.tp_size

    def weight_buffer_ipc(self):
        """Picklable description of the parameter buffer for a CUDA-IPC mapping in another process.  A rank of a
        tensor-parallel engine exports ITS shard buffer (the learners write every piece straight to its place in it,
        ``parallel.weight_sync.tp_push_plan``), tagged with its position so that the learner can order the destinations."""
        from .parallel.weight_sync import export_buffer

        eng = self.engine._e if isinstance(self.engine, _TPLeader) else self.engine
        d = export_buffer(eng.model.flat.detach())
        d.update({"tp_rank": self.tp_rank, "tp_size": self.tp_size})
        return d

    def _score(self, res: GenerationResult, req: PromptRequest) -> None:
        decoded = self.tokenizer.batch_decode(res.responses, skip_special_tokens=True) if self.tokenizer is not None else \
            [" ".join(map(str, r)) for r in res.responses]
        res.decoded_responses = decoded
        n = len(res.responses)
        if self.reward_fn is None:
            res.reward_scores, res.reward_metrics = [0.0] * n, {}
            return
        scores, metrics = asyncio.run(self.reward_fn(res.responses, decoded, [req.ground_truth] * n, [req.dataset] * n,
                                                     res.finish_reasons, res.request_info, [req.raw_query] * n))
        res.reward_scores, res.reward_metrics = [float(s) for s in scores], metrics

    def _loop(self) -> None:
        try:
            if self.engine.device.type == "cuda":
                torch.cuda.set_device(self.engine.device)  # the current device is per thread; raw kernel launches follow it
            while not self.shutdown_flag.is_set():
                admitted = False
                while self.engine.num_active() < self.engine.max_running and not self.should_stop.is_set():
                    try:
                        req = self.prompt_q.get(timeout=0.0 if self.engine.has_unfinished() else 0.05) if hasattr(self.prompt_q, "get") else None
                    except Exception:  # noqa: BLE001 - empty
                        break
                    if req is None or isinstance(req, ShutdownSentinel):
                        if isinstance(req, ShutdownSentinel):
                            self.shutdown_flag.set()
                        break
                    if self.tool_runner is not None:
                        self._start_tool_group(req)
                        admitted = True
                        continue
                    with self.lock:
                        rid = self.engine.add_request(req.prompt, req.generation_config, prompt_id=req.prompt_id, is_eval=req.is_eval,
                                                      ground_truth=req.ground_truth, dataset=req.dataset, raw_query=req.raw_query,
                                                      epoch_number=req.epoch_number)
                    self.pending[rid] = req
                    admitted = True
                if self.should_stop.is_set() and (not self.inflight_updates or getattr(self, "_paused", False)):
                    time.sleep(0.005)  # paused for a weight update, or put to sleep
                    continue
                if not self.engine.has_unfinished():
                    if not admitted:
                        time.sleep(0.005)
                    continue
                while self._control_waiting > 0:  # a control call (weight update, pause, checksum) goes first
                    time.sleep(0.0002)
                with self.lock:
                    finished = self.engine.step()
                for res in finished:
                    if res.index in self.sessions:
                        self._advance_tool_session(res)
                        continue
                    req = self.pending.pop(res.index)
                    res.index = req.index
                    self._score(res, req)
                    (self.eval_q if req.is_eval and self.eval_q is not None else self.results_q).put(res)
        except BaseException as e:  # noqa: BLE001
            self.error = e
            logger.exception("engine loop failed")

    # ------------------------------------------------------------------ multi-turn groups
    def _task_for(self, req: PromptRequest) -> dict | None:
        cfg = req.env_config
        if cfg is None:
            return None
        entries = getattr(cfg, "env_configs", None) or []
        return dict(entries[0].kwargs) if entries else None

    def _submit_turn(self, gid: int, j: int) -> None:
        g = self.groups[gid]
        prompt, cfg = g["sessions"][j].next_request()
        with self.lock:
            rid = self.engine.add_request(prompt, cfg)
        self.sessions[rid] = (gid, j)

    def _start_tool_group(self, req: PromptRequest) -> None:
        gid = self._group_ids
        self._group_ids += 1
        n = req.generation_config.n
        base = req.generation_config.seed if req.generation_config.seed is not None else self.engine.base_seed * 1000003 + gid
        task = self._task_for(req)
        sessions = [self.tool_runner.new_session(req.prompt, req.generation_config, base + j, task) for j in range(n)]
        self.groups[gid] = {"req": req, "sessions": sessions, "open": n, "start": time.perf_counter(), "task": task}
        for j in range(n):
            self._submit_turn(gid, j)

    def _advance_tool_session(self, res: GenerationResult) -> None:
        gid, j = self.sessions.pop(res.index)
        g = self.groups[gid]
        s = g["sessions"][j]
        again = self.tool_runner.on_turn(s, res.responses[0], res.logprobs[0], res.finish_reasons[0], g["task"])
        if again:
            self._submit_turn(gid, j)
            return
        self.tool_runner.close_session(s)
        g["open"] -= 1
        if g["open"] > 0:
            return
        from .data_types import RequestInfo, TokenStatistics

        req, ss = g["req"], g["sessions"]
        info = RequestInfo(num_calls=[x.num_calls for x in ss], timeouts=[int(x.timeout) for x in ss], tool_errors=[x.tool_error for x in ss],
                           tool_outputs=[x.tool_output for x in ss], tool_runtimes=[x.tool_runtime for x in ss],
                           tool_calleds=[x.tool_called for x in ss], tool_call_stats=[x.call_stats for x in ss],
                           rollout_states=[x.state.to_dict() for x in ss])
        now = time.perf_counter()
        out = GenerationResult(responses=[x.tokens for x in ss], finish_reasons=[x.finish_reason or "stop" for x in ss],
                               masks=[x.masks for x in ss], request_info=info, index=req.index, prompt_id=req.prompt_id,
                               epoch_number=req.epoch_number,
                               token_statistics=TokenStatistics(len(req.prompt), sum(len(x.tokens) for x in ss), now - g["start"], g["start"]),
                               start_time=g["start"], logprobs=[x.logprobs for x in ss], model_step=self.engine.model_step,
                               is_eval=req.is_eval, queries=[list(x.prompt) for x in ss], ground_truth=req.ground_truth,
                               dataset=req.dataset, raw_query=req.raw_query)
        del self.groups[gid]
        self._score(out, req)
        (self.eval_q if req.is_eval and self.eval_q is not None else self.results_q).put(out)

    def shutdown(self) -> None:
        if self.tp_size > 1 and self.tp_rank == 0:
            with self.lock:
                self.engine.send([("stop",)])
        self.shutdown_flag.set()
        self.thread.join(timeout=10)
        if self.tool_runner is not None:
            for p in self.tool_runner.pools.values():
                p.close()


# ======================================================================================= learner worker
class LearnerWorker:
    """One learner rank (the role of ``PolicyTrainerRayProcess``, ``open_instruct/grpo_fast.py:253-912``)."""

    def __init__(self, rank: int, world: int, master_addr: str, master_port: int, spec, args: GRPOExperimentConfig,
                 model_config: ModelConfig, num_training_steps: int, device: str | None = None):
        gpu = (os.environ.get("B200_GPU_IDS") or "0").split(",")[0]
        if device is not None and str(device).startswith("cuda:"):
            gpu = str(device).split(":")[1]
        os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "MASTER_ADDR": master_addr, "MASTER_PORT": str(master_port),
                           "LOCAL_RANK": gpu})
        self.rank, self.world = rank, world
        _, _, dev = pdist.init_distributed(backend=None if torch.cuda.is_available() and device != "cpu" else "gloo",
                                           timeout_s=args.backend_timeout * 60)
        self.device = torch.device(device) if device else dev
        from .utils.numa import bind_to_gpu

        bind_to_gpu(self.device)   # the CPUs (and, by first touch, the pinned host buffers) next to this rank's GPU
        set_seed(args.seed + rank)
        self.args, self.spec = args, spec
        warm = args.warm_up_steps or int(num_training_steps * args.warmup_ratio)
        cfg = LearnerConfig(ops=args.ops, comm=args.comm_backend, learning_rate=args.learning_rate, weight_decay=args.weight_decay,
                            max_grad_norm=args.max_grad_norm, lr_scheduler_type=args.lr_scheduler_type, warmup_steps=warm,
                            total_steps=max(1, num_training_steps * args.num_epochs * args.num_mini_batches),
                            gradient_checkpointing=model_config.gradient_checkpointing, seed=args.seed,
                            offload_optimizer=args.deepspeed_offload_optimizer, shard_parameters=args.shard_parameters,
                            decay_bias_and_norm=not args.set_weight_decay_on_bias_and_norm,
                            shard_degree=args.fsdp_shard_degree,
                            sequence_parallel_size=max(1, args.sequence_parallel_size),
                            sp_max_tokens=-(-getattr(args, "sp_max_tokens", 0) // max(1, args.sequence_parallel_size)) * max(1, args.sequence_parallel_size))
        self.learner = Learner(spec, cfg, device=self.device)
        src = model_config.model_name_or_path
        if src and os.path.isdir(src) and os.path.exists(os.path.join(src, "config.json")):
            self.learner.load_hf(src)
        self.ref: Learner | None = None
        if args.load_ref_policy and args.beta != 0.0:
            # frozen copy of the initial policy; only its forward is used (sharded like the policy when that is sharded:
            # the full weights are then staged through host memory once)
            sharded = self.learner.z3 is not None
            init = self.learner.full_flat(torch.empty(self.learner.model.layout.total, dtype=torch.bfloat16)) if sharded \
                else self.learner.model.flat.detach().clone()
            self.ref = Learner(spec, LearnerConfig(ops=args.ops, comm="nccl" if world > 1 else "none", seed=args.seed,
                                                   shard_parameters=sharded), device=self.device, flat_init=init)
        self.training_step = 0
        self._engine_views: list[torch.Tensor] = []

    def ready(self) -> bool:
        return True

    def optimizer_steps(self) -> int:
        return self.learner.global_step

    def flat_weights(self) -> torch.Tensor:
        return self.learner.full_flat()

    def weights_checksum(self, tp_rank: int = 0, tp_size: int = 1) -> float:
        """Sum of the bf16 working weights, or of the shard a tensor-parallel engine rank holds of them."""
        w = self.learner.full_flat()
        if tp_size > 1:
            from .parallel.tp import shard_flat

            return float(shard_flat(w[: self.learner.model.layout.total].contiguous(), self.spec, tp_rank, tp_size).double().sum().item())
        return float(w[: self.learner.model.layout.total].double().sum().item())

    def flat_weights_cpu(self) -> torch.Tensor:
        return self.learner.full_flat().to("cpu", copy=True)

    def step(self, data: CollatedBatchData, update_ref: bool = True) -> dict:
        """``update_ref=False``: the caller runs the reference-policy update itself (as a callback after the step)."""
        t0 = time.perf_counter()
        out = grpo_train_step(self.learner, data, self.args, self.ref)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        out["time/training"] = time.perf_counter() - t0
        self.training_step += 1
        if update_ref and self.ref is not None and self.args.ref_policy_update_freq and self.training_step % self.args.ref_policy_update_freq == 0:
            self.update_ref_policy()
        return out

    def update_ref_policy(self) -> None:
        """Polyak update ref <- alpha * policy + (1 - alpha) * ref on the flat buffers."""
        if self.ref is None:
            return
        with torch.no_grad():
            if self.learner.z3 is not None:  # both are sharded the same way: the update is local to every rank's slices
                self.ref.z3.local16.lerp_(self.learner.z3.local16, self.args.alpha)
                self.ref.z3._after_weights_changed()
            else:
                self.ref.model.flat.detach().lerp_(self.learner.model.flat.detach(), self.args.alpha)

    # ---- weight sync into engines living in other processes (CUDA IPC + multi-destination copy kernel)
    def connect_engines(self, ipc_descs: list) -> int:
        from .parallel.weight_sync import import_buffer

        self._engine_views = [import_buffer(d, self.device.index) for d in ipc_descs]
        # tensor-parallel engines: destinations ordered [engine][rank] (the caller lists leaders first, then followers)
        self._engine_tp = max([int(d.get("tp_size", 1)) for d in ipc_descs] or [1])
        if self._engine_tp > 1:
            leaders = [v for v, d in zip(self._engine_views, ipc_descs) if d.get("tp_rank", 0) == 0]
            others = [(d["tp_rank"], v) for v, d in zip(self._engine_views, ipc_descs) if d.get("tp_rank", 0) != 0]
            per_engine = self._engine_tp - 1
            ordered = []
            for e, lead in enumerate(leaders):
                mine = sorted(others[e * per_engine:(e + 1) * per_engine], key=lambda x: x[0])
                ordered += [lead] + [v for _, v in mine]
            self._engine_views = ordered
            self._tp_plans = {}
        return len(self._engine_views)

    def _tp_plan(self, lo: int, hi: int, src_shift: int = 0):
        """Device copy-tile table for the source range ``[lo, hi)`` of the full layout (built once per range)."""
        from .parallel.weight_sync import tp_push_plan

        key = (lo, hi, src_shift)
        if key not in self._tp_plans:
            plan = tp_push_plan(self.spec, self._engine_tp, lo, hi, n_engines=len(self._engine_views) // self._engine_tp, src_shift=src_shift)
            dev = torch.from_numpy(plan.view("u1").copy()).to(self.device) if len(plan) else torch.zeros(0, dtype=torch.uint8, device=self.device)
            self._tp_plans[key] = (dev, len(plan))
        return self._tp_plans[key]

    def push_weights(self) -> float:
        """Copy this rank's 1/world slice of the bf16 working copy into every engine's buffer."""
        from .parallel.weight_sync import push_slice

        t0 = time.perf_counter()
        n = self.learner.model.layout.total
        z = self.learner.z3
        if getattr(self, "_engine_tp", 1) > 1:
            # tensor-parallel engines: one kernel writes every piece of my slice to its place in every rank's shard layout
            from .parallel.weight_sync import push_tp

            if z is not None:
                ranges = [(*z._my_slice(u), u.soff - z._my_slice(u)[0]) for u in z.units]
                if self.rank == 0:
                    ranges.append((z.layout.decay_end, n, z.n_shard - z.layout.decay_end))
                src = z.local16
            else:
                per = -(-n // self.world)
                per = (per + 1023) // 1024 * 1024
                ranges = [(min(n, self.rank * per), min(n, (self.rank + 1) * per), 0)]
                src = self.learner.model.flat.detach()
            for lo, hi, shift in ranges:
                if hi > lo:
                    plan, n_tiles = self._tp_plan(lo, hi, shift)
                    push_tp(src, self._engine_views, plan, n_tiles)
        elif z is not None:
            # sharded parameters: every rank pushes the slices it owns, unit by unit, straight from its shard buffer
            # (no gather); rank 0 adds the replicated tail
            for u in z.units:
                a, b = z._my_slice(u)
                push_slice(z.local16, self._engine_views, a, b, src_offset=u.soff)
            if self.rank == 0:
                push_slice(z.local16, self._engine_views, z.layout.decay_end, n, src_offset=z.n_shard)
        else:
            per = -(-n // self.world)
            lo, hi = self.rank * per, min(n, (self.rank + 1) * per)
            push_slice(self.learner.model.flat.detach(), self._engine_views, lo, hi)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        pdist.barrier()
        return time.perf_counter() - t0

    def save_model(self, output_dir: str, tokenizer_path: str | None = None) -> None:
        full = self.learner.full_flat()  # a gather when the parameters are sharded: every rank takes part
        if self.rank == 0:
            tok = None
            if tokenizer_path:
                from transformers import AutoTokenizer

                tok = AutoTokenizer.from_pretrained(tokenizer_path)
            save_hf_checkpoint(full, self.spec, output_dir, tokenizer=tok)
            with open(os.path.join(output_dir, ".checkpoint_complete"), "w") as fh:
                fh.write("ok")
        pdist.barrier()

    def save_checkpoint_state(self, ckpt_dir: str, client_state: dict) -> None:
        d = os.path.join(ckpt_dir, f"step_{client_state['training_step']}")
        save_train_state(d, self.learner.opt, client_state)
        if self.ref is not None:
            ref_full = self.ref.full_flat()
            if self.rank == 0:
                torch.save(ref_full.detach().cpu(), os.path.join(d, "ref_policy.pt"))

    def load_checkpoint_state(self, ckpt_dir: str) -> dict | None:
        from .utils.common import get_last_checkpoint

        d = get_last_checkpoint(ckpt_dir)
        if d is None:
            return None
        st = load_train_state(d, self.learner.opt)
        self.training_step = st.get("training_step", 0)
        self.learner.global_step = st.get("optimizer_steps", self.training_step)
        p = os.path.join(d, "ref_policy.pt")
        if self.ref is not None and os.path.exists(p):
            self.ref.load_full_weights(torch.load(p, map_location="cpu" if self.ref.z3 is not None else self.device))
        return st

    def shutdown(self) -> None:
        pdist.destroy()


# ======================================================================================= driver
def setup_runtime_variables(args: GRPOExperimentConfig, streaming: StreamingDataLoaderConfig) -> GRPOExperimentConfig:
    """Derived quantities (``open_instruct/grpo_fast.py:1014-1049``)."""
    args.world_size = sum(args.num_learners_per_node)
    per_step = streaming.num_unique_prompts_rollout * streaming.num_samples_per_prompt_rollout
    args.num_training_steps = args.num_training_steps or max(1, args.total_episodes // per_step)
    if args.run_name is None:
        args.run_name = f"{args.exp_name}__{args.seed}__{int(time.time())}"
    return args


def validate_configs(args: GRPOExperimentConfig, streaming: StreamingDataLoaderConfig, vllm: VLLMConfig) -> None:
    if streaming.num_unique_prompts_rollout * streaming.num_samples_per_prompt_rollout < args.world_size:
        raise ValueError("fewer rollouts per step than learner ranks")
    if vllm.vllm_tensor_parallel_size not in (1, 2, 4, 8):
        raise ValueError("vllm_tensor_parallel_size must be 1, 2, 4 or 8")
    if args.single_gpu_mode and (args.world_size != 1 or vllm.vllm_num_engines != 1):
        raise ValueError("single_gpu_mode runs exactly one learner and one engine")
    sp = max(1, args.sequence_parallel_size)
    if args.world_size % sp:
        raise ValueError(f"sequence_parallel_size {sp} must divide the number of learner ranks {args.world_size}")
    if sp > 1 and streaming.num_unique_prompts_rollout * streaming.num_samples_per_prompt_rollout < args.world_size // sp:
        raise ValueError("fewer rollouts per step than data-parallel learner groups")


def submit_eval_prompts(eval_dataset, prompt_q, streaming: StreamingDataLoaderConfig, args: GRPOExperimentConfig, step: int, top_p: float = 1.0) -> int:
    """Queue every evaluation prompt (``is_eval`` requests go to the eval queue when they finish).  ``eval_pass_at_k``
    samples per prompt at the training temperature (cf. ``open_instruct/grpo_fast.py:1648-1720``)."""
    from .data_types import PromptRequest, SamplingConfig

    cfg = SamplingConfig(temperature=streaming.temperature if args.eval_pass_at_k > 1 else 0.0, top_p=top_p, max_tokens=streaming.eval_response_length,
                         n=max(1, args.eval_pass_at_k), stop=streaming.stop_strings or None, seed=args.seed + 7919 * step)
    for i in range(len(eval_dataset)):
        row = eval_dataset[i]
        prompt_q.put(PromptRequest(prompt=list(row["input_ids_prompt"]), generation_config=cfg, index=int(row.get("index", i)), prompt_id=f"eval_{step}_{i}",
                                   is_eval=True, raw_query=row.get("prompt"), ground_truth=row.get("ground_truth"), dataset=row.get("dataset"),
                                   training_step=step))
    return len(eval_dataset)


def collect_eval_results(eval_q, expected: int, timeout: float, args: GRPOExperimentConfig, max_possible_score: float) -> tuple[dict, int]:
    """Drain up to ``expected`` evaluation results (waiting at most ``timeout`` seconds) and reduce them to metrics."""
    from .grpo_utils import compute_pass_at_k_metrics

    got, deadline = [], time.time() + timeout
    while len(got) < expected:
        try:
            got.append(eval_q.get(timeout=max(0.0, min(1.0, deadline - time.time()))))
        except Exception:  # noqa: BLE001 - empty
            if time.time() >= deadline:
                break
    if not got:
        return {}, 0
    scores = [s for r in got for s in (r.reward_scores or [])]
    lens = [len(x) for r in got for x in r.responses]
    stops = [fr == "stop" for r in got for fr in r.finish_reasons]
    pids = [r.prompt_id for r in got for _ in r.responses]
    m = {"eval/scores": float(np.mean(scores)) if scores else 0.0, "eval/sequence_lengths": float(np.mean(lens)) if lens else 0.0,
         "eval/sequence_lengths_max": float(max(lens)) if lens else 0.0, "eval/stop_rate": float(np.mean(stops)) if stops else 0.0,
         "eval/num_prompts": float(len(got))}
    m.update(compute_pass_at_k_metrics(scores, pids, max(1, args.eval_pass_at_k), max_possible_score))
    return m, len(got)


def load_prompt_dataset(streaming: StreamingDataLoaderConfig, tc: TokenizerConfig, eval_split: bool = False):
    from .data.mixer import get_cached_dataset_tulu

    mix = streaming.dataset_mixer_eval_list if eval_split else streaming.dataset_mixer_list
    splits = streaming.dataset_mixer_eval_list_splits if eval_split else streaming.dataset_mixer_list_splits
    if not mix:
        return None
    override = None
    if streaming.system_prompt_override_file:
        override = open(streaming.system_prompt_override_file).read().strip()
    targs = [{}, {"max_prompt_token_length": streaming.max_prompt_token_length}][: len(streaming.dataset_transform_fn)]
    return get_cached_dataset_tulu(mix, splits, tc, streaming.dataset_transform_fn, targs,
                                   dataset_cache_mode=streaming.dataset_cache_mode,
                                   dataset_config_hash=streaming.dataset_config_eval_hash if eval_split else streaming.dataset_config_hash,
                                   dataset_local_cache_dir=streaming.dataset_local_cache_dir, dataset_skip_cache=streaming.dataset_skip_cache,
                                   system_prompt_override=override)


def ParamLayoutTotal(spec) -> int:
    from .models.spec import ParamLayout

    return ParamLayout(spec).total


def _weighted_average(per_rank: list[dict]) -> dict:
    """Token-weighted mean of the learners' metrics (``open_instruct/grpo_fast.py:1562-1595``)."""
    per_rank = [m for m in per_rank if m]
    if not per_rank:
        return {}
    w = np.array([max(m.get("num_response_tokens", 1.0), 1.0) for m in per_rank])
    out = {}
    for k in per_rank[0]:
        vals = np.array([m.get(k, 0.0) for m in per_rank], dtype=np.float64)
        out[k] = float(vals.sum()) if k == "num_response_tokens" else float(vals.max()) if k.startswith("time/") else float((vals * w).sum() / w.sum())
    return out


class GRPORun:
    """One GRPO run: the actor topology (learner ranks, rollout engines, data preparation, actor manager) and the pieces of
    a training step as methods, so that two drivers can share them - ``run()`` below is the plain loop of ``grpo_fast``
    (``open_instruct/grpo_fast.py:1796-2052``); ``open_instruct_b200/grpo.py`` drives the same pieces from a ``Trainer`` with
    callbacks, the structure of the reference's second entry point (``open_instruct/grpo.py``, ``grpo_callbacks.py``)."""

    def __init__(self, args: GRPOExperimentConfig, tc: TokenizerConfig, model_config: ModelConfig, streaming: StreamingDataLoaderConfig,
                 vllm: VLLMConfig, tools_config=None):
        from .actor_manager import ActorManager
        from .actors import ray_compat as ray
        from .parallel.weight_sync import sync_in_process

        args = setup_runtime_variables(args, streaming)
        args.temperature = streaming.temperature
        args.sp_max_tokens = streaming.pack_length * max(1, args.per_device_train_batch_size)  # largest packed micro-batch
        validate_configs(args, streaming, vllm)
        set_seed(args.seed)
        if tc.tokenizer_name_or_path is None:
            tc.tokenizer_name_or_path = model_config.model_name_or_path
        tokenizer = tc.tokenizer
        dataset = load_prompt_dataset(streaming, tc)
        eval_dataset = load_prompt_dataset(streaming, tc, eval_split=True)
        self.cached_only = None
        if args.cache_dataset_only:
            self.cached_only = {"cached": len(dataset)}
            return
        spec = get_spec(model_config.config_name or model_config.model_name_or_path)
        from .config.schemas import spec_with_rope_flags

        spec = spec_with_rope_flags(spec, model_config)   # --rope_scaling_factor: YaRN context extension
        if len(tokenizer) > spec.vocab_size:
            spec = spec.replace(vocab_size=(len(tokenizer) + 7) // 8 * 8)
        spec = spec.replace(pad_token_id=tokenizer.pad_token_id, eos_token_id=tokenizer.eos_token_id, bos_token_id=tokenizer.bos_token_id)
        reward_cfg = RewardConfig(apply_r1_style_format_reward=streaming.apply_r1_style_format_reward,
                                  r1_style_format_reward=streaming.r1_style_format_reward,
                                  apply_verifiable_reward=streaming.apply_verifiable_reward, verification_reward=streaming.verification_reward,
                                  non_stop_penalty=streaming.non_stop_penalty, non_stop_penalty_value=streaming.non_stop_penalty_value,
                                  additive_format_reward=streaming.additive_format_reward, reward_aggregator=streaming.reward_aggregator,
                                  verifier_functions=build_all_verifiers(args, streaming))
        followers: list = []
        few_gpus = not torch.cuda.is_available() or torch.cuda.device_count() < 2
        single = args.single_gpu_mode or (args.world_size == 1 and vllm.vllm_num_engines == 1 and few_gpus)
        max_len = streaming.max_prompt_token_length + max(streaming.response_length, streaming.eval_response_length or 0)
        tracker = Tracker(args.output_dir, args.run_name, {**asdict(args), **asdict(streaming), **asdict(vllm)},
                          report_to=("wandb", "tensorboard") if args.with_tracking else ("jsonl",), wandb_project=args.wandb_project_name,
                          wandb_entity=args.wandb_entity)
        dims = ModelDims.from_spec(spec)
        per_step = streaming.num_unique_prompts_rollout * streaming.num_samples_per_prompt_rollout
        qsize = (streaming.async_steps + 1) * streaming.num_unique_prompts_rollout
        last: dict = {}
        init_by_push = False
        if vllm.vllm_enforce_eager:
            os.environ["B200_DECODE_GRAPHS"] = "0"   # the engines (this process or its children) launch decode steps kernel by kernel

        if single:
            prompt_q, results_q, eval_q = ray.Queue(local=True), ray.Queue(maxsize=qsize, local=True), ray.Queue(local=True)
            device = "cuda:0" if torch.cuda.is_available() else "cpu"
            learner = LearnerWorker.__new__(LearnerWorker)
            LearnerWorker.__init__(learner, 0, 1, "127.0.0.1", pdist.find_free_port(), spec, args, model_config, args.num_training_steps, device=device)
            engine = EngineWorker(spec, prompt_q, results_q, eval_q, reward_cfg, tokenizer, device=device, ops=args.ops, seed=args.seed,
                                  max_model_len=max_len, num_blocks=None if torch.cuda.is_available() else 512,
                                  gpu_memory_utilization=0.25 if torch.cuda.is_available() else 0.9,
                                  flat=learner.flat_weights().clone(), inflight_updates=streaming.inflight_updates, envs_config=tools_config,
                                  enable_prefix_caching=vllm.vllm_enable_prefix_caching)
            learners, engines = [learner], [engine]
            single_objs = True
        else:
            import dataclasses

            cuda = torch.cuda.is_available()
            prompt_q, results_q, eval_q = ray.Queue(), ray.Queue(maxsize=qsize), ray.Queue()
            tc_plain = dataclasses.replace(tc)  # without the cached tokenizer object
            port = pdist.find_free_port()
            LW, EW = ray.remote(LearnerWorker), ray.remote(EngineWorker)
            from concurrent.futures import ThreadPoolExecutor

            t_up = time.time()
            stage = lambda what: logger.info("start-up: %s (%.1f s)", what, time.time() - t_up)   # where a stalled start-up stopped
            with ThreadPoolExecutor(max_workers=args.world_size) as ex:  # ranks must start together: they rendezvous in __init__
                futs = [ex.submit(LW.options(num_gpus=1 if cuda else 0, max_concurrency=4).remote, r, args.world_size, "127.0.0.1", port,
                                  spec, args, model_config, args.num_training_steps, None if cuda else "cpu")
                        for r in range(args.world_size)]
                learners = [f.result() for f in futs]
            stage(f"{args.world_size} learner ranks constructed")
            # On GPUs the engines start with random weights and receive the learners' through the first weight sync (the same
            # push kernel as every later one) instead of a by-value copy of the whole model handed to every engine process
            # (16 GB at 8B: gathered to the driver, shared with every engine rank, copied to each GPU and re-sharded there).
            # "auto": for models from a billion parameters up, where the by-value copies cost minutes and tens of GB of host memory
            mode = os.environ.get("B200_GRPO_INIT_BY_PUSH", "auto")
            big = ParamLayoutTotal(spec) >= 1_000_000_000
            init_by_push = (cuda and (mode == "1" or (mode == "auto" and big))) or mode == "force"
            init_flat = None if init_by_push else ray.get(learners[0].flat_weights_cpu.remote())
            tp = vllm.vllm_tensor_parallel_size
            followers = []
            if tp == 1:
                engines = [EW.options(num_gpus=1 if cuda else 0, max_concurrency=8).remote(
                    spec, prompt_q, results_q, eval_q, reward_cfg, tc_plain, "auto" if cuda else "cpu", args.ops, args.seed + 100 * i, max_len,
                    None if cuda else 512, vllm.vllm_gpu_memory_utilization, init_flat, streaming.inflight_updates, 256, tools_config,
                    enable_prefix_caching=vllm.vllm_enable_prefix_caching)
                    for i in range(vllm.vllm_num_engines)]
            else:
                # every rank of a tensor-parallel engine is its own process on its own GPU; the ranks of one engine rendezvous in
                # __init__, so they are created together
                tp_ports = [pdist.find_free_port() for _ in range(vllm.vllm_num_engines)]  # one rendezvous per engine
                with ThreadPoolExecutor(max_workers=tp * vllm.vllm_num_engines) as ex:
                    futs = [[ex.submit(EW.options(num_gpus=1 if cuda else 0, max_concurrency=8).remote, spec, prompt_q, results_q, eval_q, reward_cfg if r == 0 else None,
                                       tc_plain, "auto" if cuda else "cpu", args.ops, args.seed + 100 * i, max_len, None if cuda else 512, vllm.vllm_gpu_memory_utilization, init_flat,
                                       streaming.inflight_updates, 256, tools_config if r == 0 else None, r, tp, "127.0.0.1", tp_ports[i],
                                       enable_prefix_caching=vllm.vllm_enable_prefix_caching)
                             for r in range(tp)] for i in range(vllm.vllm_num_engines)]
                    handles = [[f.result() for f in row] for row in futs]
                engines = [row[0] for row in handles]
                followers = [h for row in handles for h in row[1:]]
            stage(f"{len(engines)} engines constructed (tensor-parallel size {tp}, {len(followers)} follower ranks)")
            ray.get([e.ready.remote() for e in engines + followers] + [l.ready.remote() for l in learners])
            if cuda:
                descs = ray.get([e.weight_buffer_ipc.remote() for e in engines + followers])
                ray.get([l.connect_engines.remote(descs) for l in learners])
                stage("learners mapped the engines' parameter buffers")
            single_objs = False

        # ---- everything the step methods need
        self.args, self.tc, self.model_config, self.streaming, self.vllm = args, tc, model_config, streaming, vllm
        self.ray, self.spec, self.tokenizer, self.dataset, self.eval_dataset = ray, spec, tokenizer, dataset, eval_dataset
        self.learners, self.engines, self.followers, self.single_objs, self.single = learners, engines, followers, single_objs, single
        self.prompt_q, self.results_q, self.eval_q = prompt_q, results_q, eval_q
        self.tracker, self.dims, self.per_step, self.max_len = tracker, dims, per_step, max_len
        self.total_params = ParamLayoutTotal(spec)
        self.manager = ActorManager({"prompts": prompt_q, "results": results_q, "eval": eval_q},
                                    enable_dashboard=args.enable_queue_dashboard and not single, port=args.queue_dashboard_port)
        self.manager.set_kv_cache_max_concurrency(self.call(engines[0], "get_kv_cache_info", max_len))
        self.sp = max(1, args.sequence_parallel_size)  # the ranks of one sequence-parallel group train on the same packs
        self.prep = DataPreparation(dataset, streaming, prompt_q, results_q, tokenizer, args.world_size // self.sp, args.per_device_train_batch_size,
                                    args.seed, args.num_training_steps, eval_queue=eval_q, top_p=vllm.vllm_top_p,
                                    run_name=args.run_name or args.exp_name, model_name=model_config.model_name_or_path)
        self.resume_step, self.eval_outstanding, self.total_tokens, self.t_run = 0, 0, 0, time.time()
        self.max_score = streaming.verification_reward + (streaming.r1_style_format_reward if streaming.apply_r1_style_format_reward else 0.0)
        from .utils.notify import ProgressReporter, warn_if_low_disk_space

        self.progress = ProgressReporter(args.num_training_steps)  # a no-op unless a scheduler description sink is configured
        warn_if_low_disk_space(args.output_dir, send_slack_alerts=getattr(args, "send_slack_alerts", False))
        self.last: dict = {}
        self.ref_update_in_step = True  # False: a callback of the driver updates the reference policy after the step
        self._closed = False
        if init_by_push:
            t_first = self.weight_sync(0)  # the engines' first weights
            logger.info("start-up: first weight sync %.2f s", t_first)
            if args.verify_weight_sync:
                diff = self._checksum_diff(0)
                if not diff <= 1e-3:
                    raise RuntimeError(f"engines did not receive the learners' initial weights (checksum difference {diff})")

    # ------------------------------------------------------------------ actor calls
    def call(self, obj, method, *a):
        return getattr(obj, method)(*a) if self.single_objs else self.ray.get(getattr(obj, method).remote(*a))

    def call_all(self, objs, method, *a, per_obj=None):
        if self.single_objs:
            return [getattr(o, method)(*(per_obj[i] if per_obj else a)) for i, o in enumerate(objs)]
        return self.ray.get([getattr(o, method).remote(*(per_obj[i] if per_obj else a)) for i, o in enumerate(objs)])

    # ------------------------------------------------------------------ pieces of a step
    def weight_sync(self, step: int) -> float:
        from .parallel.weight_sync import sync_in_process

        t0 = time.perf_counter()
        if self.single_objs:
            return sync_in_process(self.learners[0].flat_weights(), self.engines, step, self.total_params)
        if torch.cuda.is_available():
            # the learners store straight into the engines' parameter buffers: every engine first finishes the step it is
            # in and holds the next one back until the new version is complete
            self.call_all(self.engines, "begin_weight_update")
            try:
                self.call_all(self.learners, "push_weights")
            except BaseException:
                self.call_all(self.engines, "abort_weight_update")
                raise
            self.call_all(self.engines, "update_weights", None, step)
        else:
            flat = self.call(self.learners[0], "flat_weights_cpu")
            # every rank of a tensor-parallel engine receives the whole model and cuts its shard out of it when the leader's
            # command reaches it (the leader sends it after its own copy; a follower waits for its own copy to be complete)
            self.call_all(list(self.engines) + list(self.followers), "update_weights", flat, step)
        return time.perf_counter() - t0

    def begin(self) -> int:
        """Resume from ``checkpoint_state_dir`` when it holds a state, start the data-preparation thread; returns the step
        already completed."""
        args, prep = self.args, self.prep
        if args.checkpoint_state_dir and os.path.isdir(args.checkpoint_state_dir):
            st = self.call_all(self.learners, "load_checkpoint_state", args.checkpoint_state_dir)[0]
            if st:
                self.resume_step = st["training_step"]
                prep.set_state(st["data_prep_actor_state"])
                prep.next_step = self.resume_step + 1
                prep.trainer_step = self.resume_step
                prep.model_step = self.resume_step
                self.weight_sync(self.resume_step)
        prep.start()
        self.t_run = time.time()
        return self.resume_step

    def train_step(self, step: int) -> dict:
        """Health check, this step's packed data for every learner rank, one learner step on all ranks."""
        args = self.args
        t_step = time.perf_counter()
        self.call_all(self.engines, "check_background_threads")
        per_group = [self.prep.get_data(g, step) for g in range(args.world_size // self.sp)]
        per_rank = [per_group[r // self.sp] for r in range(args.world_size)]
        prep_metrics = per_rank[0][1]
        t_wait = time.perf_counter() - t_step
        metrics = _weighted_average(self.call_all(self.learners, "step", per_obj=[(d, self.ref_update_in_step) for d, _ in per_rank]))
        self.manager.report_training_step_time(metrics.get("time/training", 0.0))
        tokens = prep_metrics.get("val/total_response_tokens", 0) + prep_metrics.get("val/total_prompt_tokens", 0)
        self.total_tokens += tokens
        self.last = {**prep_metrics, **metrics, "training_step": step, "episode": step * self.per_step, "time/trainer_waiting_for_data": t_wait,
                     "learner_tokens_per_second_step": tokens / max(metrics.get("time/training", time.perf_counter() - t_step), 1e-9),
                     "learner_tokens_per_second_overall": self.total_tokens / max(time.time() - self.t_run, 1e-9),
                     "learner_mfu": self.dims.approximate_learner_utilization(
                         tokens, prep_metrics.get("val/sequence_lengths", 1.0) + self.streaming.max_prompt_token_length,
                         metrics.get("time/training", time.perf_counter() - t_step), args.world_size) if torch.cuda.is_available() else 0.0}
        self._t_step = t_step
        return self.last

    def _checksum_diff(self, step: int) -> float:
        """Largest difference between an engine rank's weight checksum and the learner's checksum of the same shard."""
        err = 0.0
        for h in list(self.engines) + list(self.followers):
            got, r, n = self.call(h, "weights_checksum", step)
            err = max(err, abs(got - self.call(self.learners[0], "weights_checksum", r, n)))
        return err

    def sync_step(self, step: int) -> float:
        """Pause the engines, push the new weights, (optionally) compare checksums, resume."""
        args = self.args
        self.manager.set_should_stop(True)
        self.call_all(self.engines, "set_should_stop", True)
        t_sync = self.weight_sync(step)
        if t_sync > WEIGHT_SYNC_TIMEOUT_S:
            raise TimeoutError("weight sync exceeded its time limit")
        if args.verify_weight_sync and not self.single_objs:
            self.last["debug/weight_sync_checksum_diff"] = self._checksum_diff(step)
        self.call_all(self.engines, "set_should_stop", False)
        self.manager.set_should_stop(False)
        self.prep.set_model_step(step)
        self.last["time/weight_sync"] = t_sync
        return t_sync

    def evaluate(self, step: int) -> None:
        """Evaluation prompts ride along with the training rollouts; results are picked up when they are ready."""
        args, streaming = self.args, self.streaming
        is_last = step == args.num_training_steps
        eval_due = ((args.eval_on_step_0 and step == 1) or step % args.local_eval_every == 0) if args.local_eval_every > 0 else False
        if self.eval_dataset is not None and len(self.eval_dataset) and args.local_eval_every > 0 and (eval_due or is_last) \
                and self.eval_outstanding == 0:
            self.eval_outstanding = submit_eval_prompts(self.eval_dataset, self.prompt_q, streaming, args, step,
                                                        args.eval_top_p or self.vllm.vllm_top_p)   # ``open_instruct/grpo_fast.py:1454``
        if self.eval_outstanding:
            em, n_got = collect_eval_results(self.eval_q, self.eval_outstanding, 600.0 if is_last else 0.0, args, self.max_score)
            if n_got >= self.eval_outstanding or is_last:
                self.last.update(em)
                self.eval_outstanding = 0
            elif n_got:
                # partial drain: put the count back so that the rest is not waited for twice
                self.eval_outstanding -= n_got
                self.last.update({k: v for k, v in em.items() if k == "eval/num_prompts"})

    def log_step(self, step: int) -> None:
        self.last["time/total"] = time.perf_counter() - getattr(self, "_t_step", time.perf_counter())
        self.tracker.log(self.last, step)
        self.progress.update(step)
        logger.info("step %d: score %.3f loss %.4f len %.1f sync %.3fs", step, self.last.get("scores", 0.0), self.last.get("loss/total_avg", 0.0),
                    self.last.get("val/sequence_lengths", 0.0), self.last.get("time/weight_sync", 0.0))

    def save_model(self, step: int | None = None) -> None:
        out = self.args.output_dir if step is None else os.path.join(f"{self.args.output_dir}_checkpoints", f"step_{step}")
        self.call_all(self.learners, "save_model", out, self.tc.tokenizer_name_or_path)

    def save_state(self, step: int) -> None:
        client = {"training_step": step, "optimizer_steps": self.call(self.learners[0], "optimizer_steps"), "episode": step * self.per_step,
                  "num_total_tokens": self.total_tokens, "data_prep_actor_state": self.prep.get_state()}
        self.call_all(self.learners, "save_checkpoint_state", self.args.checkpoint_state_dir, client)

    def checkpoint(self, step: int) -> None:
        args = self.args
        if args.save_freq > 0 and (step % args.save_freq == 0 or (args.eval_on_step_0 and step == 1)):
            self.save_model(step)
        if args.checkpoint_state_dir and args.checkpoint_state_freq > 0 and step % args.checkpoint_state_freq == 0:
            self.save_state(step)

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        ray = self.ray
        self.prep.shutdown()
        if self.single_objs:
            for e in self.engines:
                e.shutdown()
        else:
            for h in list(self.engines):
                try:
                    ray.get(h.shutdown.remote(), timeout=20)  # tensor-parallel leaders release their followers first
                except Exception:  # noqa: BLE001
                    pass
            for h in list(self.engines) + list(self.followers) + list(self.learners):
                ray.kill(h)
            for q in (self.prompt_q, self.results_q, self.eval_q):
                q.shutdown()
        self.manager.shutdown()
        self.tracker.close()

    # ------------------------------------------------------------------ the plain loop
    def run(self) -> dict:
        args = self.args
        try:
            start = self.begin()
            for step in range(start + 1, args.num_training_steps + 1):
                self.train_step(step)
                self.sync_step(step)
                self.evaluate(step)
                self.log_step(step)
                self.checkpoint(step)
            if args.save_final_model:
                self.save_model()
        finally:
            self.close()
        self.last["num_training_steps"] = args.num_training_steps
        return self.last


def main(args: GRPOExperimentConfig, tc: TokenizerConfig, model_config: ModelConfig, streaming: StreamingDataLoaderConfig,
         vllm: VLLMConfig, tools_config=None) -> dict:
    from .utils.notify import alert_on_failure

    return alert_on_failure(_main)(args, tc, model_config, streaming, vllm, tools_config)


def _main(args, tc, model_config, streaming, vllm, tools_config=None) -> dict:
    run = GRPORun(args, tc, model_config, streaming, vllm, tools_config)
    if run.cached_only is not None:
        return run.cached_only
    return run.run()


def cli() -> None:
    """Command line: a YAML / JSON recipe and / or ``--key value`` flags."""
    from .environments.tools.utils import EnvsConfig

    parser = ArgumentParserPlus((GRPOExperimentConfig, TokenizerConfig, ModelConfig, StreamingDataLoaderConfig, VLLMConfig, EnvsConfig))
    parser.set_defaults(exp_name="grpo", warmup_ratio=0.0, max_grad_norm=1.0, per_device_train_batch_size=1)
    main(*parser.parse())


if __name__ == "__main__":
    cli()
