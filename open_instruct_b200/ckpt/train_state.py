"""Resumable training state: ``<output_dir>/step_N`` (or ``epoch_N``) + ``COMPLETED`` marker.

Layout of one checkpoint directory (every rank writes its own shard file, rank 0 the rest):

    optim_rank{r}_of_{w}.pt     fp32 master / exp_avg / exp_avg_sq slices + optimizer step
    trainer_state.json          global step, epoch, loader state, scheduler position, extra client state
    rng_rank{r}.pt              python / numpy / torch CPU / torch CUDA generator states
    COMPLETED                   written last, after a barrier: a directory without it is ignored on resume

The bf16 working parameters are not stored: they are the rounded master weights, rebuilt on load.
Mirrors what ``accelerator.save_state`` + the ``COMPLETED`` marker give the reference
(``open_instruct/finetune.py:966-990``, ``open_instruct/utils.py:789-835``) and what DeepSpeed's
``save_checkpoint(client_state=...)`` gives its GRPO learner (``open_instruct/grpo_fast.py:767-825``).
``reshard_optimizer`` re-partitions saved shards for a different world size (the role of ZeRO
universal checkpoints, ``open_instruct/utils.py:929-964``).
"""

from __future__ import annotations

import json
import os
import random

import numpy as np
import torch

from ..parallel import dist as pdist


def rng_state() -> dict:
    st = {"python": random.getstate(), "numpy": np.random.get_state(), "torch": torch.get_rng_state()}
    if torch.cuda.is_available():
        st["cuda"] = torch.cuda.get_rng_state_all()
    return st


def set_rng_state(st: dict) -> None:
    random.setstate(st["python"])
    np.random.set_state(st["numpy"])
    torch.set_rng_state(st["torch"])
    if "cuda" in st and torch.cuda.is_available():
        try:
            torch.cuda.set_rng_state_all(st["cuda"])
        except Exception:  # noqa: BLE001 - device count may differ between save and load
            pass


def save_train_state(ckpt_dir: str, optimizer, trainer_state: dict, group=None, before_complete=None) -> None:
    """``before_complete(ckpt_dir)`` runs on rank 0 after the regular files and before the ``COMPLETED`` marker: state
    that lives beside the optimizer (LoRA adapters and their moments) is written there, so a marked directory is whole."""
    rank, world = pdist.rank(group), pdist.world_size(group)
    os.makedirs(ckpt_dir, exist_ok=True)
    sd = optimizer.state_dict()
    torch.save({k: (v.detach().cpu() if torch.is_tensor(v) else v) for k, v in sd.items()},
               os.path.join(ckpt_dir, f"optim_rank{rank}_of_{world}.pt"))
    torch.save(rng_state(), os.path.join(ckpt_dir, f"rng_rank{rank}.pt"))
    if rank == 0:
        tmp = os.path.join(ckpt_dir, "trainer_state.json.tmp")
        with open(tmp, "w") as fh:
            json.dump(trainer_state, fh, indent=2, default=str)
        os.replace(tmp, os.path.join(ckpt_dir, "trainer_state.json"))
        if before_complete is not None:
            before_complete(ckpt_dir)
    pdist.barrier(group)
    if rank == 0:
        with open(os.path.join(ckpt_dir, "COMPLETED"), "w") as fh:
            fh.write("COMPLETED")
    pdist.barrier(group)


def load_train_state(ckpt_dir: str, optimizer, group=None, restore_rng: bool = True) -> dict:
    rank, world = pdist.rank(group), pdist.world_size(group)
    path = os.path.join(ckpt_dir, f"optim_rank{rank}_of_{world}.pt")
    if os.path.exists(path):
        sd = torch.load(path, map_location=optimizer.master.device, weights_only=False)
    else:
        sd = reshard_optimizer(ckpt_dir, rank, world, optimizer.shard, optimizer.master.device)
    optimizer.load_state_dict(sd)
    # every rank refreshed only its own slice of the working copy: exchange them (parameter-sharded state keeps slices only)
    if world > 1 and not getattr(optimizer, "is_param_sharded", False):
        mine = optimizer.flat[optimizer.lo:optimizer.hi].contiguous()
        if optimizer.flat.is_cuda:
            torch.distributed.all_gather_into_tensor(optimizer.flat, mine, group=group)
        else:
            parts = [torch.empty_like(mine) for _ in range(world)]
            torch.distributed.all_gather(parts, mine, group=group)
            optimizer.flat.copy_(torch.cat(parts))
    rng_path = os.path.join(ckpt_dir, f"rng_rank{rank}.pt")
    if restore_rng and os.path.exists(rng_path):
        set_rng_state(torch.load(rng_path, weights_only=False))
    with open(os.path.join(ckpt_dir, "trainer_state.json")) as fh:
        return json.load(fh)


def reshard_optimizer(ckpt_dir: str, rank: int, world: int, shard: int, device) -> dict:
    """Rebuild this rank's optimizer slice from shards saved with another world size."""
    files = sorted(f for f in os.listdir(ckpt_dir) if f.startswith("optim_rank") and f.endswith(".pt"))
    if not files:
        raise FileNotFoundError(f"no optimizer shards in {ckpt_dir}")
    old_world = int(files[0].split("_of_")[1].split(".")[0])
    parts = [torch.load(os.path.join(ckpt_dir, f"optim_rank{r}_of_{old_world}.pt"), map_location="cpu", weights_only=False)
             for r in range(old_world)]
    out = {"step": parts[0]["step"], "rank": rank, "world": world, "shard": shard}
    lo, hi = rank * shard, (rank + 1) * shard
    for key in ("master", "m", "v"):
        full = torch.cat([p[key] for p in parts])
        piece = torch.zeros(shard, dtype=full.dtype)
        n = max(0, min(hi, full.numel()) - lo)
        if n > 0:
            piece[:n] = full[lo : lo + n]
        out[key] = piece.to(device)
    return out
