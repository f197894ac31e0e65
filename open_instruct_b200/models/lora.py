"""Low-rank adapters over the flat parameter buffer, and folding PEFT adapters into a checkpoint.

The reference wraps the model with ``peft.get_peft_model(LoraConfig(r, alpha, dropout, target_modules=q/k/v/o/gate/up/down))``
(``open_instruct/finetune.py:443-470``) and later merges with ``merge_lora.py``.  Here an adapter pair lives
per Hugging Face projection, i.e. per row slice of a fused entry (``wqkv`` holds q, k and v):

    W_eff[rows a:b] = W_base[a:b] + (alpha / r) * B @ A          A: [r, in]  B: [b - a, r]

* ``ops="ref"``: ``apply_ref(model)`` replaces the model's parameter views by differentiable ``W_eff`` tensors,
  autograd reaches ``A`` and ``B``.
* ``ops="fused"``: ``merge_into(model)`` writes ``W_eff`` into the bf16 working buffer (one small GEMM per
  projection), the unchanged fused engine produces ``dL/dW_eff`` in ``main_grad``, and ``pull_grads(model)``
  contracts it: ``dA = s * B^T dW``, ``dB = s * dW A^T``.  Base weights never receive an update.

Adapter files use PEFT's names (``base_model.model.<module>.lora_A.weight`` / ``lora_B.weight`` and an
``adapter_config.json`` with ``r`` and ``lora_alpha``) so either tool can merge the other's output.
"""

from __future__ import annotations

import json
import math
import os
import shutil
from pathlib import Path

import torch

from .spec import ModelSpec, ParamLayout

DEFAULT_TARGETS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


class LoRAAdapters:
    def __init__(self, spec: ModelSpec, layout: ParamLayout, rank: int = 64, alpha: float = 16.0, dropout: float = 0.0,
                 targets=DEFAULT_TARGETS, device="cpu", dtype=torch.float32, seed: int = 0):
        self.spec, self.layout, self.rank, self.alpha, self.dropout = spec, layout, rank, float(alpha), dropout
        self.scale = self.alpha / rank
        self.slots: list[tuple[str, str, int, int, int]] = []  # (hf module name, fused entry, row a, row b, in_features)
        for name, e in layout.entries.items():
            if len(e.shape) != 2 or name in ("embed", "lm_head"):
                continue
            for hf_name, a, b in layout.hf_names(name):
                module = hf_name.rsplit(".", 1)[0]
                if module.rsplit(".", 1)[-1] in targets:
                    self.slots.append((module, name, a, b, e.shape[1]))
        n = sum(rank * (inf + (b - a)) for _, _, a, b, inf in self.slots)
        self.flat = torch.zeros(n, device=device, dtype=dtype)
        self.A: dict[str, torch.Tensor] = {}
        self.B: dict[str, torch.Tensor] = {}
        off = 0
        g = torch.Generator().manual_seed(seed)
        for module, _, a, b, inf in self.slots:
            self.A[module] = self.flat[off:off + rank * inf].view(rank, inf)
            off += rank * inf
            self.B[module] = self.flat[off:off + rank * (b - a)].view(b - a, rank)
            off += rank * (b - a)
            # PEFT's default: A ~ kaiming-uniform(a=sqrt(5)), B = 0 so that training starts from the base model
            bound = 1.0 / math.sqrt(inf)
            self.A[module].copy_((torch.rand(rank, inf, generator=g) * 2 - 1) * bound)
        self.flat.requires_grad_(True)
        self.grad = None

    def num_parameters(self) -> int:
        return self.flat.numel()

    # ---------------------------------------------------------------- ref path
    def apply_ref(self, model, base_flat: torch.Tensor | None = None) -> None:
        """Install differentiable ``W_eff`` tensors as the autograd path's parameters (base frozen).  Call again after every
        optimizer step on the adapters: the override holds the graph of one forward."""
        base = (base_flat if base_flat is not None else model.flat).detach()
        views = model.layout.views(base)
        delta: dict[str, list] = {}
        for module, entry, a, b, _ in self.slots:
            delta.setdefault(entry, []).append((a, b, module))
        p = dict(views)
        for entry, parts in delta.items():
            rows = []
            cursor = 0
            w = views[entry]
            for a, b, module in sorted(parts):
                if a > cursor:
                    rows.append(w[cursor:a])
                rows.append(w[a:b] + self.scale * (self.B[module] @ self.A[module]).to(w.dtype))
                cursor = b
            if cursor < w.shape[0]:
                rows.append(w[cursor:])
            p[entry] = torch.cat(rows, 0)
        model.param_override = p

    # -------------------------------------------------------------- fused path
    @torch.no_grad()
    def merge_into(self, model, base) -> None:
        """``model.flat <- base + scale * B A`` for every adapted slice (other entries are copied once by the caller).
        ``base``: the frozen flat parameters, or a ``QuantizedBase`` that dequantises one entry at a time."""
        work_v = model.layout.views(model.flat)
        quant = isinstance(base, QuantizedBase)
        base_v = None if quant else model.layout.views(base)
        cur_name, cur = None, None
        for module, entry, a, b, _ in self.slots:
            if quant:
                if entry != cur_name:
                    cur_name, cur = entry, base.entry(entry)
                w0 = cur[a:b]
            else:
                w0 = base_v[entry][a:b]
            d = (self.B[module].float() @ self.A[module].float()) * self.scale
            work_v[entry][a:b].copy_((w0.float() + d).to(model.flat.dtype))

    @torch.no_grad()
    def pull_grads(self, model) -> torch.Tensor:
        """Contract ``main_grad`` (dL/dW_eff, fp32) into adapter gradients; returns the flat adapter gradient."""
        if self.grad is None:
            self.grad = torch.zeros_like(self.flat, dtype=torch.float32)
        gv = model.layout.views(model.main_grad)
        off = 0
        for module, entry, a, b, inf in self.slots:
            dw = gv[entry][a:b]
            r = self.rank
            self.grad[off:off + r * inf].view(r, inf).add_(self.scale * (self.B[module].float().t() @ dw))
            off += r * inf
            self.grad[off:off + r * (b - a)].view(b - a, r).add_(self.scale * (dw @ self.A[module].float().t()))
            off += r * (b - a)
        return self.grad

    # ------------------------------------------------------------------- files
    def save(self, out_dir: str, base_model_name_or_path: str = "") -> None:
        from safetensors.torch import save_file

        os.makedirs(out_dir, exist_ok=True)
        sd = {}
        for module, *_ in self.slots:
            sd[f"base_model.model.{module}.lora_A.weight"] = self.A[module].detach().to("cpu", torch.float32).contiguous()
            sd[f"base_model.model.{module}.lora_B.weight"] = self.B[module].detach().to("cpu", torch.float32).contiguous()
        save_file(sd, os.path.join(out_dir, "adapter_model.safetensors"), metadata={"format": "pt"})
        cfg = {"peft_type": "LORA", "task_type": "CAUSAL_LM", "r": self.rank, "lora_alpha": self.alpha, "lora_dropout": self.dropout,
               "target_modules": sorted({m.rsplit(".", 1)[-1] for m, *_ in self.slots}), "base_model_name_or_path": base_model_name_or_path,
               "bias": "none", "inference_mode": True}
        Path(out_dir, "adapter_config.json").write_text(json.dumps(cfg, indent=2))

    def load(self, adapter_dir: str) -> None:
        from safetensors.torch import load_file

        sd = load_file(os.path.join(adapter_dir, "adapter_model.safetensors"))
        with torch.no_grad():
            for module, *_ in self.slots:
                for which, dst in (("lora_A", self.A), ("lora_B", self.B)):
                    for key in (f"base_model.model.{module}.{which}.weight", f"base_model.model.{module}.{which}.default.weight"):
                        if key in sd:
                            dst[module].copy_(sd[key])
                            break


def merge_lora_checkpoint(base_dir: str, adapter_dir: str, output_dir: str, dtype=torch.bfloat16, save_tokenizer: bool = True) -> int:
    """Fold a PEFT LoRA adapter into a Hugging Face checkpoint shard by shard.  Returns the number of merged matrices.

    (``open_instruct/merge_lora.py:100-190`` does the same through ``PeftModel.merge_and_unload``; the 4-bit
    ``--qlora`` dequantisation branch needs bitsandbytes and is not provided.)"""
    from safetensors import safe_open
    from safetensors.torch import load_file, save_file

    cfg = json.loads(Path(adapter_dir, "adapter_config.json").read_text())
    scale = float(cfg["lora_alpha"]) / float(cfg["r"])
    ad = load_file(os.path.join(adapter_dir, "adapter_model.safetensors"))
    pairs: dict[str, dict[str, torch.Tensor]] = {}
    for k, v in ad.items():
        k2 = k.replace(".default", "")
        for which in ("lora_A", "lora_B"):
            tag = f".{which}.weight"
            if k2.endswith(tag):
                module = k2[: -len(tag)]
                module = module[len("base_model.model."):] if module.startswith("base_model.model.") else module
                pairs.setdefault(module + ".weight", {})[which] = v.float()
    out = Path(output_dir)
    out.mkdir(parents=True, exist_ok=True)
    merged = 0
    for f in sorted(Path(base_dir).glob("*.safetensors")):
        tensors = {}
        with safe_open(str(f), framework="pt") as h:
            for name in h.keys():
                t = h.get_tensor(name)
                if name in pairs and len(pairs[name]) == 2:
                    t = (t.float() + scale * (pairs[name]["lora_B"] @ pairs[name]["lora_A"])).to(dtype)
                    merged += 1
                tensors[name] = t.to(dtype) if t.is_floating_point() else t
        save_file(tensors, str(out / f.name), metadata={"format": "pt"})
    if merged != len([p for p in pairs.values() if len(p) == 2]):
        raise ValueError(f"adapter has {len(pairs)} matrices but only {merged} matched tensors of the base checkpoint")
    for f in Path(base_dir).iterdir():
        if f.is_file() and f.suffix != ".safetensors" and (save_tokenizer or "token" not in f.name):
            shutil.copy2(f, out / f.name)
    return merged


def main(argv=None) -> None:
    import argparse

    ap = argparse.ArgumentParser(description="Merge a LoRA adapter into its base model")
    ap.add_argument("--lora_model_name_or_path", required=True)
    ap.add_argument("--base_model_name_or_path", required=True)
    ap.add_argument("--output_dir", required=True)
    ap.add_argument("--save_tokenizer", action="store_true")
    ap.add_argument("--qlora", action="store_true")
    a = ap.parse_args(argv)
    if a.qlora:
        raise SystemExit("--qlora needs bitsandbytes 4-bit dequantisation, which this framework does not ship")
    n = merge_lora_checkpoint(a.base_model_name_or_path, a.lora_model_name_or_path, a.output_dir, save_tokenizer=a.save_tokenizer)
    print(f"merged {n} matrices into {a.output_dir}")


if __name__ == "__main__":
    main()


class QuantizedBase:
    """The frozen base of a QLoRA run: every adapted 2-D entry as NF4 blocks (``models/nf4.py``, 4.5 bits per weight), handed
    out dequantised one entry at a time.  Embeddings, the output head and norm weights are not quantised (they stay in the
    working buffer, which nothing updates)."""

    def __init__(self, model, entries: list[str]):
        from .nf4 import NF4Tensor

        views = model.layout.views(model.flat.detach())
        self.q = {name: NF4Tensor(views[name]) for name in entries}
        self.dtype = model.flat.dtype

    def entry(self, name: str) -> torch.Tensor:
        return self.q[name].dequantize(torch.float32)

    def nbytes(self) -> int:
        return sum(t.nbytes() for t in self.q.values())


class LoRATrainer:
    """Adapter training around a ``Learner``: the base weights stay frozen, AdamW runs on the adapters only.

    Both paths produce ``dL/dW_eff`` for the whole model first (autograd on the ref path, the fused engine's ``main_grad``
    on the GPU path) and contract it into adapter gradients (``pull_grads``); adapter gradients are summed over ranks, the
    adapters are updated identically everywhere, and the merged weights are written back into the working buffer."""

    def __init__(self, learner, rank: int = 64, alpha: float = 16.0, dropout: float = 0.0, lr: float = 1e-4, weight_decay: float = 0.0,
                 quantize_base: bool = False, eight_bit_optimizer: bool = False):
        """``quantize_base`` (QLoRA, ``open_instruct/finetune.py:551-570``): the frozen copy of the adapted matrices is kept as
        NF4 blocks and the model computes with their dequantised values, so the adapters learn on top of the quantised base."""
        self.learner = learner
        m = learner.model
        self.adapters = LoRAAdapters(m.spec, m.layout, rank, alpha, dropout, device=m.device, dtype=torch.float32, seed=learner.cfg.seed)
        if quantize_base:
            self.base = QuantizedBase(m, sorted({entry for _, entry, _, _, _ in self.adapters.slots}))
            with torch.no_grad():
                self.adapters.merge_into(m, self.base)  # B = 0: the working copy now holds the NF4-rounded base
        else:
            self.base = m.flat.detach().clone()
        if eight_bit_optimizer:   # ``use_8bit_optimizer``: the adapters' two moments in 8 bits, block-wise
            from ..parallel.adam8bit import AdamW8bit

            self.opt = AdamW8bit([self.adapters.flat], lr=lr, weight_decay=weight_decay)
        else:
            self.opt = torch.optim.AdamW([self.adapters.flat], lr=lr, weight_decay=weight_decay)

    def step(self, micro_batches: list[dict], lr: float | None = None) -> dict:
        """One optimizer step on the adapters over packed SFT micro-batches (token-mean loss)."""
        from ..data.collate import IGNORE
        from ..parallel import dist as pdist

        L = self.learner
        self.begin()
        losses, ntok = [], 0
        for mb in micro_batches:
            logp, _ = L.token_logprobs(mb)
            n = (mb["labels_shifted"] != IGNORE).sum().clamp(min=1)
            loss = -logp.sum() / n
            loss.backward()
            losses.append(loss.detach())
            ntok += int(n)
        g_norm = self.finish(len(micro_batches), lr)
        return {"loss": torch.stack(losses).mean(), "grad_norm": g_norm, "target_tokens": ntok}

    def begin(self) -> None:
        """Start an adapter step: clear the model's gradient buffer.  The caller then runs any number of forward / backward
        passes of ITS loss through the learner's model (whose working weights are the merged ones) and calls ``finish``."""
        self.learner.model.zero_grad()

    def finish(self, num_micro_batches: int, lr: float | None = None, max_grad_norm: float | None = None) -> torch.Tensor:
        """Contract the accumulated ``dL/dW_eff`` into adapter gradients (mean over micro-batches and ranks), step the adapters'
        AdamW and write the merged weights back.  Returns the adapter gradient norm (before clipping)."""
        from ..parallel import dist as pdist

        L, m = self.learner, self.learner.model
        if m.ops == "ref":
            if m.flat.grad is None:
                raise RuntimeError("adapter step without any backward pass")
            m.main_grad = m.flat.grad.float()
        self.adapters.grad = None
        g = self.adapters.pull_grads(m).div_(num_micro_batches * L.world)
        pdist.all_reduce_(g, group=L.group)
        norm = g.norm()
        if max_grad_norm and max_grad_norm > 0:
            g.mul_(torch.clamp(max_grad_norm / (norm + 1e-6), max=1.0))
        self.adapters.flat.grad = g.to(self.adapters.flat.dtype)
        if lr is not None:
            for grp in self.opt.param_groups:
                grp["lr"] = lr
        self.opt.step()
        self.opt.zero_grad(set_to_none=True)
        if m.ops == "ref":
            m.main_grad = None
        m.zero_grad()
        with torch.no_grad():
            self.adapters.merge_into(m, self.base)
        L._accum = 0   # micro-batches that went through ``Learner.backward`` were counted there
        return norm

    def save(self, out_dir: str, base_model_name_or_path: str = "") -> None:
        self.adapters.save(out_dir, base_model_name_or_path)

    # ---- training-state checkpoints (adapters are replicated: rank 0 writes, every rank reads)
    def state_dict(self) -> dict:
        return {"adapters": self.adapters.flat.detach().cpu().clone(), "optimizer": self.opt.state_dict(),
                "rank": self.adapters.rank if hasattr(self.adapters, "rank") else None}

    def load_state_dict(self, sd: dict) -> None:
        """Restore adapter weights and their AdamW moments, then rebuild the merged working weights from the frozen base."""
        if sd["adapters"].numel() != self.adapters.flat.numel():
            raise ValueError("checkpointed LoRA adapters have a different size (rank or target modules changed)")
        with torch.no_grad():
            self.adapters.flat.copy_(sd["adapters"].to(self.adapters.flat.device, self.adapters.flat.dtype))
        self.opt.load_state_dict(sd["optimizer"])
        with torch.no_grad():
            self.adapters.merge_into(self.learner.model, self.base)

    def save_state(self, ckpt_dir: str) -> None:
        import os

        tmp = os.path.join(ckpt_dir, "lora_state.pt.tmp")
        torch.save(self.state_dict(), tmp)
        os.replace(tmp, os.path.join(ckpt_dir, "lora_state.pt"))

    def load_state(self, ckpt_dir: str) -> None:
        import os

        path = os.path.join(ckpt_dir, "lora_state.pt")
        if not os.path.exists(path):
            raise FileNotFoundError(f"{ckpt_dir} holds no LoRA adapter state: resuming would restart the adapters from their "
                                    "initialisation; remove the checkpoint or resume without use_lora")
        self.load_state_dict(torch.load(path, map_location="cpu", weights_only=False))
