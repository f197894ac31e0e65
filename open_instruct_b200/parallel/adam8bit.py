"""AdamW whose two moments are stored in 8 bits, block by block.

The reference turns this on with ``use_8bit_optimizer`` next to QLoRA (``bnb.optim.AdamW(optim_bits=8, is_paged=True)``,
``open_instruct/finetune.py:668-678``).  Here it is a small PyTorch optimizer for the adapter tensors: every moment is cut into
blocks of ``block`` values, each block keeps one fp32 scale (its largest magnitude) and one byte per value indexing a fixed
256-entry code book that is dense near zero (values in a block spread over orders of magnitude: the first moment is signed, the
second is not and uses all 256 codes for one sign).  A step dequantises a block, applies the fp32 AdamW update, and quantises the
moments back; parameters and the update itself stay fp32.  State: 2 bytes per parameter + 8 bytes per block.
"""

from __future__ import annotations

import torch


def _codebook(signed: bool) -> torch.Tensor:
    """Sorted fp32 codes in [-1, 1] (signed: 127 negative, 0, 128 positive) or [0, 1]: log-spaced over seven decades."""
    n = 128 if signed else 255
    pos = torch.logspace(-7, 0, n, dtype=torch.float64)
    # signed: the negative side gives up its smallest code, not its largest: a block's extreme value must be exactly representable
    codes = torch.cat([-pos[1:].flip(0), torch.zeros(1, dtype=torch.float64), pos]) if signed else torch.cat([torch.zeros(1, dtype=torch.float64), pos])
    assert codes.numel() == 256
    return codes.float()


class _Quantised:
    """A flat fp32 tensor held as bytes + per-block scales."""

    def __init__(self, numel: int, block: int, signed: bool, device):
        self.numel, self.block = numel, block
        self.nblocks = -(-numel // block)
        self.codes = _codebook(signed).to(device)
        self.edges = (self.codes[1:] + self.codes[:-1]) / 2        # nearest code = bucket between midpoints
        zero = int((self.codes == 0).nonzero()[0])
        self.q = torch.full((self.nblocks * block,), zero, dtype=torch.uint8, device=device)
        self.scale = torch.zeros(self.nblocks, dtype=torch.float32, device=device)

    def get(self) -> torch.Tensor:
        x = self.codes[self.q.long()].view(self.nblocks, self.block) * self.scale[:, None]
        return x.reshape(-1)[: self.numel]

    def put(self, x: torch.Tensor) -> None:
        pad = self.nblocks * self.block - self.numel
        xb = torch.nn.functional.pad(x.reshape(-1), (0, pad)).view(self.nblocks, self.block)
        self.scale = xb.abs().amax(dim=1)
        unit = xb / self.scale.clamp(min=1e-38)[:, None]
        self.q = torch.bucketize(unit.reshape(-1), self.edges).to(torch.uint8)

    def nbytes(self) -> int:
        return self.q.numel() + 4 * self.scale.numel()


class AdamW8bit(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0, block: int = 256):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.block = block

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["m"] = _Quantised(p.numel(), self.block, True, p.device)
                    st["v"] = _Quantised(p.numel(), self.block, False, p.device)
                st["step"] += 1
                g = p.grad.float().reshape(-1)
                m = st["m"].get().mul_(b1).add_(g, alpha=1 - b1)
                v = st["v"].get().mul_(b2).addcmul_(g, g, value=1 - b2)
                st["m"].put(m)
                st["v"].put(v)
                if group["weight_decay"]:
                    p.mul_(1 - group["lr"] * group["weight_decay"])
                mhat = m / (1 - b1 ** st["step"])
                vhat = v / (1 - b2 ** st["step"])
                p.add_((mhat / (vhat.sqrt() + group["eps"])).view_as(p).to(p.dtype), alpha=-group["lr"])
        return loss

    def state_bytes(self) -> int:
        return sum(st["m"].nbytes() + st["v"].nbytes() for st in self.state.values() if st)

    # the quantised state holds plain tensors: make it picklable the way torch's state_dict expects
    def state_dict(self):
        sd = {"param_groups": [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups], "state": []}
        for group in self.param_groups:
            for p in group["params"]:
                st = self.state.get(p)
                sd["state"].append(None if not st else {"step": st["step"], "m_q": st["m"].q.cpu(), "m_scale": st["m"].scale.cpu(),
                                                          "v_q": st["v"].q.cpu(), "v_scale": st["v"].scale.cpu()})
        return sd

    def load_state_dict(self, sd):
        params = [p for g in self.param_groups for p in g["params"]]
        for g, saved in zip(self.param_groups, sd["param_groups"]):
            g.update(saved)
        for p, st in zip(params, sd["state"]):
            if st is None:
                continue
            m, v = _Quantised(p.numel(), self.block, True, p.device), _Quantised(p.numel(), self.block, False, p.device)
            m.q, m.scale, v.q, v.scale = (st[k].to(p.device) for k in ("m_q", "m_scale", "v_q", "v_scale"))
            self.state[p] = {"step": st["step"], "m": m, "v": v}
