"""4-bit NormalFloat (NF4) block quantisation of frozen base weights, for QLoRA.

The reference reaches QLoRA through bitsandbytes (``BitsAndBytesConfig(load_in_4bit=True, bnb_4bit_quant_type="nf4",
bnb_4bit_use_double_quant=True)``, ``open_instruct/finetune.py:551-570``).  This is the same number format written in PyTorch:
a weight tensor is cut into blocks of 64 consecutive values, each block is scaled by its absolute maximum and every value is
replaced by the nearest of 16 code values - the quantiles of a standard normal rescaled to [-1, 1], with an exact zero - so a
block costs 64 x 4 bits + one fp32 scale (4.5 bits per weight; the scales' own second quantisation is not done).
"""

from __future__ import annotations

import torch

BLOCK = 64
# the 16 NF4 code values (Dettmers et al., "QLoRA", appendix E)
NF4_CODE = torch.tensor([-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
                         -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
                         0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0])


def quantize_nf4(t: torch.Tensor, block: int = BLOCK) -> tuple[torch.Tensor, torch.Tensor]:
    """(packed codes uint8 [ceil(n / 2)], per-block absmax fp32 [ceil(n / block)]) of the flattened tensor (zero-padded to a
    whole number of blocks)."""
    x = t.detach().reshape(-1).float()
    n = x.numel()
    pad = (-n) % block
    if pad:
        x = torch.cat([x, x.new_zeros(pad)])
    xb = x.view(-1, block)
    absmax = xb.abs().amax(dim=1).clamp(min=1e-12)
    y = xb / absmax[:, None]
    code = NF4_CODE.to(x.device)
    # nearest code value: the codes are sorted, so compare against the midpoints
    mids = (code[1:] + code[:-1]) / 2
    idx = torch.bucketize(y.reshape(-1), mids).to(torch.uint8)
    if idx.numel() % 2:
        idx = torch.cat([idx, idx.new_zeros(1)])
    packed = (idx[0::2] << 4) | idx[1::2]
    return packed.contiguous(), absmax.contiguous()


def dequantize_nf4(packed: torch.Tensor, absmax: torch.Tensor, numel: int, dtype=torch.float32, block: int = BLOCK) -> torch.Tensor:
    idx = torch.stack([packed >> 4, packed & 0xF], dim=1).reshape(-1).long()
    vals = NF4_CODE.to(packed.device)[idx][: absmax.numel() * block].view(-1, block) * absmax[:, None]
    return vals.reshape(-1)[:numel].to(dtype)


class NF4Tensor:
    """A frozen 2-D weight held as NF4 blocks; ``dequantize()`` gives it back (rounded) in the requested dtype."""

    def __init__(self, t: torch.Tensor):
        self.shape, self.numel = tuple(t.shape), t.numel()
        self.packed, self.absmax = quantize_nf4(t)

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        return dequantize_nf4(self.packed, self.absmax, self.numel, dtype).view(self.shape)

    def nbytes(self) -> int:
        return self.packed.numel() + 4 * self.absmax.numel()
