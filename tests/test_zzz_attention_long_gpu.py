"""Attention at the shapes that are timed (one 4096- / 8192-token document), a pack of many short documents and a row maximum
that keeps growing, against fp32 PyTorch.  Kept in a file of its own, late in the run: the references hold [heads, L, L] fp32
score matrices (1 GiB at 8192 tokens)."""

import pytest
import torch

from test_kernels_gpu import _attn_case, _rel

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("lens", [[4096], [8192], [37] * 60 + [1] * 20 + [129] * 9, [3000, 5, 1091]])
def test_attention_long_documents_and_many_short_ones(lens):
    """The shapes that are timed (one 4096- / 8192-token document) and a pack of many short documents, against fp32 PyTorch."""
    _attn_case(lens, 4, 2)


def test_attention_row_maximum_that_keeps_growing():
    """Scores whose row maximum keeps rising from one key tile to the next (keys scaled up along the sequence), so that the
    forward's lazy rescale of the running output takes its slow path again and again; compared with fp32 PyTorch."""
    from open_instruct_b200.ops import fused, ref

    torch.manual_seed(5)
    Hq, Hkv, Dh, T = 4, 2, 128, 1024
    cu = torch.tensor([0, 600, T], device="cuda", dtype=torch.int32)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * Dh, device="cuda")
    ramp = (1.0 + 6.0 * torch.arange(T, device="cuda") / T)[:, None]
    qkv[:, Hq * Dh:(Hq + Hkv) * Dh] *= ramp            # later keys are longer: the maximum of a row moves with every tile
    qkv[:, :Hq * Dh] *= 2.0
    qkv = qkv.bfloat16()
    scale = Dh ** -0.5
    out, lse = fused.attn_fwd(qkv, cu, Hq, Hkv, Dh, scale)
    ref_out = ref.attention_varlen(qkv.float(), cu, Hq, Hkv, Dh, scale)
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    assert _rel(out, ref_out) < 2e-2
