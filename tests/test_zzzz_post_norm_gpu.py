"""OLMo-2 / OLMo-3 block structure (norm after the sub-layer, q/k norm over all heads) on the sm_100a kernels against the PyTorch
fp32 statement of the same model.  The driver logic is covered on CPU (``test_fused_driver_cpu.py``); this file runs the same
comparison through the real kernels and sorts after the other GPU files."""

import pytest
import torch

from test_model_gpu import _batch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kv_heads", [None, "all"], ids=["gqa", "mha"])
@pytest.mark.parametrize("ckpt", [False, True])
def test_fused_post_norm_matches_ref(ckpt, kv_heads):
    from open_instruct_b200.models import LlamaModel, get_spec
    from open_instruct_b200.ops import lib

    spec = get_spec("tiny128").replace(post_norm=True, qk_norm=True, qk_norm_full=True, model_type="olmo2")
    if kv_heads == "all":
        spec = spec.replace(num_kv_heads=spec.num_heads)
    fused = LlamaModel(spec, device="cuda", dtype=torch.bfloat16, ops="fused", seed=3, gradient_checkpointing=ckpt)
    with torch.no_grad():
        for name, v in fused.p.items():
            if name.endswith("norm"):
                v.add_(torch.randn_like(v.float()).mul_(0.1).to(v.dtype))
    refm = LlamaModel(spec, device="cuda", dtype=torch.float32, ops="ref", flat=fused.flat.float().clone())
    ids, pos, cu, labels = _batch([200, 57, 300], spec.vocab_size, "cuda")
    lp_f, ent_f = fused.token_logprobs(ids, pos, cu, labels, want_entropy=True)
    lp_r, ent_r = refm.token_logprobs(ids, pos, cu, labels, want_entropy=True)
    n = (labels >= 0).sum()
    assert (lp_f - lp_r).abs().max().item() < 0.05
    assert (ent_f - ent_r).abs().max().item() < 0.05
    (-(lp_f.sum()) / n).backward()
    (-(lp_r.sum()) / n).backward()
    lib.check_status()
    gf, gr = fused.grad_flat(), refm.grad_flat()
    for name, e in fused.layout.entries.items():
        a = gf[e.offset:e.offset + e.numel]
        b = gr[e.offset:e.offset + e.numel]
        rel = ((a - b).norm() / (b.norm() + 1e-9)).item()
        assert rel < 0.06, f"{name}: rel grad error {rel}"


def test_fused_engine_generates_like_the_ref_engine_with_post_norm_blocks():
    from open_instruct_b200.data_types import SamplingConfig
    from open_instruct_b200.models import get_spec
    from open_instruct_b200.ops import lib
    from open_instruct_b200.rollout.engine import RolloutEngine

    spec = get_spec("tiny128").replace(post_norm=True, qk_norm=True, qk_norm_full=True, model_type="olmo2", eos_token_id=None)
    fused = RolloutEngine(spec, device="cuda", ops="fused", num_blocks=64, seed=2)
    refe = RolloutEngine(spec, device="cuda", ops="ref", num_blocks=64, seed=2, flat=fused.model.flat.clone())
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, spec.vocab_size, (n,), generator=g).tolist() for n in (7, 64, 150)]
    cfg = SamplingConfig(temperature=0.0, max_tokens=16, n=2)
    a, b = fused.generate(prompts, cfg), refe.generate(prompts, cfg)
    agree = total = 0
    for ra, rb in zip(a, b):
        for x, y, lx, ly in zip(ra.responses, rb.responses, ra.logprobs, rb.logprobs):
            n = next((i for i, (u, v) in enumerate(zip(x, y)) if u != v), len(x))  # bf16 may flip a near tie late
            agree += n
            total += len(x)
            for i in range(n):
                assert abs(lx[i] - ly[i]) < 0.08
    assert agree / total > 0.8
    lib.check_status()
    assert fused.host.free_blocks() == 64


def test_fused_mixture_of_experts_matches_ref():
    """OLMoE-style layers through the kernels (per-expert GEMMs over the sorted assignments) against the PyTorch fp32 model.  The
    router sees bf16 logits here and fp32 logits there, so a token whose two best experts are nearly tied may be routed
    differently: the bounds are on averages, not on the worst token."""
    from open_instruct_b200.models import LlamaModel, get_spec
    from open_instruct_b200.ops import lib

    spec = get_spec("tiny128").replace(qk_norm=True, qk_norm_full=True, num_experts=8, num_experts_per_tok=2, intermediate_size=256,
                                       model_type="olmoe")
    fused = LlamaModel(spec, device="cuda", dtype=torch.bfloat16, ops="fused", seed=3)
    refm = LlamaModel(spec, device="cuda", dtype=torch.float32, ops="ref", flat=fused.flat.float().clone())
    ids, pos, cu, labels = _batch([200, 57, 300], spec.vocab_size, "cuda")
    fused.aux_loss_coef = 0.1
    lp_f, _ = fused.token_logprobs(ids, pos, cu, labels)
    lp_r, _ = refm.token_logprobs(ids, pos, cu, labels)
    n = (labels >= 0).sum()
    assert (lp_f - lp_r).abs().mean().item() < 0.02
    assert abs(float(fused.aux_loss) - float(refm.aux_loss)) < 0.02
    (-(lp_f.sum()) / n).backward()
    (-(lp_r.sum()) / n + 0.1 * refm.aux_loss).backward()
    lib.check_status()
    gf, gr = fused.grad_flat(), refm.grad_flat()
    assert ((gf - gr).norm() / gr.norm()).item() < 0.15


def test_fused_sliding_window_layers_longer_than_the_window_match_ref():
    """OLMo-3-like layers (three windowed, one full) with documents longer than the window: the windowed layers go through the
    FlashAttention library on the fused path; log-probs and gradients against the PyTorch fp32 model with its band mask."""
    pytest.importorskip("flash_attn")
    from open_instruct_b200.models import LlamaModel, get_spec
    from open_instruct_b200.ops import lib

    spec = get_spec("tiny128").replace(post_norm=True, qk_norm=True, qk_norm_full=True, model_type="olmo3", num_layers=4, sliding_window=64,
                                       layer_types=("sliding", "sliding", "sliding", "attention"))
    fused = LlamaModel(spec, device="cuda", dtype=torch.bfloat16, ops="fused", seed=3)
    refm = LlamaModel(spec, device="cuda", dtype=torch.float32, ops="ref", flat=fused.flat.float().clone())
    ids, pos, cu, labels = _batch([200, 57, 300], spec.vocab_size, "cuda")
    lp_f, _ = fused.token_logprobs(ids, pos, cu, labels)
    lp_r, _ = refm.token_logprobs(ids, pos, cu, labels)
    n = (labels >= 0).sum()
    assert (lp_f - lp_r).abs().max().item() < 0.05
    (-(lp_f.sum()) / n).backward()
    (-(lp_r.sum()) / n).backward()
    lib.check_status()
    gf, gr = fused.grad_flat(), refm.grad_flat()
    assert ((gf - gr).norm() / gr.norm()).item() < 0.06
