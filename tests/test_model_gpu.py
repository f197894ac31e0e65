"""Fused sm_100a model path against the PyTorch fp32 statement of the same model."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _batch(lens, vocab, device):
    T = sum(lens)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, vocab, (T,), generator=g).to(device)
    pos = torch.cat([torch.arange(n) for n in lens]).to(device)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=device)
    labels = torch.cat([ids[1:], ids.new_tensor([-100])]).clone()
    for e in cu[1:].tolist():
        labels[e - 1] = -100
    labels[:: 7] = -100
    return ids, pos, cu, labels


@pytest.mark.parametrize("variant", ["llama", "qwen2_bias", "qwen3_qknorm"])
@pytest.mark.parametrize("ckpt", [False, True])
def test_fused_matches_ref(ckpt, variant):
    from open_instruct_b200.models import LlamaModel, get_spec
    from open_instruct_b200.ops import lib

    spec = get_spec("tiny128")
    if variant == "qwen2_bias":
        spec = spec.replace(attention_bias=True, model_type="qwen2")
    elif variant == "qwen3_qknorm":
        spec = spec.replace(qk_norm=True, model_type="qwen3")
    fused = LlamaModel(spec, device="cuda", dtype=torch.bfloat16, ops="fused", seed=3, gradient_checkpointing=ckpt)
    if variant != "llama":  # biases start at zero and norm weights at one: move them so that their gradients are exercised
        with torch.no_grad():
            for name, v in fused.p.items():
                if name.endswith(("bqkv", "q_norm", "k_norm")):
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
    # a second micro-batch accumulates into main_grad
    lp2, _ = fused.token_logprobs(ids, pos, cu, labels)
    (-(lp2.sum()) / n).backward()
    assert ((fused.grad_flat() - 2 * gr).norm() / (2 * gr).norm()).item() < 0.06


def test_logits_no_grad_path():
    from open_instruct_b200.models import LlamaModel, get_spec

    spec = get_spec("tiny128")
    fused = LlamaModel(spec, device="cuda", dtype=torch.bfloat16, ops="fused", seed=5)
    refm = LlamaModel(spec, device="cuda", dtype=torch.float32, ops="ref", flat=fused.flat.float().clone())
    ids, pos, cu, _ = _batch([129, 64], spec.vocab_size, "cuda")
    a = fused.logits(ids, pos, cu).float()
    b = refm.logits(ids, pos, cu)
    assert ((a - b).norm() / b.norm()).item() < 0.03


@pytest.mark.parametrize("temp", [1.0, 0.7])
def test_chunked_head_matches_unchunked_and_ref(monkeypatch, temp):
    """A micro-batch longer than the logit chunk goes through the reused [chunk, V] workspace and recomputes each chunk's
    logits in the backward; log-probs, entropy and every gradient must match the one-piece path and the fp32 model."""
    from open_instruct_b200.models import LlamaModel, get_spec, llama
    from open_instruct_b200.ops import lib

    spec = get_spec("tiny128")
    ids, pos, cu, labels = _batch([500, 130, 270], spec.vocab_size, "cuda")
    n = (labels >= 0).sum()
    out = {}
    for name, chunk in (("whole", 8192), ("chunked", 256)):
        monkeypatch.setattr(llama, "LOGIT_CHUNK_TOKENS", chunk)
        m = LlamaModel(spec, device="cuda", dtype=torch.bfloat16, ops="fused", seed=11)
        lp, ent = m.token_logprobs(ids, pos, cu, labels, temperature=temp, want_entropy=True)
        ((lp * lp.detach().exp()).sum() / n).backward()  # a loss whose gradient differs from token to token
        out[name] = (lp.detach(), ent.detach(), m.grad_flat().clone(), m)
    lib.check_status()
    assert out["chunked"][3]._logit_ws.shape[0] == 256 and not hasattr(out["whole"][3], "_logit_ws")
    torch.testing.assert_close(out["chunked"][0], out["whole"][0], atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(out["chunked"][1], out["whole"][1], atol=1e-5, rtol=1e-5)
    a, b = out["chunked"][2], out["whole"][2]
    assert ((a - b).norm() / b.norm()).item() < 2e-3  # same kernels; only the fp32 accumulation order of the head's wgrad differs
    refm = LlamaModel(spec, device="cuda", dtype=torch.float32, ops="ref", flat=out["whole"][3].flat.float().clone())
    lp_r, ent_r = refm.token_logprobs(ids, pos, cu, labels, temperature=temp, want_entropy=True)
    ((lp_r * lp_r.detach().exp()).sum() / n).backward()
    assert (out["chunked"][0] - lp_r).abs().max().item() < 0.05 and (out["chunked"][1] - ent_r).abs().max().item() < 0.05
    assert ((a - refm.grad_flat()).norm() / refm.grad_flat().norm()).item() < 0.06


def test_chunked_head_memory_does_not_grow_with_tokens(monkeypatch):
    """Peak memory of the head: with chunking the logits of a long micro-batch take one [chunk, V] workspace, not [T, V]."""
    from open_instruct_b200.models import LlamaModel, get_spec, llama

    spec = get_spec("tiny128").replace(vocab_size=32768, num_layers=1)
    T = 8192
    ids, pos, cu, labels = _batch([T], spec.vocab_size, "cuda")
    peak = {}
    for name, chunk in (("whole", 1 << 20), ("chunked", 1024)):
        monkeypatch.setattr(llama, "LOGIT_CHUNK_TOKENS", chunk)
        m = LlamaModel(spec, device="cuda", dtype=torch.bfloat16, ops="fused", seed=1)
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        base = torch.cuda.memory_allocated()
        lp, _ = m.token_logprobs(ids, pos, cu, labels)
        (-lp.sum() / T).backward()
        torch.cuda.synchronize()
        peak[name] = torch.cuda.max_memory_allocated() - base
        del m, lp
    logits_bytes = T * spec.vocab_size * 2
    assert peak["whole"] - peak["chunked"] > 0.8 * (logits_bytes - 1024 * spec.vocab_size * 2)
