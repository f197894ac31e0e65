"""Rollout engine on CPU (ops='ref'): scheduler + paged cache + sampler against a plain forward."""

import torch


import pytest


def _engine(spec_kw=None, **kw):
    from open_instruct_b200.models import get_spec
    from open_instruct_b200.rollout.engine import RolloutEngine

    spec = get_spec("tiny").replace(eos_token_id=3, **(spec_kw or {}))
    eng = RolloutEngine(spec, device="cpu", ops="ref", seed=1, **kw)
    if spec_kw:  # biases start at zero and q/k norm weights at one: move them so that leaving them out would show
        with torch.no_grad():
            for name, v in eng.model.layout.views(eng.model.flat).items():
                if name.endswith(("bqkv", "q_norm", "k_norm")):
                    v.add_(0.3 * torch.randn(v.shape, generator=torch.Generator().manual_seed(5)))
    return eng, spec


@pytest.mark.parametrize("family", [None, {"attention_bias": True, "model_type": "qwen2"}, {"qk_norm": True, "model_type": "qwen3"}])
def test_greedy_matches_full_forward(family):
    from open_instruct_b200.data_types import SamplingConfig

    eng, spec = _engine(family, num_blocks=64)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(4, spec.vocab_size, (n,), generator=g).tolist() for n in (5, 70, 130)]
    res = eng.generate(prompts, SamplingConfig(temperature=0.0, max_tokens=12, n=1))
    for p, r in zip(prompts, res):
        toks = list(p)
        for step in range(len(r.responses[0])):
            ids = torch.tensor(toks)
            logits = eng.model.logits(ids, torch.arange(len(toks)), torch.tensor([0, len(toks)], dtype=torch.int32))
            nxt = int(torch.argmax(logits[-1]))
            lp = torch.log_softmax(logits[-1].float(), -1)[nxt].item()
            assert nxt == r.responses[0][step]
            assert abs(lp - r.logprobs[0][step]) < 1e-3
            toks.append(nxt)
        assert r.finish_reasons[0] in ("length", "stop")
    assert eng.host.free_blocks() == 64  # everything returned


def test_n_samples_share_prompt_and_are_reproducible():
    from open_instruct_b200.data_types import SamplingConfig

    eng, spec = _engine(num_blocks=64)
    prompt = list(range(10, 10 + 150))
    cfg = SamplingConfig(temperature=1.0, top_p=0.9, max_tokens=8, n=4, seed=123)
    a = eng.generate([prompt], cfg)[0]
    b = eng.generate([prompt], cfg)[0]
    assert a.responses == b.responses and len(a.responses) == 4
    assert len({tuple(r) for r in a.responses}) > 1  # different seeds per sample
    assert all(lp <= 1e-6 for r in a.logprobs for lp in r)
    assert a.token_statistics.num_prompt_tokens == 150


def test_preemption_recovers():
    from open_instruct_b200.data_types import SamplingConfig

    big, spec = _engine(num_blocks=64)
    small, _ = _engine(num_blocks=7)  # forces preemption: 3 sequences x up to 3 blocks each
    prompts = [list(range(5, 5 + n)) for n in (100, 110, 120)]
    cfg = SamplingConfig(temperature=0.0, max_tokens=40, n=1)
    ra = big.generate(prompts, cfg)
    rb = small.generate(prompts, cfg)
    assert [r.responses for r in ra] == [r.responses for r in rb]
    assert small.host.preemptions() > 0 and small.host.free_blocks() == 7


def test_sampler_distribution():
    from open_instruct_b200.rollout.sampler import sample_ref

    logits = torch.log(torch.tensor([[0.5, 0.3, 0.15, 0.05]])).repeat(2000, 1)
    temp, top_p = torch.ones(2000), torch.full((2000,), 0.9)
    seeds, ctr = torch.arange(2000), torch.zeros(2000, dtype=torch.int32)
    toks, lps = sample_ref(logits, temp, top_p, seeds, ctr)
    counts = torch.bincount(torch.tensor(toks), minlength=4).float() / 2000
    assert counts[3] == 0  # outside the nucleus
    assert abs(counts[0] - 0.5 / 0.95) < 0.04 and abs(counts[1] - 0.3 / 0.95) < 0.04


def test_native_decode_packing_matches_per_sequence_queries():
    """One native call fills positions, cache slots, context lengths, counters and the padded block table of a decode
    step exactly as the per-sequence block queries would."""
    import numpy as np

    from open_instruct_b200.rollout.engine import KV_BLOCK, _Host

    h = _Host(64, 8)
    prompt_lens = [70, 70, 130, 5]
    for sid, (g, pl) in enumerate(zip([0, 0, 1, 2], prompt_lens)):
        h.add(sid, g, pl, pl + 100)
    pre, dec, _ = h.schedule()
    assert pre == [0, 1, 2, 3] and not dec
    for sid in pre:
        h.advance(sid, 1)
    for step in range(70):
        pre, dec, _ = h.schedule()
        assert not pre and len(dec) == 4
        sids = np.asarray(dec, dtype=np.int64)
        B = len(dec)
        pos, slots = np.zeros(B, np.int64), np.zeros(B, np.int64)
        ctx, ctr, bt = np.zeros(B, np.int32), np.zeros(B, np.int32), np.full(B * 64, -7, np.int32)
        w = h.pack_decode(sids, pos, slots, ctx, ctr, bt)
        tables = [h.blocks(s)[0] for s in dec]
        assert w == -(-max(len(t) for t in tables) // 4) * 4
        btm = bt[: B * w].reshape(B, w)
        for i, (s, t) in enumerate(zip(dec, tables)):
            n = prompt_lens[s] + 1 + step
            assert list(btm[i, : len(t)]) == t and (btm[i, len(t):] == 0).all()
            assert ctx[i] == n and pos[i] == n - 1 and ctr[i] == step + 1
            assert slots[i] == t[(n - 1) // KV_BLOCK] * KV_BLOCK + (n - 1) % KV_BLOCK
        h.advance_many(sids)
    assert h.pack_decode(sids, pos, slots, ctx, ctr, np.zeros(3, np.int32)) == -2  # staging too small: the caller grows it
    with pytest.raises(KeyError):
        h.pack_decode(np.asarray([99], np.int64), pos, slots, ctx, ctr, bt)
