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


def test_block_manager_prefix_cache():
    """Full blocks outlive their sequence: a later sequence with the same first tokens starts from them; unreferenced cached
    blocks are evicted (oldest first) only when no free block is left; a reset forgets them."""
    from open_instruct_b200.rollout.engine import KV_BLOCK, _Host

    h = _Host(8, 4)
    h.enable_prefix_cache(True)
    a = list(range(1000, 1000 + 150))           # 2 full blocks + 22 tokens
    h.add(1, 1, len(a), len(a) + 20)
    h.set_tokens(1, a)
    assert h.schedule()[0] == [1] and h.cached_tokens(1) == 0
    blocks_a = h.blocks(1)[0]
    h.advance(1, 1)                                # the prompt pass is done: its full blocks are findable
    b = a[:130] + [7, 8, 9]                        # shares the first 130 tokens = 2 full blocks
    h.add(2, 2, len(b), len(b) + 20)
    h.set_tokens(2, b)
    assert h.schedule()[0] == [2] and h.cached_tokens(2) == 2 * KV_BLOCK
    assert h.blocks(2)[0][:2] == blocks_a[:2] and h.blocks(2)[0][2] != blocks_a[2]
    c = a[:KV_BLOCK]                               # exactly one block: at least one token is always computed
    h.add(3, 3, len(c), len(c) + 4)
    h.set_tokens(3, c)
    assert h.schedule()[0] == [3] and h.cached_tokens(3) == 0
    st = h.prefix_cache_stats()
    assert st["block_hits"] == 2 and st["cached_blocks"] == 2
    # generated tokens become findable when the sequence finishes with its full token list
    h.advance(2, 1)
    for _ in range(70):
        h.schedule()
        h.advance(2, 1)
    full_b = b + [11] * 71                          # 133 + 71 = 204 tokens, K/V written for 203: 3 full blocks
    h.finish(2, full_b)
    h.finish(1)
    h.finish(3)
    assert h.prefix_cache_stats()["cached_blocks"] >= 3 and h.free_blocks() == 8   # cached blocks count as available
    d = full_b[:200]
    h.add(4, 4, len(d), len(d) + 8)
    h.set_tokens(4, d)
    assert h.schedule()[0] == [4] and h.cached_tokens(4) == 3 * KV_BLOCK           # prompt + generated history of sequence 2
    h.finish(4)
    # eviction: a request that needs every block takes the cached ones back
    e = list(range(5000, 5000 + 8 * KV_BLOCK - 10))
    h.add(5, 5, len(e), len(e) + 4)
    h.set_tokens(5, e)
    assert h.schedule()[0] == [5] and h.cached_tokens(5) == 0
    assert h.prefix_cache_stats()["evictions"] >= 3 and h.prefix_cache_stats()["cached_blocks"] == 0
    h.advance(5, 1)
    assert h.prefix_cache_stats()["cached_blocks"] == 7
    h.reset_prefix_cache()
    assert h.prefix_cache_stats()["cached_blocks"] == 0
    h.finish(5)
    assert h.free_blocks() == 8


@pytest.mark.parametrize("n_samples", [1, 3])
def test_engine_prefix_cache_gives_the_same_tokens(n_samples):
    """Generation with the prefix cache equals generation without it, for a repeated prompt and for a follow-up turn that
    extends prompt + answer; the second and third requests skip the cached part of their prompt pass."""
    import torch

    from open_instruct_b200.data_types import SamplingConfig
    from open_instruct_b200.models import get_spec
    from open_instruct_b200.rollout.engine import RolloutEngine

    spec = get_spec("tiny").replace(eos_token_id=None)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, spec.vocab_size, (150,), generator=g).tolist()
    cfg = SamplingConfig(temperature=0.0 if n_samples == 1 else 0.8, top_p=1.0, max_tokens=70, n=n_samples, seed=4)

    def run(cache: bool):
        eng = RolloutEngine(spec, device="cpu", ops="ref", num_blocks=64, seed=2, enable_prefix_caching=cache)
        first = eng.generate([prompt], cfg)[0]
        again = eng.generate([prompt], cfg)[0]
        follow = prompt + first.responses[0] + [3, 1, 4, 1, 5]
        turn2 = eng.generate([follow], cfg)[0]
        return eng, [first.responses, again.responses, turn2.responses], [first.logprobs, again.logprobs, turn2.logprobs]

    plain, want, want_lp = run(False)
    cached, got, got_lp = run(True)
    assert got == want
    for a, b in zip(got_lp, want_lp):
        for x, y in zip(a, b):
            assert all(abs(p - q) < 1e-4 for p, q in zip(x, y))
    st = cached.host.prefix_cache_stats()
    assert st["block_hits"] >= 2 + 3                       # 128 of 150 prompt tokens again, 192 of the 225-token second turn
    assert cached.stats["prefix_cached_tokens"] >= 128 + 192
    assert cached.stats["prefill_tokens"] <= plain.stats["prefill_tokens"] - (128 + 192)
    assert plain.stats.get("prefix_cached_tokens", 0) == 0
    cached.update_weights(cached.model.flat.detach().clone(), 1)
    assert cached.host.prefix_cache_stats()["cached_blocks"] == 0   # K/V of the old weights are not served after an update


def test_hybrid_model_survives_preemption():
    """Gated-DeltaNet layers keep a recurrent state per sequence beside the paged KV cache: a sequence that loses its blocks and is
    recomputed later rebuilds that state from its tokens - same greedy outputs as with a cache that never fills."""
    import torch

    from open_instruct_b200.data_types import SamplingConfig
    from open_instruct_b200.models import get_spec
    from open_instruct_b200.rollout.engine import RolloutEngine

    spec = get_spec("olmo-hybrid-7b").replace(vocab_size=300, hidden_size=64, intermediate_size=128, num_layers=4, num_heads=4, num_kv_heads=2,
                                              head_dim=16, layer_types=("gdn", "gdn", "gdn", "attention"), gdn_key_heads=2, gdn_value_heads=4,
                                              gdn_key_dim=12, gdn_value_dim=24, eos_token_id=None)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 300, (n,), generator=g).tolist() for n in (50, 70, 90, 60)]
    cfg = SamplingConfig(temperature=0.0, max_tokens=80, n=2)
    roomy = RolloutEngine(spec, device="cpu", ops="auto", num_blocks=256, seed=1)
    tight = RolloutEngine(spec, device="cpu", ops="auto", num_blocks=14, seed=1, flat=roomy.model.flat.detach().clone())
    a, b = roomy.generate(prompts, cfg), tight.generate(prompts, cfg)
    assert tight.host.preemptions() > 0 and roomy.host.preemptions() == 0
    assert all(x.responses == y.responses for x, y in zip(a, b))
    assert tight._gdn_state == {} and tight.host.free_blocks() == 14
