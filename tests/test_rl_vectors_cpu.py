"""Packing and advantage vectors with the values the reference's unit tests pin (``open_instruct/test_rl_utils.py``)."""

import numpy as np
import pytest
import torch

from open_instruct_b200 import rl_utils


@pytest.mark.parametrize("mask_tool_use,want0,want1", [
    (True, [False, False, False, True, False, True], [False, False, False, True]),
    (False, [False, False, False, True, True, True], [False, False, True, True]),
])
def test_pack_sequences_mask_tool_use(mask_tool_use, want0, want1):
    packed = rl_utils.pack_sequences(queries=[[1, 2, 3], [4, 5]], responses=[[10, 11, 12], [20, 21]], masks=[[1, 0, 1], [0, 1]],
                                     pack_length=8, pad_token_id=0, vllm_logprobs=[[0.0] * 3, [0.0] * 2], mask_tool_use=mask_tool_use)
    assert len(packed.response_masks) == 2
    assert packed.response_masks[0].dtype == torch.long
    assert packed.response_masks[0].bool().tolist() == want0
    assert packed.response_masks[1].bool().tolist() == want1
    assert packed.query_responses[0].tolist() == [1, 2, 3, 10, 11, 12] and packed.query_responses[1].tolist() == [4, 5, 20, 21]


def test_pack_sequences_strips_pad_tokens_from_queries_and_responses():
    """A left-padded prompt (or pad == eos inside a prompt) is packed without its pad tokens, as in the reference
    (``open_instruct/rl_utils.py:294``); log-probs and masks of padded response positions go with them."""
    packed = rl_utils.pack_sequences(queries=[[0, 0, 1, 2, 3], [4, 0, 5]], responses=[[10, 0, 12], [20, 21]], masks=[[1, 1, 1], [1, 1]],
                                     pack_length=16, pad_token_id=0, vllm_logprobs=[[-0.1, -0.2, -0.3], [-0.4, -0.5]])
    assert packed.query_responses[0].tolist() == [1, 2, 3, 10, 12, 4, 5, 20, 21]
    assert packed.position_ids[0].tolist() == [0, 1, 2, 3, 4, 0, 1, 2, 3]
    lp = packed.vllm_logprobs[0]
    assert torch.isnan(lp[:3]).all() and lp[3:5].tolist() == pytest.approx([-0.1, -0.3]) and lp[7:].tolist() == pytest.approx([-0.4, -0.5])
    assert packed.cu_seqlens[0].tolist() == [0, 5, 9]


def _three_samples():
    queries = [list(range(100, 112)), list(range(200, 214)), list(range(300, 314))]
    responses = [list(range(400, 407)), [500], [600]]
    return queries, responses


def test_pack_sequences_layout_and_min_num_batches():
    queries, responses = _three_samples()  # 19 + 15 + 15 tokens, pack length 40: two packs by default
    kw = dict(queries=queries, responses=responses, masks=[[1] * len(r) for r in responses], pack_length=40, pad_token_id=0,
              vllm_logprobs=[[0.0] * len(r) for r in responses])
    packed = rl_utils.pack_sequences(**kw)
    assert len(packed.query_responses) == 2
    assert packed.query_responses[0][:19].tolist() == queries[0] + responses[0]
    assert packed.query_responses[0][19:34].tolist() == queries[1] + responses[1]
    assert packed.query_responses[1][:15].tolist() == queries[2] + responses[2]
    spread = rl_utils.pack_sequences(**kw, min_num_batches=3)
    assert len(spread.query_responses) == 3 and all(len(s) > 0 for s in spread.query_responses)
    assert sum(len(s) for s in spread.query_responses) == sum(len(s) for s in packed.query_responses)


def test_calculate_advantages_packed_matches_unpacked():
    gamma = lam = 1.0
    values = np.array([[1] * 6 + [0] * 7, [2] * 7 + [0] * 6, [3] * 13])
    rewards = np.zeros((3, 13))
    rewards[0, 5], rewards[1, 6], rewards[2, 12] = 10, 20, 30
    adv, ret = rl_utils.calculate_advantages(values, rewards, gamma, lam)

    pv = np.full((1, 37), -1)
    pv[0, 4:9], pv[0, 12:18], pv[0, 24:36], pv[0, 36] = 1, 2, 3, 0
    pr = np.zeros((1, 37))
    pr[0, 8], pr[0, 17], pr[0, 35] = 10, 20, 30
    pd = np.zeros((1, 37))
    pd[0, 8] = pd[0, 17] = pd[0, 35] = 1
    pm = np.zeros((1, 37), dtype=int)
    pm[0, 4:9] = pm[0, 12:18] = pm[0, 24:36] = 1
    padv, pret = rl_utils.calculate_advantages_packed(pv, pr, gamma, lam, pd, pm)
    np.testing.assert_allclose(adv[0, :5], padv[0, 4:9])
    np.testing.assert_allclose(ret[1, :6], pret[0, 12:18])
    np.testing.assert_allclose(adv[2, :12], padv[0, 24:36])

    # the padded variant: values masked outside the responses, dones carry the sample index
    m = np.zeros((1, 42), dtype=int)
    m[0, 5:11] = m[0, 15:22] = m[0, 29:42] = 1
    v = np.full((1, 41), 5)
    v[0, 4:10], v[0, 14:21], v[0, 28:41] = 1, 2, 3
    r = np.zeros((1, 42))
    r[0, 10], r[0, 21], r[0, 41] = 10, 20, 30
    d = np.zeros((1, 42))
    d[0, 10], d[0, 21], d[0, 41] = 1, 2, 3
    v = np.where(m[:, 1:] == 0, 0, v)
    padv2, _ = rl_utils.calculate_advantages_packed(v, r[:, 1:], gamma, lam, d[:, 1:], m[:, 1:])
    np.testing.assert_allclose(adv[0, :6], padv2[0, 4:10])
    np.testing.assert_allclose(adv[1, :7], padv2[0, 14:21])


def test_masked_mean_vectors():
    v = torch.tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]])
    m = torch.tensor([[1.0, 1.0, 0.0], [1.0, 0.0, 0.0]])
    assert rl_utils.masked_mean(v, m).item() == pytest.approx((1 + 2 + 4) / 3)
    assert rl_utils.masked_mean(v, m, axis=1).item() == pytest.approx((1.5 + 4.0) / 2)   # mean of the per-row means
    assert rl_utils.masked_mean(v, torch.zeros_like(m), axis=1).item() == 0.0
    assert rl_utils.masked_mean(v, torch.tensor([[1.0, 1.0, 0.0], [0.0, 0.0, 0.0]]), axis=1).item() == pytest.approx(0.75)
    assert rl_utils.masked_mean(v, m, denominator=7.0).item() == pytest.approx(1.0)
    stacked = torch.stack([v * s for s in (1.0, 10.0, 100.0, 1000.0)])   # four estimators over one mask
    got = rl_utils.masked_mean(stacked, m, axis=1)
    assert got.shape == (4,)
    assert torch.allclose(got, torch.tensor([2.75, 27.5, 275.0, 2750.0]))
    got = rl_utils.masked_mean(stacked, m)
    assert torch.allclose(got, torch.tensor([7 / 3, 70 / 3, 700 / 3, 7000 / 3]))


def test_packed_batch_logps_vectors():
    """The per-sequence aggregation of ``open_instruct/test_dpo_utils.py`` (average: a fully masked row gives 0, not NaN),
    restated for packed rows with shifted labels."""
    from open_instruct_b200.data.collate import get_batch_logps

    lp = torch.tensor([-1.0, -2, -3, -4, -1, -2, -3, -4, -1, -2, -3, -4])
    shifted = torch.tensor([1, 2, 3, -100, -100, -100, -100, -100, 1, 2, -100, -100])
    cu = torch.tensor([0, 4, 8, 12])
    assert get_batch_logps(lp, shifted, cu, True).tolist() == [-2.0, 0.0, -1.5]
    assert get_batch_logps(lp, shifted, cu, False).tolist() == [-6.0, 0.0, -3.0]
