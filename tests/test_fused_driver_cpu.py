"""The fused path's hand-driven forward / backward (layer stash, recomputation, chunked output head, in-place gradient
rewrites) with every kernel replaced by its PyTorch restatement (``ops="emulated"``), against autograd over the plain PyTorch
path.  The kernels are tested one by one on the GPU; this is the test of what calls them."""
import pytest
import torch

from open_instruct_b200.models import LlamaModel, ModelSpec
from open_instruct_b200.models import llama as llama_mod

BASE = dict(vocab_size=300, hidden_size=64, intermediate_size=128, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16)
OLMO2 = dict(post_norm=True, qk_norm=True, qk_norm_full=True)
VARIANTS = {
    "llama": ({}, {}),
    "llama-checkpointing": ({}, dict(ckpt=True)),
    "llama-chunked-head-recompute": ({}, dict(chunk=128, keep_cheap=False, temperature=0.7)),
    "qwen2-bias": (dict(attention_bias=True), {}),
    "llama-yarn": (dict(rope_scaling={"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32}), {}),
    "qwen3-head-norm": (dict(qk_norm=True), {}),
    "tied-embeddings": (dict(tie_word_embeddings=True), {}),
    "olmo2": (OLMO2, {}),
    "olmo2-checkpointing": (OLMO2, dict(ckpt=True)),
    "olmo2-chunked-head-recompute": (OLMO2, dict(chunk=128, keep_cheap=False)),
    "olmo2-mha": ({**OLMO2, "num_kv_heads": 4}, {}),
    "post-norm-only": (dict(post_norm=True), {}),
    "olmo3-documents-longer-than-the-window": ({**OLMO2, "num_layers": 4, "sliding_window": 16, "layer_types": ("sliding", "sliding", "sliding", "attention")}, {}),
    "olmo3-longer-than-the-window-checkpointing": ({**OLMO2, "num_layers": 4, "sliding_window": 16, "layer_types": ("sliding", "sliding", "sliding", "attention")}, dict(ckpt=True)),
    "mistral-all-layers-windowed": (dict(sliding_window=32), {}),
    "olmoe": (dict(qk_norm=True, qk_norm_full=True, num_experts=4, num_experts_per_tok=2, intermediate_size=48), {}),
    "olmoe-renormalised-checkpointing": (dict(num_experts=4, num_experts_per_tok=2, norm_topk_prob=True, intermediate_size=48), dict(ckpt=True)),
    "olmoe-balancing-loss": (dict(num_experts=8, num_experts_per_tok=2, intermediate_size=48), dict(aux=0.3)),
    "olmoe-balancing-loss-checkpointing": (dict(num_experts=8, num_experts_per_tok=3, intermediate_size=48), dict(aux=0.3, ckpt=True, keep_cheap=False)),
}


def _pair(spec, ckpt=False):
    a = LlamaModel(spec, ops="ref", seed=1)
    with torch.no_grad():
        for v in a.layout.views(a.flat).values():
            if v.dim() == 1:
                v.uniform_(0.5, 1.5)  # norm weights and biases away from their trivial initialisation
    b = LlamaModel(spec, ops="emulated", seed=1, flat=a.flat.detach().clone(), gradient_checkpointing=ckpt)
    return a, b


def _batch(spec, lens=(70, 130, 33), seed=0):
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    ids = torch.randint(0, spec.vocab_size, (T,), generator=g)
    pos = torch.cat([torch.arange(n) for n in lens])
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32)
    labels = torch.roll(ids, -1)
    labels[::7] = -100
    return ids, pos, cu, labels, torch.randn(T, generator=g)


@pytest.mark.parametrize("name", list(VARIANTS))
def test_hand_driven_backward_equals_autograd(name, monkeypatch):
    extra, opts = VARIANTS[name]
    spec = ModelSpec(**{**BASE, **extra})
    a, b = _pair(spec, ckpt=opts.get("ckpt", False))
    b.keep_cheap_activations = opts.get("keep_cheap", True)
    if "chunk" in opts:
        monkeypatch.setattr(llama_mod, "LOGIT_CHUNK_TOKENS", opts["chunk"])
    ids, pos, cu, labels, wgt = _batch(spec)
    got = []
    aux = opts.get("aux", 0.0)   # mixture of experts: weight of the load-balancing loss in the trainer's loss
    b.aux_loss_coef = aux
    for m in (a, b):
        for _ in range(2):  # two micro-batches: gradients accumulate
            lp, ent = m.token_logprobs(ids, pos, cu, labels, opts.get("temperature", 1.0), want_entropy=True)
            loss = (lp * wgt).sum()
            if aux:   # differentiable on the autograd path; a number on the hand-driven path, whose backward adds the gradient itself
                loss = loss + aux * m.aux_loss
            loss.backward()
        got.append((lp.detach(), ent.detach(), m.grad_flat().clone()))
    if spec.num_experts:
        assert abs(float(a.aux_loss) - float(b.aux_loss)) < 1e-5 and not b.aux_loss.requires_grad
    (lp0, e0, g0), (lp1, e1, g1) = got
    assert (lp0 - lp1).abs().max().item() < 1e-5
    assert (e0 - e1).abs().max().item() < 1e-5
    assert g0.abs().max().item() > 1.0
    for n, e in a.layout.entries.items():
        d = (g0[e.offset:e.offset + e.numel] - g1[e.offset:e.offset + e.numel]).abs().max().item()
        assert d < 2e-4, (n, d)


def test_hidden_state_bridge_for_the_reward_head():
    spec = ModelSpec(**{**BASE, **OLMO2})
    a, b = _pair(spec)
    ids, pos, cu, _, _ = _batch(spec)
    w = torch.randn(sum((70, 130, 33)), spec.hidden_size, generator=torch.Generator().manual_seed(3))
    for m in (a, b):
        (m.hidden_states(ids, pos, cu) * w).sum().backward()
    ga, gb = a.grad_flat(), b.grad_flat()
    assert (ga - gb).abs().max().item() < 1e-5 * ga.abs().max().item()


@pytest.mark.parametrize("family", ["llama", "olmo2", "olmoe"])
def test_learner_steps_on_the_emulated_path_follow_the_pytorch_path(family):
    """Three optimizer steps of two micro-batches each through ``Learner``: the fused path's branches of the learner (fp32
    gradient buffer, zeroing after the step, gradient-ready hook around the last backward) give the parameters of the autograd path."""
    from open_instruct_b200.learner import Learner, LearnerConfig

    extra = {"olmo2": OLMO2, "olmoe": dict(num_experts=4, num_experts_per_tok=2, intermediate_size=48), "llama": {}}[family]
    spec = ModelSpec(**{**BASE, **extra})
    flats = []
    for ops in ("ref", "emulated"):
        ln = Learner(spec, LearnerConfig(ops=ops, learning_rate=1e-2, warmup_steps=0, total_steps=10, max_grad_norm=1.0, seed=4,
                                         load_balancing_weight=0.5 if family == "olmoe" else 0.0), device="cpu")
        for step in range(3):
            for mb in range(2):
                ids, pos, cu, labels, _ = _batch(spec, seed=10 * step + mb)
                batch = {"input_ids": ids, "position_ids": pos, "cu_seq_lens_q": cu, "labels_shifted": labels}
                ln.sft_micro_step(batch, last=mb == 1)
            ln.optimizer_step()
        flats.append(ln.model.flat.detach().clone())
    # Adam divides by the gradient's own scale, so entries whose gradient is rounding noise may move differently: the bound
    # is a small fraction of the distance travelled (three steps of 1e-2)
    assert (flats[0] - flats[1]).abs().max().item() < 1e-3
    start = LlamaModel(spec, ops="ref", seed=4).flat.detach()   # the learner pads its buffer to a multiple of the world size
    assert (flats[0][: start.numel()] - start).abs().max().item() > 1e-2  # it trained


def test_lora_on_the_emulated_path_follows_the_pytorch_path():
    """Adapter training contracts ``dL/dW_eff`` from the fused path's fp32 gradient buffer; same adapters as from autograd."""
    from open_instruct_b200.learner import Learner, LearnerConfig
    from open_instruct_b200.models.lora import LoRATrainer

    spec = ModelSpec(**BASE)
    got = []
    for ops in ("ref", "emulated"):
        ln = Learner(spec, LearnerConfig(ops=ops, seed=4), device="cpu")
        tr = LoRATrainer(ln, rank=4, alpha=8.0, lr=1e-2)
        for step in range(3):
            mbs = []
            for mb in range(2):
                ids, pos, cu, labels, _ = _batch(spec, seed=10 * step + mb)
                mbs.append({"input_ids": ids, "position_ids": pos, "cu_seq_lens_q": cu, "labels_shifted": labels})
            out = tr.step(mbs)
        got.append((tr.adapters.flat.detach().clone(), ln.model.flat.detach().clone(), float(out["loss"])))
    assert abs(got[0][2] - got[1][2]) < 1e-4
    assert (got[0][0] - got[1][0]).abs().max().item() < 1e-3
    assert (got[0][1] - got[1][1]).abs().max().item() < 1e-3
    assert got[0][0].abs().max().item() > 1e-2


def test_grpo_step_on_the_emulated_path_follows_the_pytorch_path():
    """``grpo_train_step`` (old / new log-probs, clipped ratio, token-level normalisation, entropy) through the hand-driven path."""
    from open_instruct_b200.data_types import CollatedBatchData
    from open_instruct_b200.grpo_fast import grpo_train_step
    from open_instruct_b200.grpo_utils import GRPOExperimentConfig
    from open_instruct_b200.learner import Learner, LearnerConfig
    from open_instruct_b200.rl_utils import pack_sequences

    spec = ModelSpec(**BASE)
    q = [[5, 6, 7, 8]] * 4
    r = [[10, 11, 12], [20, 21, 22, 23], [30, 31], [40, 41, 42]]
    lp = [[-1.0] * len(x) for x in r]
    args = GRPOExperimentConfig(beta=0.0, load_ref_policy=False, use_rho_correction=False, record_entropy=True)
    args.temperature = 0.8   # copied from the sampling configuration by the trainer's main()
    outs = []
    for ops in ("ref", "emulated"):
        p = pack_sequences(q, r, [[1] * len(x) for x in r], 64, 0, lp)
        adv = torch.tensor([0.0, 1.0, -1.0, 0.5, -0.5])
        p.advantages = [adv[m.long()] for m in p.response_masks]
        data = CollatedBatchData(p.query_responses, p.attention_masks, p.position_ids, p.advantages, p.response_masks, p.vllm_logprobs, p.cu_seqlens)
        ln = Learner(spec, LearnerConfig(ops=ops, learning_rate=5e-3, lr_scheduler_type="constant", seed=2), device="cpu")
        metrics = [grpo_train_step(ln, data, args) for _ in range(2)]
        outs.append((ln.model.flat.detach().clone(), metrics[-1]))
    (w0, m0), (w1, m1) = outs
    assert (w0 - w1).abs().max().item() < 1e-3
    for k in ("loss/total_avg", "policy/entropy_avg", "val/ratio"):
        if k in m0:
            assert abs(float(m0[k]) - float(m1[k])) < 1e-4, (k, m0[k], m1[k])


@pytest.mark.parametrize("forward", ["concatenated", "separate"])
def test_dpo_forward_and_gradient_on_the_emulated_path(forward):
    """The preference trainer's two forward forms through the hand-driven path: same sequence log-probs and, after a DPO loss,
    the same gradient as autograd over the PyTorch path."""
    from open_instruct_b200.data.collate import TensorDataCollatorWithFlatteningDPO
    from open_instruct_b200.data.synthetic import dpo_pairs
    from open_instruct_b200.dpo_utils import concatenated_forward, dpo_loss, separate_forward
    from open_instruct_b200.learner import Learner, LearnerConfig

    spec = ModelSpec(**BASE)
    rows = dpo_pairs(3, spec.vocab_size, seed=0, max_len=200)
    for r in rows:
        for k in list(r):
            if k.endswith("input_ids") or k.endswith("labels"):
                r[k] = r[k][:60]
    batch = TensorDataCollatorWithFlatteningDPO()(rows)
    fn = concatenated_forward if forward == "concatenated" else separate_forward
    got = []
    for ops in ("ref", "emulated"):
        ln = Learner(spec, LearnerConfig(ops=ops, seed=3), device="cpu")
        pc, pr, _ = fn(ln, batch, average_log_prob=True)
        losses, _, _ = dpo_loss(pc, pr, torch.zeros_like(pc), torch.zeros_like(pr), beta=0.5)
        ln.backward(losses.mean(), last=True)
        got.append((pc.detach(), pr.detach(), ln.model.grad_flat().clone()))
    assert torch.allclose(got[0][0], got[1][0], atol=1e-5) and torch.allclose(got[0][1], got[1][1], atol=1e-5)
    assert (got[0][2] - got[1][2]).abs().max().item() < 1e-5 * max(1.0, got[0][2].abs().max().item())
