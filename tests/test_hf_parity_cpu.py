"""Logit parity with the Hugging Face implementations, family by family: a small random model built by transformers is saved,
read back through this package's checkpoint reader into the PyTorch path, and must give the same logits; the export goes the other
way.  Families: Llama (plain, Llama-3.1 frequency-dependent RoPE scaling, tied embeddings), Qwen2 (q/k/v bias), Qwen3 (per-head q/k
norm), Mistral, OLMo-2 and OLMo-3 (norm after the sub-layer, q/k norm over all heads)."""
import tempfile

import pytest
import torch

transformers = pytest.importorskip("transformers")

BASE = dict(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
            max_position_embeddings=256)
LLAMA3_SCALING = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 64}
FAMILIES = {
    "llama": ("Llama", dict(rope_theta=500000.0)),
    "llama3.1-rope-scaling": ("Llama", dict(rope_theta=500000.0, rope_scaling=LLAMA3_SCALING)),
    "llama-tied": ("Llama", dict(tie_word_embeddings=True)),
    "llama-yarn": ("Llama", dict(rope_theta=10000.0, rope_scaling={"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32})),
    "olmo3-yarn-with-attention-factor": ("Olmo3", dict(sliding_window=16, num_hidden_layers=4, rope_scaling={
        "rope_type": "yarn", "factor": 8.0, "original_max_position_embeddings": 32, "attention_factor": 1.2079441541679836, "beta_fast": 32, "beta_slow": 1})),
    "qwen2": ("Qwen2", {}),
    "qwen3": ("Qwen3", dict(head_dim=32)),
    "qwen2-windowed-upper-layers": ("Qwen2", dict(num_hidden_layers=4, use_sliding_window=True, sliding_window=16, max_window_layers=2)),
    "mistral": ("Mistral", dict(sliding_window=None)),
    "olmo2": ("Olmo2", {}),
    "olmo3": ("Olmo3", dict(sliding_window=4096)),
    "olmo3-window-shorter-than-the-text": ("Olmo3", dict(sliding_window=16, num_hidden_layers=4)),
    "mistral-window-shorter-than-the-text": ("Mistral", dict(sliding_window=16)),
    "olmo-hybrid": ("OlmoHybrid", dict(num_hidden_layers=4, pad_token_id=0, eos_token_id=1, rope_parameters={"rope_type": "default", "rope_theta": 10000.0})),
    "olmo-hybrid-grouped-key-heads": ("OlmoHybrid", dict(num_hidden_layers=4, pad_token_id=0, eos_token_id=1, linear_num_key_heads=2, linear_num_value_heads=4,
                                                         linear_key_head_dim=8, linear_value_head_dim=16, layer_types=["linear_attention", "full_attention", "linear_attention", "full_attention"])),
    "olmo-hybrid-no-rope": ("OlmoHybrid", dict(num_hidden_layers=4, pad_token_id=0, eos_token_id=1, rope_parameters={"rope_type": "default", "rope_theta": None})),
    "olmoe": ("Olmoe", dict(intermediate_size=96, num_key_value_heads=4, num_experts=4, num_experts_per_tok=2)),
}


def _hf_model(cls_name, extra):
    if not hasattr(transformers, cls_name + "ForCausalLM"):
        pytest.skip(f"transformers has no {cls_name}")
    torch.manual_seed(0)
    cfg = getattr(transformers, cls_name + "Config")(**{**BASE, **extra})
    m = getattr(transformers, cls_name + "ForCausalLM")(cfg).eval().float()
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() == 1:
                p.uniform_(0.5, 1.5)  # norm weights and biases away from their trivial initialisation
    return m, cfg


def _our_logits(model, ids):
    B, L = ids.shape
    pos = torch.arange(L).repeat(B)
    cu = torch.arange(0, (B + 1) * L, L, dtype=torch.int32)
    with torch.no_grad():
        return model.logits(ids.reshape(-1), pos, cu).reshape(B, L, -1)


@pytest.mark.parametrize("family", list(FAMILIES))
def test_checkpoint_import_gives_hf_logits(family):
    from open_instruct_b200.ckpt.hf_io import load_hf_checkpoint
    from open_instruct_b200.models import LlamaModel
    from open_instruct_b200.models.spec import ModelSpec

    cls_name, extra = FAMILIES[family]
    hf, cfg = _hf_model(cls_name, extra)
    with tempfile.TemporaryDirectory() as d:
        hf.save_pretrained(d, safe_serialization=True)
        spec = ModelSpec.from_pretrained(d)
        ours = LlamaModel(spec, device="cpu", dtype=torch.float32, ops="ref")
        load_hf_checkpoint(d, ours.flat.detach(), spec, strict=True)
    ids = torch.randint(0, cfg.vocab_size, (2, 40), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf(ids).logits
    assert (_our_logits(ours, ids) - want).abs().max().item() < 1e-5


@pytest.mark.parametrize("family", ["llama3.1-rope-scaling", "qwen3", "olmo2", "olmoe", "olmo-hybrid", "olmo-hybrid-no-rope", "olmo3-window-shorter-than-the-text",
                                    "mistral-window-shorter-than-the-text", "llama-yarn", "qwen2-windowed-upper-layers"])
def test_checkpoint_export_is_read_by_hf(family):
    from open_instruct_b200.ckpt.hf_io import save_hf_checkpoint
    from open_instruct_b200.models import LlamaModel
    from open_instruct_b200.models.spec import ModelSpec

    cls_name, extra = FAMILIES[family]
    _, cfg = _hf_model(cls_name, extra)
    with tempfile.TemporaryDirectory() as d0:
        cfg.save_pretrained(d0)
        spec = ModelSpec.from_pretrained(d0)
    ours = LlamaModel(spec, device="cpu", dtype=torch.float32, ops="ref", seed=3)
    with tempfile.TemporaryDirectory() as d:
        save_hf_checkpoint(ours.flat.detach(), spec, d, dtype=torch.float32)
        hf = transformers.AutoModelForCausalLM.from_pretrained(d, torch_dtype=torch.float32).eval()
    ids = torch.randint(0, spec.vocab_size, (2, 33), generator=torch.Generator().manual_seed(2))
    with torch.no_grad():
        got = hf(ids).logits
    assert (got - _our_logits(ours, ids)).abs().max().item() < 1e-5


@pytest.mark.parametrize("family", ["olmo2", "olmo3-window-shorter-than-the-text", "olmo3-yarn-with-attention-factor", "olmo-hybrid", "olmo-hybrid-no-rope", "olmo-hybrid-grouped-key-heads"])
def test_engine_generates_with_a_post_norm_model(family):
    """The rollout engine's PyTorch path follows the block structure (the sliding-window layers, with a prompt longer than the
    window; the gated-DeltaNet layers, whose recurrent state it keeps per sequence) too: greedy tokens equal argmax decoding
    with the HF model."""
    from open_instruct_b200.ckpt.hf_io import load_hf_checkpoint
    from open_instruct_b200.data_types import SamplingConfig
    from open_instruct_b200.models.spec import ModelSpec
    from open_instruct_b200.rollout.engine import RolloutEngine

    hf, cfg = _hf_model(*FAMILIES[family])
    with tempfile.TemporaryDirectory() as d:
        hf.save_pretrained(d, safe_serialization=True)
        spec = ModelSpec.from_pretrained(d).replace(eos_token_id=None)
        eng = RolloutEngine(spec, device="cpu", ops="auto", num_blocks=32)
        load_hf_checkpoint(d, eng.model.flat.detach(), spec)
    prompt = torch.randint(0, cfg.vocab_size, (70,), generator=torch.Generator().manual_seed(4)).tolist()
    outs = eng.generate([prompt, prompt[:33]], SamplingConfig(temperature=0.0, max_tokens=6, n=2))   # the samples share their prompt pass
    for res, pr in zip(outs, (prompt, prompt[:33])):
        ids = list(pr)
        with torch.no_grad():
            for _ in range(6):
                ids.append(int(hf(torch.tensor([ids])).logits[0, -1].argmax()))
        assert res.responses == [ids[len(pr):]] * 2
    assert eng._gdn_state == {}   # per-sequence recurrent state is dropped with the sequence


@pytest.mark.parametrize("family", ["llama", "qwen2", "qwen3", "olmo2", "olmo3", "olmoe", "olmo-hybrid"])
def test_reward_model_export_is_read_by_hf_sequence_classification(family):
    """The reward-model folder loads with ``AutoModelForSequenceClassification`` and scores like this package's ``get_reward``."""
    from open_instruct_b200.models import LlamaModel
    from open_instruct_b200.models.spec import ModelSpec
    import open_instruct_b200.olmo_adapter  # noqa: F401  (registers the OLMo families' sequence-classification classes)
    from open_instruct_b200.reward_modeling import load_score_weight, save_reward_model

    cls_name, extra = FAMILIES[family]
    _, cfg = _hf_model(cls_name, extra)
    with tempfile.TemporaryDirectory() as d0:
        cfg.save_pretrained(d0)
        spec = ModelSpec.from_pretrained(d0).replace(pad_token_id=0)
    ours = LlamaModel(spec, device="cpu", dtype=torch.float32, ops="ref", seed=5)
    score = torch.randn(1, spec.hidden_size, generator=torch.Generator().manual_seed(6)) * 0.1
    with tempfile.TemporaryDirectory() as d:
        save_reward_model(ours.flat.detach(), score, spec, d, dtype=torch.float32)
        assert torch.equal(load_score_weight(d), score)
        hf = transformers.AutoModelForSequenceClassification.from_pretrained(d, torch_dtype=torch.float32).eval()
    assert type(hf).__name__ == cls_name + "ForSequenceClassification"
    ids = torch.randint(1, spec.vocab_size, (1, 29), generator=torch.Generator().manual_seed(7))
    with torch.no_grad():
        want = hf(ids).logits.reshape(-1)
        h = ours.hidden_states(ids.reshape(-1), torch.arange(29), torch.tensor([0, 29], dtype=torch.int32))
        got = (h[-1:].float() @ score.t()).reshape(-1)
    assert (got - want).abs().max().item() < 1e-5


@pytest.mark.parametrize("kind", ["linear", "cosine", "constant", "constant_with_warmup", "polynomial", "cosine_with_restarts"])
def test_learning_rate_schedules_equal_transformers(kind):
    """Every schedule name the trainers accept gives the multipliers of ``transformers.get_scheduler`` step by step."""
    from open_instruct_b200.parallel.zero import lr_at

    p = torch.nn.Parameter(torch.zeros(1))
    opt = torch.optim.SGD([p], lr=1.0)
    sch = transformers.get_scheduler(kind, opt, num_warmup_steps=10, num_training_steps=100)
    for step in range(100):
        assert abs(opt.param_groups[0]["lr"] - lr_at(step, 1.0, 100, 10, kind)) < 1e-12, step
        opt.step()
        sch.step()


def test_mixture_of_experts_aux_loss_and_per_expert_checkpoints():
    """OLMoE: the load-balancing loss of a forward equals transformers' ``load_balancing_loss_func`` on the routers' raw logits
    (the installed transformers feeds that function already-softmaxed values, so its own ``aux_loss`` applies the softmax
    twice; the definition - and this package - applies it once); a checkpoint that stores one tensor per expert (the spelling
    older exports use) loads to the same model as the stacked form."""
    from safetensors.torch import load_file, save_file

    from open_instruct_b200.ckpt.hf_io import load_hf_checkpoint
    from open_instruct_b200.models import LlamaModel
    from open_instruct_b200.models.spec import ModelSpec

    hf, cfg = _hf_model(*FAMILIES["olmoe"])
    ids = torch.randint(0, cfg.vocab_size, (2, 40), generator=torch.Generator().manual_seed(1))
    raw = []
    hooks = [layer.mlp.gate.register_forward_pre_hook(lambda mod, args: raw.append(torch.nn.functional.linear(args[0].reshape(-1, args[0].shape[-1]), mod.weight)))
             for layer in hf.model.layers]
    with torch.no_grad():
        want = hf(ids)
    for h in hooks:
        h.remove()
    from transformers.models.olmoe.modeling_olmoe import load_balancing_loss_func

    want_aux = float(load_balancing_loss_func(tuple(raw), 4, 2))
    with tempfile.TemporaryDirectory() as d:
        hf.save_pretrained(d, safe_serialization=True)
        spec = ModelSpec.from_pretrained(d)
        assert spec.num_experts == 4 and spec.num_experts_per_tok == 2 and spec.qk_norm_full and not spec.post_norm
        ours = LlamaModel(spec, device="cpu", dtype=torch.float32, ops="ref")
        load_hf_checkpoint(d, ours.flat.detach(), spec, strict=True)
        # rewrite the weight file with one tensor per expert
        import os

        sd = load_file(os.path.join(d, "model.safetensors"))
        per = {}
        for k, t in sd.items():
            if k.endswith("experts.gate_up_proj"):
                for e in range(t.shape[0]):
                    g, u = t[e].chunk(2, dim=0)
                    per[k.replace("gate_up_proj", f"{e}.gate_proj.weight")] = g.contiguous()
                    per[k.replace("gate_up_proj", f"{e}.up_proj.weight")] = u.contiguous()
            elif k.endswith("experts.down_proj"):
                for e in range(t.shape[0]):
                    per[k.replace("down_proj", f"{e}.down_proj.weight")] = t[e].contiguous()
            else:
                per[k] = t
        save_file(per, os.path.join(d, "model.safetensors"), metadata={"format": "pt"})
        other = LlamaModel(spec, device="cpu", dtype=torch.float32, ops="ref", seed=9)
        load_hf_checkpoint(d, other.flat.detach(), spec, strict=True)
    assert torch.equal(other.flat.detach()[: ours.layout.total], ours.flat.detach()[: ours.layout.total])
    got = _our_logits(ours, ids)
    assert (got - want.logits).abs().max().item() < 1e-5
    assert abs(float(ours.aux_loss) - want_aux) < 1e-5


def test_sft_on_a_mixture_of_experts_model_with_the_balancing_loss():
    from open_instruct_b200.data.collate import to_device
    from open_instruct_b200.data.synthetic import sft_step_batches
    from open_instruct_b200.learner import Learner, LearnerConfig
    from open_instruct_b200.models.spec import ModelSpec

    spec = ModelSpec(vocab_size=256, hidden_size=64, intermediate_size=96, num_layers=2, num_heads=4, num_kv_heads=4, head_dim=16, rope_theta=1e4,
                     max_position_embeddings=512, model_type="olmoe", qk_norm=True, qk_norm_full=True, num_experts=4, num_experts_per_tok=2)
    lr = Learner(spec, LearnerConfig(ops="auto", learning_rate=3e-3, lr_scheduler_type="constant", load_balancing_weight=0.5), device="cpu")
    assert lr.ops == "ref"
    mbs = [to_device(b, "cpu") for b in sft_step_batches(2, 96, spec.vocab_size, seed=0)]
    losses = [float(lr.sft_step(mbs)["loss"]) for _ in range(8)]
    assert losses[-1] < losses[0] - 0.3                       # the same batch is learned
    assert 0.9 < float(lr.last_aux_loss) < 4.0                # 1.0 = perfectly balanced routing, num_experts = collapsed
    g = lr.model.layout.view(lr.opt.m, "l0.router") if hasattr(lr.opt, "m") and lr.world == 1 else None
    assert g is None or float(g.abs().sum()) > 0              # the router itself is trained


@pytest.mark.parametrize("window", [None, 7])
def test_fused_attention_branch_of_the_pytorch_path_equals_the_explicit_softmax(window):
    """Models that only run on the PyTorch path use PyTorch's fused attention for half-precision GPU tensors; the branch is forced
    here on CPU and must agree with the explicit-softmax statement, values and gradients, for packed documents with grouped heads."""
    from open_instruct_b200.ops import ref

    torch.manual_seed(0)
    Hq, Hkv, Dh = 4, 2, 16
    qkv = torch.randn(50, (Hq + 2 * Hkv) * Dh, requires_grad=True)
    cu = torch.tensor([0, 20, 21, 50], dtype=torch.int32)
    a = ref.attention_varlen(qkv, cu, Hq, Hkv, Dh, window=window)
    if window:  # the window changes the result for the documents longer than it
        assert (a - ref.attention_varlen(qkv, cu, Hq, Hkv, Dh)).abs().max().item() > 1e-3
    ga, = torch.autograd.grad(a.square().sum(), qkv)
    ref._FORCE_SDPA = True
    try:
        b = ref.attention_varlen(qkv, cu, Hq, Hkv, Dh, window=window)
        gb, = torch.autograd.grad(b.square().sum(), qkv)
    finally:
        ref._FORCE_SDPA = False
    assert (a - b).abs().max().item() < 1e-5 and (ga - gb).abs().max().item() < 1e-4


@pytest.mark.parametrize("cls_name", ["Olmo2", "Qwen3", "OlmoHybrid"])
def test_sft_starts_from_a_hugging_face_folder_and_exports_the_same_architecture(tmp_path, cls_name):
    """``model_name_or_path`` pointing at a transformers checkpoint: the trainer reads the architecture and the weights from it,
    and its export loads as the same transformers class.  With a zero learning rate the exported model gives the source
    model's logits (up to the bf16 the export is written in)."""
    import os

    from open_instruct_b200.finetune import main
    from test_finetune_cpu import _args

    hf, cfg = _hf_model(cls_name, dict(vocab_size=600, **(FAMILIES["olmo-hybrid"][1] if cls_name == "OlmoHybrid" else {})))
    src = os.path.join(str(tmp_path), "hf")
    hf.save_pretrained(src, safe_serialization=True)
    args, tc = _args(str(tmp_path), model_name_or_path=src, num_train_epochs=1, learning_rate=0.0)
    main(args, tc)
    back = transformers.AutoModelForCausalLM.from_pretrained(args.output_dir, dtype=torch.float32).eval()
    assert type(back) is type(hf)
    ids = torch.randint(0, 300, (2, 20), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        assert (back(ids).logits - hf(ids).logits).abs().max().item() < 0.03


def test_gated_delta_rule_in_chunks_equals_the_token_by_token_recurrence():
    """Outputs, final state and every input gradient; a chunk length that does not divide the sequence."""
    from open_instruct_b200.models import gdn

    g0 = torch.Generator().manual_seed(0)
    L, H, dk, dv = 150, 3, 8, 16
    q = torch.randn(L, H, dk, generator=g0)
    k = gdn._l2norm(torch.randn(L, H, dk, generator=g0))
    v = torch.randn(L, H, dv, generator=g0)
    g = -torch.rand(L, H, generator=g0) * 0.5
    beta = torch.rand(L, H, generator=g0) * 2
    s0 = torch.randn(H, dk, dv, generator=g0) * 0.1
    args = [t.requires_grad_(True) for t in (q, k, v, g, beta, s0)]
    o1, S1 = gdn.gated_delta_rule_sequential(*args)
    o2, S2 = gdn.gated_delta_rule(*args, chunk=32)
    assert (o1 - o2).abs().max().item() < 1e-4 and (S1 - S2).abs().max().item() < 1e-4
    w, ws = torch.randn(o1.shape, generator=g0), torch.randn(S1.shape, generator=g0)
    for a, b in zip(torch.autograd.grad((o1 * w).sum() + (S1 * ws).sum(), args), torch.autograd.grad((o2 * w).sum() + (S2 * ws).sum(), args)):
        assert (a - b).abs().max().item() < 2e-4 * max(1.0, a.abs().max().item())


def test_hybrid_layers_do_not_leak_across_packed_documents():
    """Two documents packed into one row give the logits of each document run alone (state and convolution restart)."""
    from open_instruct_b200.models import LlamaModel, get_spec

    spec = get_spec("olmo-hybrid-7b").replace(vocab_size=300, hidden_size=64, intermediate_size=128, num_layers=4, num_heads=4, num_kv_heads=2,
                                              head_dim=16, layer_types=("gdn", "gdn", "gdn", "attention"), gdn_key_heads=2, gdn_value_heads=4,
                                              gdn_key_dim=12, gdn_value_dim=24)
    m = LlamaModel(spec, ops="ref", seed=2)
    ids = torch.randint(0, 300, (100,), generator=torch.Generator().manual_seed(1))
    packed = m.logits(ids, torch.cat([torch.arange(70), torch.arange(30)]), torch.tensor([0, 70, 100], dtype=torch.int32))
    alone = m.logits(ids[70:], torch.arange(30), torch.tensor([0, 30], dtype=torch.int32))
    assert (packed[70:] - alone).abs().max().item() < 1e-5
    assert (packed[:70] - m.logits(ids[:70], torch.arange(70), torch.tensor([0, 70], dtype=torch.int32))).abs().max().item() < 1e-5


def test_qwen2_windowed_upper_layers_equal_transformers():
    """Qwen2 with ``use_sliding_window``: the layers from ``max_window_layers`` up are windowed, the lower ones attend to everything."""
    from open_instruct_b200.ckpt.hf_io import load_hf_checkpoint
    from open_instruct_b200.models import LlamaModel
    from open_instruct_b200.models.spec import ModelSpec

    hf, cfg = _hf_model("Qwen2", dict(num_hidden_layers=4, use_sliding_window=True, sliding_window=16, max_window_layers=2))
    with tempfile.TemporaryDirectory() as d:
        hf.save_pretrained(d, safe_serialization=True)
        spec = ModelSpec.from_pretrained(d)
        assert spec.layer_types == ("attention", "attention", "sliding", "sliding") and spec.sliding_window == 16
        ours = LlamaModel(spec, device="cpu", dtype=torch.float32, ops="ref")
        load_hf_checkpoint(d, ours.flat.detach(), spec, strict=True)
    ids = torch.randint(0, cfg.vocab_size, (2, 40), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf(ids).logits
    assert (_our_logits(ours, ids) - want).abs().max().item() < 1e-5
    assert ModelSpec.from_hf_config({**cfg.to_dict(), "use_sliding_window": False}).sliding_window is None
