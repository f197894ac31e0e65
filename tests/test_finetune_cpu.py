"""End-to-end SFT on CPU: tokenise -> train -> checkpoint -> resume -> HF export."""

import json
import os

import torch

from helpers import make_sft_jsonl, make_tokenizer


def _args(tmp, **kw):
    from open_instruct_b200.data.tokenize import TokenizerConfig
    from open_instruct_b200.finetune import FlatArguments

    tok = make_tokenizer(os.path.join(tmp, "tok"))
    data = make_sft_jsonl(os.path.join(tmp, "sft.jsonl"))
    base = dict(model_name_or_path="tiny", dataset_mixer_list=[data, "1.0"], max_seq_length=128, per_device_train_batch_size=4,
                gradient_accumulation_steps=2, learning_rate=1e-3, num_train_epochs=2, output_dir=os.path.join(tmp, "out"),
                dataset_local_cache_dir=os.path.join(tmp, "cache"), logging_steps=1, lr_scheduler_type="linear", seed=0,
                clean_checkpoints_at_end=False, ops="ref")
    base.update(kw)
    return FlatArguments(**base), TokenizerConfig(tokenizer_name_or_path=tok, chat_template_name="tulu")


def test_sft_trains_and_exports(tmp_path):
    from open_instruct_b200.ckpt.hf_io import load_hf_checkpoint
    from open_instruct_b200.finetune import main
    from open_instruct_b200.models import LlamaModel, ModelSpec

    args, tc = _args(str(tmp_path))
    out = main(args, tc)
    lines = [json.loads(l) for l in open(os.path.join(args.output_dir, "metrics.jsonl"))]
    assert lines[-1]["train_loss"] < lines[0]["train_loss"]
    assert out["completed_steps"] == 10
    spec = ModelSpec.from_pretrained(args.output_dir)
    model = LlamaModel(spec, ops="ref")
    load_hf_checkpoint(args.output_dir, model.flat.detach())
    assert os.path.exists(os.path.join(args.output_dir, "model.safetensors"))
    assert os.path.exists(os.path.join(args.output_dir, "tokenizer.json"))


import pytest


@pytest.mark.parametrize("extra", [{}, dict(use_lora=True, lora_rank=4, lora_alpha=8.0, lora_dropout=0.0, learning_rate=5e-3)],
                         ids=["full", "lora"])
def test_resume_is_bitwise_identical(tmp_path, extra):
    """With LoRA the checkpoint must carry the adapters and their AdamW moments: a resume that restarted them from their
    initialisation would still finish, with different weights."""
    from open_instruct_b200.finetune import main
    from safetensors.torch import load_file

    a, tc = _args(str(tmp_path / "a"), checkpointing_steps="4", **extra)
    main(a, tc)
    full = load_file(os.path.join(a.output_dir, "model.safetensors"))
    # interrupted run: stop after 4 steps, then resume in a fresh call
    b, tc_b = _args(str(tmp_path / "b"), checkpointing_steps="4", **extra)
    b1 = type(b)(**{**b.__dict__, "max_train_steps": None})
    import open_instruct_b200.finetune as ft

    first = type(b)(**{**b.__dict__})
    first.max_train_steps = None
    # run the first 4 steps only by capping epochs' steps through max_train_steps on a copy that keeps the schedule
    orig = ft._micro_batches
    calls = {"n": 0}

    def limited(it, accum):
        if calls["n"] >= 4:
            return []
        calls["n"] += 1
        return orig(it, accum)

    ft._micro_batches = limited
    try:
        main(first, tc_b)
    finally:
        ft._micro_batches = orig
    assert os.path.exists(os.path.join(b.output_dir, "step_4", "COMPLETED"))
    if extra:
        assert os.path.exists(os.path.join(b.output_dir, "step_4", "lora_state.pt"))
    main(b, tc_b)
    resumed = load_file(os.path.join(b.output_dir, "model.safetensors"))
    for k in full:
        assert torch.equal(full[k], resumed[k]), k


def test_lora_finetune_trains_adapters_only(tmp_path):
    from safetensors.torch import load_file

    from open_instruct_b200.finetune import main
    from open_instruct_b200.models import LlamaModel, get_spec

    args, tc = _args(str(tmp_path), use_lora=True, lora_rank=4, lora_alpha=8.0, lora_dropout=0.0, learning_rate=5e-3, num_train_epochs=3)
    out = main(args, tc)
    lines = [json.loads(l) for l in open(os.path.join(args.output_dir, "metrics.jsonl"))]
    assert lines[-1]["train_loss"] < lines[0]["train_loss"] and out["completed_steps"] == 15
    ad = load_file(os.path.join(args.output_dir, "adapter", "adapter_model.safetensors"))
    assert any(k.endswith("lora_B.weight") and v.abs().sum() > 0 for k, v in ad.items())
    # embeddings have no adapter: the exported (merged) model keeps the base embedding exactly
    merged = load_file(os.path.join(args.output_dir, "model.safetensors"))
    spec = get_spec("tiny").replace(vocab_size=merged["model.embed_tokens.weight"].shape[0])
    base = LlamaModel(spec, seed=0)
    assert torch.allclose(merged["model.embed_tokens.weight"].float(), base.p["embed"].detach().to(torch.bfloat16).float(), atol=1e-6)
    assert not torch.allclose(merged["model.layers.0.self_attn.q_proj.weight"].float(), base.p["l0.wqkv"][: spec.q_dim].detach().to(torch.bfloat16).float())


def test_nf4_block_quantisation():
    """16 code values per 64-value block scaled by the block's absolute maximum: code values come back exactly, Gaussian weights
    within the format's known error (about 9 % relative), storage is 4.5 bits per weight, odd sizes are padded."""
    from open_instruct_b200.models.nf4 import NF4_CODE, NF4Tensor, dequantize_nf4, quantize_nf4

    torch.manual_seed(0)
    exact = NF4_CODE.repeat(4) * 3.0
    p, a = quantize_nf4(exact)
    assert torch.allclose(dequantize_nf4(p, a, exact.numel()), exact)
    w = torch.randn(301, 199) * 0.02
    q = NF4Tensor(w)
    d = q.dequantize()
    assert d.shape == w.shape and 0.05 < float((d - w).norm() / w.norm()) < 0.12
    assert q.nbytes() / w.numel() < 0.57
    blocks = torch.cat([w.reshape(-1), w.new_zeros((-w.numel()) % 64)]).view(-1, 64)
    assert torch.allclose(d.reshape(-1)[:64].abs().max(), blocks[0].abs().max())      # a block's largest value is exact
    assert torch.equal(q.dequantize(), NF4Tensor(d).dequantize())                     # quantising again changes nothing


def test_qlora_finetune_trains_on_the_quantised_base(tmp_path):
    """``use_qlora``: the model computes with NF4-rounded base weights from the first step, only the adapters are trained, the
    loss goes down, and the frozen copy of the adapted matrices takes a quarter of the bf16 size."""
    from open_instruct_b200.finetune import FlatArguments, main
    from open_instruct_b200.models.lora import QuantizedBase

    args, tc = _args(str(tmp_path), use_qlora=True, lora_rank=4, lora_alpha=8.0, lora_dropout=0.0, learning_rate=5e-3, num_train_epochs=3)
    assert args.use_lora                                   # QLoRA implies LoRA
    out = main(args, tc)
    lines = [json.loads(l) for l in open(os.path.join(args.output_dir, "metrics.jsonl"))]
    assert lines[-1]["train_loss"] < lines[0]["train_loss"] and out["completed_steps"] == 15
    with pytest.raises(ValueError, match="adapter training"):   # 8-bit moments are for the adapters' optimizer only
        FlatArguments(model_name_or_path="tiny", dataset_mixer_list=["x.jsonl", "1.0"], use_8bit_optimizer=True)
    # the quantised base: working weights equal dequantised NF4 before any adapter update
    from open_instruct_b200.learner import Learner, LearnerConfig
    from open_instruct_b200.models import get_spec
    from open_instruct_b200.models.lora import LoRATrainer

    lr = Learner(get_spec("tiny"), LearnerConfig(ops="ref", seed=1), device="cpu")
    before = lr.model.flat.detach().clone()
    tr = LoRATrainer(lr, rank=4, quantize_base=True)
    assert isinstance(tr.base, QuantizedBase)
    v0, v1 = lr.model.layout.views(before), lr.model.layout.views(lr.model.flat.detach())
    assert torch.equal(v1["embed"], v0["embed"]) and not torch.equal(v1["l0.wqkv"], v0["l0.wqkv"])
    assert torch.allclose(v1["l0.wqkv"], tr.base.entry("l0.wqkv"))
    adapted = sum(lr.model.layout.entries[n].numel for n in tr.base.q)
    assert tr.base.nbytes() < 0.3 * adapted * 2


def test_training_state_checkpoint_converts_to_a_hugging_face_folder(tmp_path):
    """A mid-run checkpoint (optimizer shards with the fp32 master weights) becomes an HF folder without the trainer; converting the
    last checkpoint of a run gives the run's own export."""
    from safetensors import safe_open

    from open_instruct_b200.ckpt import convert_state_to_hf
    from open_instruct_b200.finetune import main

    args, tc = _args(str(tmp_path), checkpointing_steps="5", keep_last_n_checkpoints=-1)
    main(args, tc)
    assert os.path.exists(os.path.join(args.output_dir, "step_5", "COMPLETED"))
    out = convert_state_to_hf.main(["--checkpoint-dir", os.path.join(args.output_dir, "step_10"), "--model-name", "tiny",
                                    "--output-dir", str(tmp_path / "hf10"), "--tokenizer-name", tc.tokenizer_name_or_path])
    assert os.path.exists(os.path.join(out, "tokenizer.json")) and os.path.exists(os.path.join(out, "config.json"))
    with safe_open(os.path.join(out, "model.safetensors"), "pt") as a, safe_open(os.path.join(args.output_dir, "model.safetensors"), "pt") as b:
        assert sorted(a.keys()) == sorted(b.keys())
        for k in a.keys():
            assert torch.equal(a.get_tensor(k), b.get_tensor(k)), k
    mid = convert_state_to_hf.main(["--checkpoint-dir", os.path.join(args.output_dir, "step_5"), "--model-name", "tiny",
                                    "--output-dir", str(tmp_path / "hf5")])
    with safe_open(os.path.join(mid, "model.safetensors"), "pt") as a, safe_open(os.path.join(out, "model.safetensors"), "pt") as b:
        assert any(not torch.equal(a.get_tensor(k), b.get_tensor(k)) for k in a.keys())
    os.remove(os.path.join(args.output_dir, "step_5", "COMPLETED"))
    with pytest.raises(RuntimeError, match="COMPLETED"):
        convert_state_to_hf.main(["--checkpoint-dir", os.path.join(args.output_dir, "step_5"), "--model-name", "tiny", "--output-dir", str(tmp_path / "x")])


def test_eight_bit_adamw_follows_the_fp32_one_and_qlora_trains_with_it(tmp_path):
    """Block-wise 8-bit moments: on a least-squares problem the trajectory stays with torch's AdamW; the state is two bytes per
    parameter plus the block scales; ``use_qlora`` + ``use_8bit_optimizer`` trains, checkpoints and resumes."""
    from open_instruct_b200.finetune import main
    from open_instruct_b200.parallel.adam8bit import AdamW8bit, _codebook

    for signed in (True, False):
        cb = _codebook(signed)
        assert cb.numel() == 256 and bool((cb[1:] > cb[:-1]).all()) and cb.max().item() == 1.0 and (cb.min().item() == (-1.0 if signed else 0.0))
    torch.manual_seed(0)
    A, y = torch.randn(300, 40), torch.randn(300)

    def run(cls, **kw):
        w = torch.zeros(40, requires_grad=True)
        opt = cls([w], lr=1e-2, weight_decay=0.01, **kw)
        for _ in range(300):
            opt.zero_grad()
            ((A @ w - y) ** 2).mean().backward()
            opt.step()
        return w.detach(), opt

    w32, _ = run(torch.optim.AdamW)
    w8, opt8 = run(AdamW8bit, block=16)
    assert (w32 - w8).abs().max().item() < 2e-3 and opt8.state_bytes() == 2 * (48 + 4 * 3)      # 40 values -> 3 blocks of 16
    sd = opt8.state_dict()
    again = AdamW8bit([torch.zeros(40, requires_grad=True)], lr=1e-2, block=16)
    again.load_state_dict(sd)
    st = next(iter(again.state.values()))
    assert st["step"] == 300 and torch.equal(st["m"].get(), next(iter(opt8.state.values()))["m"].get())
    args, tc = _args(str(tmp_path), use_qlora=True, use_8bit_optimizer=True, lora_rank=4, lora_alpha=8.0, lora_dropout=0.0, learning_rate=5e-3,
                     num_train_epochs=3, checkpointing_steps="5")
    out = main(args, tc)
    lines = [json.loads(l) for l in open(os.path.join(args.output_dir, "metrics.jsonl"))]
    assert lines[-1]["train_loss"] < lines[0]["train_loss"] and out["completed_steps"] == 15


def test_sft_on_the_emulated_kernel_path_gives_the_pytorch_path_losses(tmp_path):
    """The whole trainer with ``ops: emulated`` (the kernel path's driver, kernels restated in PyTorch): step losses equal ``ops: ref``."""
    from open_instruct_b200.finetune import main

    losses = {}
    for ops in ("ref", "emulated"):
        args, tc = _args(str(tmp_path / ops), ops=ops, num_train_epochs=1)
        main(args, tc)
        losses[ops] = [json.loads(l)["train_loss"] for l in open(os.path.join(args.output_dir, "metrics.jsonl"))]
    assert len(losses["ref"]) == 5 and max(abs(a - b) for a, b in zip(losses["ref"], losses["emulated"])) < 1e-5
