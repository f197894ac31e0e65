"""DPO: loss math against hand-computed values, packed forward vs per-sequence forward, end-to-end run."""

import json
import math
import os

import torch

from helpers import make_pref_jsonl, make_tokenizer


def test_dpo_loss_values():
    from open_instruct_b200.dpo_utils import dpo_loss, simpo_loss, wpo_loss

    pc, pr = torch.tensor([-1.0, -2.0]), torch.tensor([-2.0, -1.5])
    rc, rr = torch.tensor([-1.5, -2.0]), torch.tensor([-1.5, -2.0])
    losses, cr, rj = dpo_loss(pc, pr, rc, rr, beta=0.5)
    z = (pc - pr) - (rc - rr)
    expect = -torch.nn.functional.logsigmoid(0.5 * z)
    assert torch.allclose(losses, expect)
    assert torch.allclose(cr, 0.5 * (pc - rc)) and torch.allclose(rj, 0.5 * (pr - rr))
    ls, _, _ = dpo_loss(pc, pr, rc, rr, beta=0.5, label_smoothing=0.1)
    assert torch.allclose(ls, 0.9 * expect - 0.1 * torch.nn.functional.logsigmoid(-0.5 * z))
    sl, _, _ = simpo_loss(pc, pr, beta=2.0, gamma_beta_ratio=0.3)
    assert torch.allclose(sl, -torch.nn.functional.logsigmoid(2.0 * (pc - pr - 0.3)))
    wl, _, _ = wpo_loss(pc, pr, rc, rr, beta=0.5)
    w = torch.clamp(torch.exp(pc + pr), max=1)
    assert torch.allclose(wl, expect * w)


def test_concatenated_forward_matches_separate():
    from open_instruct_b200.data.collate import TensorDataCollatorWithFlatteningDPO
    from open_instruct_b200.data.synthetic import dpo_pairs
    from open_instruct_b200.dpo_utils import concatenated_forward, separate_forward
    from open_instruct_b200.learner import Learner, LearnerConfig
    from open_instruct_b200.models import get_spec

    spec = get_spec("tiny")
    learner = Learner(spec, LearnerConfig(ops="ref"))
    rows = dpo_pairs(3, spec.vocab_size, seed=0, max_len=200)
    for r in rows:
        for k in list(r):
            if k.endswith("input_ids") or k.endswith("labels"):
                r[k] = r[k][:60]
    batch = TensorDataCollatorWithFlatteningDPO()(rows)
    for avg in (False, True):
        c1, r1, aux1 = concatenated_forward(learner, batch, average_log_prob=avg)
        c2, r2, aux2 = separate_forward(learner, batch, average_log_prob=avg)
        assert torch.allclose(c1, c2, atol=1e-4) and torch.allclose(r1, r2, atol=1e-4)
        assert torch.equal(aux1["chosen_tokens"], aux2["chosen_tokens"])
    # against a per-sequence loop
    ids = rows[0]["chosen_input_ids"]
    lab = rows[0]["chosen_labels"]
    logits = learner.model.logits(ids, torch.arange(len(ids)), torch.tensor([0, len(ids)], dtype=torch.int32))
    lp = torch.log_softmax(logits[:-1].float(), -1).gather(-1, ids[1:, None]).squeeze(-1)
    mask = lab[1:] != -100
    c_sum, _, _ = concatenated_forward(learner, batch, average_log_prob=False)
    assert abs((lp * mask).sum().item() - c_sum[0].item()) < 1e-3


def test_dpo_end_to_end(tmp_path, monkeypatch):
    import open_instruct_b200.dpo_tune_cache as dtc
    import open_instruct_b200.dpo_utils as du
    from open_instruct_b200.data.tokenize import TokenizerConfig

    tmp = str(tmp_path)
    monkeypatch.setattr(dtc, "REFERENCE_LOGPROBS_CACHE_PATH", os.path.join(tmp, "refcache"))
    tok = make_tokenizer(os.path.join(tmp, "tok"))
    data = make_pref_jsonl(os.path.join(tmp, "pref.jsonl"))
    args = du.DPOExperimentConfig(model_name_or_path="tiny", mixer_list=[data, "1.0"], max_seq_length=96,
                                  per_device_train_batch_size=4, gradient_accumulation_steps=2, learning_rate=2e-3, num_epochs=3,
                                  output_dir=os.path.join(tmp, "out"), local_cache_dir=os.path.join(tmp, "cache"), beta=0.5,
                                  loss_type="dpo_norm", checkpointing_steps=1000, ops="ref", seed=1, warmup_ratio=0.0)
    tc = TokenizerConfig(tokenizer_name_or_path=tok, chat_template_name="tulu")
    out = dtc.main(args, tc)
    lines = [json.loads(l) for l in open(os.path.join(args.output_dir, "metrics.jsonl"))]
    assert abs(lines[0]["train_loss"] - math.log(2)) < 0.05  # policy == reference at step 0
    assert lines[-1]["train_loss"] < lines[0]["train_loss"]
    assert lines[-1]["rewards/accuracy"] >= 0.5
    assert len(os.listdir(os.path.join(tmp, "refcache"))) == 1
    assert os.path.exists(os.path.join(args.output_dir, "model.safetensors"))


def test_dpo_with_lora_adapters(tmp_path, monkeypatch):
    """``use_lora``: the base weights stay what they were (they are the reference policy too), only the adapters learn; the output
    folder holds the merged model and the adapter files; a checkpoint carries the adapter state."""
    import torch

    import open_instruct_b200.dpo_tune_cache as dtc
    import open_instruct_b200.dpo_utils as du
    from open_instruct_b200.ckpt.hf_io import load_hf_checkpoint
    from open_instruct_b200.data.tokenize import TokenizerConfig
    from open_instruct_b200.models import LlamaModel, get_spec

    tmp = str(tmp_path)
    monkeypatch.setattr(dtc, "REFERENCE_LOGPROBS_CACHE_PATH", os.path.join(tmp, "refcache"))
    tok = make_tokenizer(os.path.join(tmp, "tok"))
    data = make_pref_jsonl(os.path.join(tmp, "pref.jsonl"))
    args = du.DPOExperimentConfig(model_name_or_path="tiny", mixer_list=[data, "1.0"], max_seq_length=96, per_device_train_batch_size=4,
                                  gradient_accumulation_steps=2, learning_rate=1e-2, num_epochs=3, output_dir=os.path.join(tmp, "out"),
                                  local_cache_dir=os.path.join(tmp, "cache"), beta=0.5, loss_type="dpo_norm", checkpointing_steps=2, ops="ref",
                                  seed=1, warmup_ratio=0.0, use_lora=True, lora_rank=4, lora_alpha=8, lora_dropout=0.0, max_grad_norm=1.0)
    out = dtc.main(args, TokenizerConfig(tokenizer_name_or_path=tok, chat_template_name="tulu"))
    lines = [json.loads(l) for l in open(os.path.join(args.output_dir, "metrics.jsonl"))]
    assert abs(lines[0]["train_loss"] - math.log(2)) < 0.05 and lines[-1]["train_loss"] < lines[0]["train_loss"]
    assert os.path.exists(os.path.join(args.output_dir, "adapter", "adapter_config.json"))
    kept = sorted(d for d in os.listdir(args.output_dir) if d.startswith("step_"))
    assert kept and all(os.path.exists(os.path.join(args.output_dir, d, "lora_state.pt")) for d in kept)
    # merged weights = base + low-rank update: embeddings and norms (not adapted) are the base's, the projections moved by a rank <= 4 matrix
    spec = get_spec("tiny")
    base = LlamaModel(spec, ops="ref", seed=args.seed)
    tuned = LlamaModel(spec, ops="ref", seed=args.seed)
    load_hf_checkpoint(args.output_dir, tuned.flat.detach(), spec)
    b, t = base.layout.views(base.flat.detach()), tuned.layout.views(tuned.flat.detach())
    assert (b["embed"] - t["embed"]).abs().max().item() < 4e-3 and (b["final_norm"] - t["final_norm"]).abs().max().item() < 4e-3   # bf16 export
    delta = (t["l0.wo"] - b["l0.wo"]).float()
    sv = torch.linalg.svdvals(delta)
    assert sv[0] > 0.05 and sv[4] < 0.02 * sv[0]
