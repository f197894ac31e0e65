"""The callback-driven entry points (``dpo``, ``grpo``): a ``Trainer`` runs a train module and callbacks over the same learner
and actors as the loop-style entry points.  Checked here: the trainer mechanics (hook order, metric reduction, resume),
the token-weighted micro-batch loss of the DPO module, and both entry points end to end on CPU."""

import json
import math
import os

import torch

from helpers import make_pref_jsonl, make_rlvr_jsonl, make_tokenizer


def test_trainer_hook_order_and_metrics():
    from open_instruct_b200.trainer import Callback, TrainModule, Trainer

    events = []

    class Learner_:
        device = torch.device("cpu")
        global_step = 0

        def optimizer_step(self, **kw):
            self.global_step += 1
            events.append("optim")
            return torch.tensor(1.5)

        def lr(self, s=None):
            return 0.1

    class M(TrainModule):
        def train_batch(self, batch, dry_run=False):
            events.append(f"train:{batch}")
            self.record_metric("loss", 2.0 * batch, "mean")
            self.record_metric("tokens", 10, "sum")

    class C(Callback):
        def pre_train(self): events.append("pre_train")
        def pre_step(self, b): events.append(f"pre:{b}")
        def post_step(self): events.append(f"post:{self.trainer.global_step}")
        def post_train(self): events.append("post_train")

    logged = []

    class T:
        def log(self, m, s): logged.append((s, dict(m)))

    tr = Trainer(M(Learner_()), [1, 2], max_steps=3, callbacks=[C()], tracker=T())
    out = tr.fit()
    assert events == ["pre_train", "pre:1", "train:1", "optim", "post:1", "pre:2", "train:2", "optim", "post:2",
                      "pre:1", "train:1", "optim", "post:3", "post_train"]  # the loader is restarted for the next epoch
    assert [s for s, _ in logged] == [1, 2, 3] and logged[1][1]["loss"] == 4.0 and logged[1][1]["tokens"] == 10.0
    assert out["training_step"] == 3 and out["optim/grad_norm"] == 1.5


def test_dpo_module_weights_micro_batches_by_tokens():
    """Two micro-batches of very different size: the step's gradient is sum_k (tokens_k / tokens) * grad(loss_k), and the
    reported loss is the same token-weighted mean (``open_instruct/olmo_core_train_modules.py:236-245``)."""
    from open_instruct_b200.data.collate import TensorDataCollatorWithFlatteningDPO
    from open_instruct_b200.data.synthetic import dpo_pairs
    from open_instruct_b200.dpo_utils import DPOExperimentConfig, compute_loss, concatenated_forward
    from open_instruct_b200.learner import Learner, LearnerConfig
    from open_instruct_b200.models import get_spec
    from open_instruct_b200.train_modules import DPOTrainModule, num_tokens
    from open_instruct_b200.trainer import Trainer

    spec = get_spec("tiny")
    cfg = DPOExperimentConfig(model_name_or_path="tiny", mixer_list=["x", "1.0"], loss_type="simpo", beta=2.0)
    rows = dpo_pairs(5, spec.vocab_size, seed=1, max_len=90)
    for i, r in enumerate(rows):
        for k in list(r):
            if k.endswith(("input_ids", "labels")):
                r[k] = r[k][: (20 if i == 0 else 70)]
    coll = TensorDataCollatorWithFlatteningDPO()
    micro = [coll(rows[:1]), coll(rows[1:])]
    learner = Learner(spec, LearnerConfig(ops="ref", learning_rate=0.0, seed=0))
    module = DPOTrainModule(learner, cfg, None, concatenated_forward)
    tr = Trainer(module, [micro], max_steps=1)
    module.train_batch(micro)
    got = learner.model.grad_flat().clone()
    learner.model.zero_grad()
    toks = [num_tokens(m) for m in micro]
    want_loss = 0.0
    for m, t in zip(micro, toks):
        pc, pr, aux = concatenated_forward(learner, m, average_log_prob=True)
        losses, _, _ = compute_loss(cfg, m, pc, pr, None, (aux["chosen_tokens"], aux["rejected_tokens"]))
        (losses.mean() * t / sum(toks)).backward()
        want_loss += float(losses.mean()) * t / sum(toks)
    assert torch.allclose(got, learner.model.grad_flat(), atol=1e-7)
    assert abs(tr._metrics["train_loss"][0] - want_loss) < 1e-6 and toks[0] * 3 < toks[1]


def test_dpo_entry_point_trains_checkpoints_and_resumes(tmp_path, monkeypatch):
    import open_instruct_b200.dpo as dpo
    import open_instruct_b200.dpo_tune_cache as dtc
    import open_instruct_b200.dpo_utils as du
    from open_instruct_b200.data.tokenize import TokenizerConfig

    tmp = str(tmp_path)
    monkeypatch.setattr(dtc, "REFERENCE_LOGPROBS_CACHE_PATH", os.path.join(tmp, "refcache"))
    tok = make_tokenizer(os.path.join(tmp, "tok"))
    data = make_pref_jsonl(os.path.join(tmp, "pref.jsonl"))

    def cfg(**kw):
        return du.DPOExperimentConfig(model_name_or_path="tiny", mixer_list=[data, "1.0"], max_seq_length=96, per_device_train_batch_size=4,
                                      gradient_accumulation_steps=2, learning_rate=2e-3, num_epochs=3, output_dir=os.path.join(tmp, "out"),
                                      local_cache_dir=os.path.join(tmp, "cache"), beta=0.5, loss_type="dpo_norm", checkpointing_steps=4,
                                      ops="ref", seed=1, warmup_ratio=0.0, **kw)

    tc = TokenizerConfig(tokenizer_name_or_path=tok, chat_template_name="tulu")
    out = dpo.main(cfg(max_train_steps=6), tc)
    lines = [json.loads(l) for l in open(os.path.join(tmp, "out", "metrics.jsonl"))]
    assert out["completed_steps"] == 6 and len(lines) == 6
    assert abs(lines[0]["train_loss"] - math.log(2)) < 0.05 and lines[-1]["train_loss"] < lines[0]["train_loss"]
    assert "perf/tokens_per_second_step" in lines[-1] and "time/training" in lines[-1] and lines[-1]["rewards/accuracy"] >= 0.5
    assert os.path.exists(os.path.join(tmp, "out", "step_4", "COMPLETED")) and os.path.exists(os.path.join(tmp, "out", "model.safetensors"))
    # a second call picks the newest complete checkpoint up and continues from it
    out2 = dpo.main(cfg(max_train_steps=8), tc)
    lines2 = [json.loads(l) for l in open(os.path.join(tmp, "out", "metrics.jsonl"))]
    assert out2["completed_steps"] == 8 and [l["training_step"] for l in lines2[6:]] == [5, 6, 7, 8]


def test_grpo_entry_point_runs_callbacks(tmp_path):
    from open_instruct_b200.config.schemas import ModelConfig
    from open_instruct_b200.data.tokenize import TokenizerConfig
    from open_instruct_b200.grpo import main
    from open_instruct_b200.grpo_utils import GRPOExperimentConfig
    from open_instruct_b200.streaming import StreamingDataLoaderConfig, VLLMConfig

    tmp = str(tmp_path)
    tok = make_tokenizer(os.path.join(tmp, "tok"))
    data = make_rlvr_jsonl(os.path.join(tmp, "rl.jsonl"), n=12)
    eval_data = make_rlvr_jsonl(os.path.join(tmp, "eval.jsonl"), n=3)
    args = GRPOExperimentConfig(total_episodes=3 * 4 * 4, learning_rate=1e-3, beta=0.05, load_ref_policy=True, ref_policy_update_freq=2, alpha=0.5,
                                output_dir=os.path.join(tmp, "out"), single_gpu_mode=True, ops="ref", seed=3, save_freq=-1, checkpoint_state_freq=2,
                                checkpoint_state_dir=os.path.join(tmp, "state"), lr_scheduler_type="constant", local_eval_every=2, eval_on_step_0=True)
    streaming = StreamingDataLoaderConfig(max_prompt_token_length=64, response_length=12, pack_length=256, async_steps=1,
                                          num_samples_per_prompt_rollout=4, num_unique_prompts_rollout=4, dataset_mixer_list=[data, "1.0"],
                                          dataset_mixer_eval_list=[eval_data, "1.0"], dataset_mixer_eval_list_splits=["train"],
                                          dataset_local_cache_dir=os.path.join(tmp, "cache"), filter_zero_std_samples=False, temperature=1.0)
    out = main(args, TokenizerConfig(tokenizer_name_or_path=tok, chat_template_name="tulu"), ModelConfig(model_name_or_path="tiny"), streaming,
               VLLMConfig())
    assert out["num_training_steps"] == 3 and out["training_step"] == 3
    lines = [json.loads(l) for l in open(os.path.join(args.output_dir, "metrics.jsonl"))]
    assert len(lines) == 3 and all(l["time/weight_sync"] >= 0 for l in lines)
    assert any("eval/num_prompts" in l for l in lines)  # step 1 (eval_on_step_0) or step 2 or the last step
    assert os.path.exists(os.path.join(args.output_dir, "model.safetensors"))
    assert os.path.exists(os.path.join(tmp, "state", "step_2", "COMPLETED"))
