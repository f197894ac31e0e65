"""Reward model: Bradley-Terry training end to end on CPU."""

import json
import os

from helpers import make_pref_jsonl, make_tokenizer


def test_reward_model_learns(tmp_path):
    from open_instruct_b200.config.schemas import ModelConfig
    from open_instruct_b200.data.tokenize import TokenizerConfig
    from open_instruct_b200.reward_modeling import Args, main

    tmp = str(tmp_path)
    tok = make_tokenizer(os.path.join(tmp, "tok"))
    data = make_pref_jsonl(os.path.join(tmp, "pref.jsonl"), n=32)
    args = Args(dataset_mixer_list=[data, "1.0"], dataset_mixer_eval_list=[data, "8"], dataset_mixer_eval_list_splits=["train"],
                dataset_local_cache_dir=os.path.join(tmp, "cache"), output_dir=os.path.join(tmp, "out"), learning_rate=3e-3,
                gradient_accumulation_steps=2, per_device_train_batch_size=4, num_train_epochs=4, ops="ref", num_evals=2)
    out = main(args, TokenizerConfig(tokenizer_name_or_path=tok, chat_template_name="tulu"), ModelConfig(model_name_or_path="tiny"))
    lines = [json.loads(l) for l in open(os.path.join(args.output_dir, "metrics.jsonl"))]
    assert lines[-1]["train/rm/loss"] < lines[0]["train/rm/loss"]
    assert out["train/rm/accuracy"] > 0.7
    assert "eval/rm/accuracy" in out
    from open_instruct_b200.reward_modeling import load_score_weight

    w = load_score_weight(args.output_dir)   # the head travels inside the weight files, where HF looks for it
    assert w is not None and tuple(w.shape)[0] == 1
