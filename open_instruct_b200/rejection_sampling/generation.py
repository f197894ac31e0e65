"""Sample ``n`` completions per prompt with the rollout engine and write them as jsonl.

Output rows: ``{"messages": [... prompt ..., {"role": "assistant", "content": completion}], "model_completion": ...,
"reference_completion": last assistant turn of the source row}`` - ``n`` consecutive rows per prompt, which is the
input format of ``rejection_sampling.py`` (cf. ``open_instruct/rejection_sampling/generation.py:45-303``).
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field

from ..data_types import SamplingConfig


@dataclass
class GenerationArgs:
    num_completions: int = 3
    temperature: float = 0.8
    response_length: int = 2048
    top_p: float = 0.9
    seed: int = 0


@dataclass
class Args:
    dataset_mixer_list: list[str] = field(default_factory=lambda: ["allenai/tulu-v2-sft-mixture", "100"])
    dataset_splits: list[str] = field(default_factory=lambda: ["train"])
    model_name_or_path: str = "tiny"
    save_filename: str = "completions.jsonl"
    max_prompts: int | None = None


def generate_rows(engine, tokenizer, rows: list[dict], gen: GenerationArgs) -> list[dict]:
    """``rows`` carry ``messages`` whose last turn is the reference answer."""
    prompts = []
    for r in rows:
        ids = tokenizer.apply_chat_template(r["messages"][:-1], add_generation_prompt=True, tokenize=True)
        prompts.append(list(ids["input_ids"] if isinstance(ids, dict) else ids))
    cfg = SamplingConfig(temperature=gen.temperature, top_p=gen.top_p, max_tokens=gen.response_length, n=gen.num_completions, seed=gen.seed)
    results = engine.generate(prompts, cfg)
    out = []
    for r, res in zip(rows, results):
        for resp in res.responses:
            text = tokenizer.decode([t for t in resp if t not in engine.eos], skip_special_tokens=True)
            out.append({"messages": r["messages"][:-1] + [{"role": "assistant", "content": text}], "model_completion": text,
                        "reference_completion": r["messages"][-1]["content"]})
    return out


def save_jsonl(path: str, rows: list[dict]) -> None:
    with open(path, "w") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")


def main(args: Args, gen: GenerationArgs) -> list[dict]:
    from ..data.legacy_mix import get_datasets
    from ..data.tokenize import TokenizerConfig
    from ..models.spec import get_spec
    from ..rollout.engine import RolloutEngine

    ds = get_datasets(args.dataset_mixer_list, splits=args.dataset_splits, columns_to_keep=["messages"])["train"]
    rows = [ds[i] for i in range(len(ds) if args.max_prompts is None else min(len(ds), args.max_prompts))]
    tc = TokenizerConfig(tokenizer_name_or_path=args.model_name_or_path)
    import os

    import torch

    spec = get_spec(args.model_name_or_path)
    engine = RolloutEngine(spec, device="cuda" if torch.cuda.is_available() else "cpu", tokenizer=tc.tokenizer)
    if os.path.isdir(args.model_name_or_path):
        from ..ckpt.hf_io import load_hf_checkpoint

        load_hf_checkpoint(args.model_name_or_path, engine.model.flat, spec, engine.model.layout)
    out = generate_rows(engine, tc.tokenizer, rows, gen)
    save_jsonl(args.save_filename, out)
    return out


if __name__ == "__main__":
    from ..config.argparser import ArgumentParserPlus

    main(*ArgumentParserPlus((Args, GenerationArgs)).parse())
