"""Linear merge of Hugging Face checkpoints: weighted average of safetensors shards, file by file.

    python -m open_instruct_b200.ckpt.merge_models --models A B C --model_weights 1 1 2 --output_dir out

All models must have the same shard files and tensor names (``open_instruct/merge_models.py:69-129``): weights
are normalised to sum to one, each shard is averaged in fp32 and written in ``--dtype``; config, index and
tokenizer files are copied from the first model.
"""

from __future__ import annotations

import argparse
import shutil
from pathlib import Path

import torch

_DTYPES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}


def get_safetensor_files(model_path: Path) -> list[str]:
    return sorted(p.name for p in Path(model_path).glob("*.safetensors"))


def merge_models(model_paths: list[str], output_dir: str, model_weights: list[float] | None = None, dtype: str = "bfloat16") -> None:
    from safetensors import safe_open
    from safetensors.torch import save_file

    paths = [Path(p) for p in model_paths]
    weights = list(model_weights) if model_weights else [1.0] * len(paths)
    if len(weights) != len(paths):
        raise ValueError(f"Number of weights ({len(weights)}) must match number of models ({len(paths)})")
    total = sum(weights)
    if total <= 0:
        raise ValueError("model weights must sum to a positive number")
    weights = [w / total for w in weights]
    out = Path(output_dir)
    out.mkdir(parents=True, exist_ok=True)
    files = get_safetensor_files(paths[0])
    if not files:
        raise FileNotFoundError(f"no safetensors files in {paths[0]}")
    for p in paths[1:]:
        if get_safetensor_files(p) != files:
            raise ValueError(f"{p} has different shard files than {paths[0]}")
    td = _DTYPES[dtype]
    for fname in files:
        handles = [safe_open(str(p / fname), framework="pt") for p in paths]
        names = list(handles[0].keys())
        merged = {}
        for name in names:
            acc = None
            for h, w in zip(handles, weights):
                t = h.get_tensor(name).to(torch.float32) * w
                acc = t if acc is None else acc.add_(t)
            merged[name] = acc.to(td)
        save_file(merged, str(out / fname), metadata={"format": "pt"})
    for f in paths[0].iterdir():
        if f.is_file() and f.suffix != ".safetensors" and not f.name.startswith("."):
            shutil.copy2(f, out / f.name)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description="Linear merge of Hugging Face models")
    ap.add_argument("--models", nargs="+", required=True)
    ap.add_argument("--model_weights", nargs="+", type=float, default=None)
    ap.add_argument("--output_dir", required=True)
    ap.add_argument("--dtype", default="bfloat16", choices=list(_DTYPES))
    a = ap.parse_args(argv)
    merge_models(a.models, a.output_dir, a.model_weights, a.dtype)


if __name__ == "__main__":
    main()
