"""Turn a training-state checkpoint (``step_N`` / ``epoch_N``: the sharded optimizer's fp32 master weights, one file per
rank) into a Hugging Face checkpoint folder, without the trainer and for any number of ranks it was written by.

The counterpart of the reference's ``scripts/train/convert_olmo_core_to_hf.py`` (distributed training checkpoint -> HF
folder): a run that was interrupted, or a step in the middle of a run, becomes a model that evaluation tools can load.

    python -m open_instruct_b200.ckpt.convert_state_to_hf --checkpoint-dir out/step_1000 --model-name llama3.1-8b \\
        --output-dir out/step_1000_hf [--tokenizer-name path-or-name] [--dtype bfloat16]

``--model-name`` is a preset or a folder with a ``config.json`` (the architecture the run trained); the tokenizer files are
copied when ``--tokenizer-name`` (default: ``--model-name`` if it is a folder) holds any.
"""

from __future__ import annotations

import argparse
import os

import torch

from ..models.spec import ParamLayout, get_spec
from .hf_io import save_hf_checkpoint


def master_weights(ckpt_dir: str) -> torch.Tensor:
    """The fp32 master weights of a checkpoint directory, whole: the ranks' slices in rank order."""
    files = [f for f in os.listdir(ckpt_dir) if f.startswith("optim_rank") and f.endswith(".pt")]
    if not files:
        raise FileNotFoundError(f"no optimizer shards (optim_rank*_of_*.pt) in {ckpt_dir}")
    world = int(files[0].split("_of_")[1].split(".")[0])
    missing = [r for r in range(world) if f"optim_rank{r}_of_{world}.pt" not in files]
    if missing:
        raise FileNotFoundError(f"{ckpt_dir} was written by {world} ranks; the shards of ranks {missing} are missing")
    if not os.path.exists(os.path.join(ckpt_dir, "COMPLETED")):
        raise RuntimeError(f"{ckpt_dir} has no COMPLETED marker: the checkpoint was not written to the end")
    parts = []
    for r in range(world):
        sd = torch.load(os.path.join(ckpt_dir, f"optim_rank{r}_of_{world}.pt"), map_location="cpu", weights_only=False)
        if "master" not in sd:
            raise KeyError(f"optim_rank{r}_of_{world}.pt holds no master weights (keys: {sorted(sd)})")
        parts.append(sd["master"].float())
    return torch.cat(parts)


def main(argv=None) -> str:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--checkpoint-dir", required=True)
    ap.add_argument("--model-name", required=True)
    ap.add_argument("--output-dir", required=True)
    ap.add_argument("--tokenizer-name", default=None)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"])
    a = ap.parse_args(argv)
    spec = get_spec(a.model_name)
    layout = ParamLayout(spec)
    flat = master_weights(a.checkpoint_dir)
    if flat.numel() < layout.total:
        raise ValueError(f"the checkpoint holds {flat.numel()} parameters, {a.model_name} needs {layout.total}: not the architecture of this run")
    tokenizer = None
    tok_src = a.tokenizer_name or (a.model_name if os.path.isdir(a.model_name) else None)
    if tok_src and (not os.path.isdir(tok_src) or any(f.startswith("tokenizer") for f in os.listdir(tok_src))):
        from transformers import AutoTokenizer

        tokenizer = AutoTokenizer.from_pretrained(tok_src)
    save_hf_checkpoint(flat[: layout.total], spec, a.output_dir, tokenizer=tokenizer, layout=layout, dtype=getattr(torch, a.dtype))
    return a.output_dir


if __name__ == "__main__":
    main()
