"""Hugging Face checkpoint directories <-> the flat parameter buffer.

Export writes what ``save_pretrained`` writes (``open_instruct/model_utils.py:525-583``,
``open_instruct/grpo_fast.py:843-894``): ``config.json``, ``generation_config.json``, sharded
``model-0000x-of-0000y.safetensors`` + ``model.safetensors.index.json`` with Hugging Face tensor names
(fused ``wqkv`` / ``w_gate_up`` are split back into q/k/v and gate/up), tokenizer files.  Import reads
the same layout (single-file or sharded) into the flat buffer, fusing on the fly.
"""

from __future__ import annotations

import json
import os
from pathlib import Path

import torch

from ..models.spec import ModelSpec, ParamLayout

MAX_SHARD_BYTES = 5 * 1024**3


def state_dict_from_flat(flat: torch.Tensor, layout: ParamLayout, dtype=torch.bfloat16) -> dict[str, torch.Tensor]:
    """HF-named CPU tensors (views of one host copy per fused entry)."""
    out = {}
    for name in layout.entries:
        t = layout.view(flat.detach(), name).to("cpu", dtype)
        for hf_name, a, b in layout.hf_names(name):
            out[hf_name] = _hf_shape(hf_name, t[a:b].contiguous(), layout.spec)
    return out


def _hf_shape(hf_name: str, piece: torch.Tensor, spec: ModelSpec) -> torch.Tensor:
    """The shape a checkpoint stores ``piece`` in where it differs from the flat layout's 2-D entry."""
    if spec.num_experts and hf_name.endswith(("experts.gate_up_proj", "experts.down_proj")):
        return piece.view(spec.num_experts, -1, piece.shape[1])  # the stacked [experts, rows, cols] form
    if hf_name.endswith("conv1d.weight"):
        return piece.unsqueeze(1)                                # depthwise convolution: [channels, 1, taps]
    return piece


def save_hf_checkpoint(flat: torch.Tensor, spec: ModelSpec, out_dir: str, tokenizer=None, layout: ParamLayout | None = None,
                       dtype=torch.bfloat16, max_shard_bytes: int = MAX_SHARD_BYTES, extra_config: dict | None = None,
                       extra_tensors: dict | None = None, skip: set | None = None) -> None:
    """Write ``flat`` as a Hugging Face checkpoint folder.  ``extra_tensors``: tensors outside the layout that belong in the
    weight files (a reward model's ``score.weight``); ``skip``: HF tensor names to leave out (its ``lm_head.weight``)."""
    from safetensors.torch import save_file

    layout = layout or ParamLayout(spec)
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    cfg = spec.to_hf_config()
    cfg.update(extra_config or {})
    (out / "config.json").write_text(json.dumps(cfg, indent=2))
    gen = {"bos_token_id": spec.bos_token_id, "eos_token_id": spec.eos_token_id, "pad_token_id": spec.pad_token_id,
           "do_sample": True, "transformers_version": "4.0"}
    (out / "generation_config.json").write_text(json.dumps({k: v for k, v in gen.items() if v is not None}, indent=2))
    # shard greedily in layout order, one fused entry at a time (bounded host memory)
    shards: list[dict[str, torch.Tensor]] = [{}]
    size = 0
    for name in layout.entries:
        t = layout.view(flat.detach(), name).to("cpu", dtype)
        for hf_name, a, b in layout.hf_names(name):
            if skip and hf_name in skip:
                continue
            piece = _hf_shape(hf_name, t[a:b].contiguous(), spec)
            nbytes = piece.numel() * piece.element_size()
            if size + nbytes > max_shard_bytes and shards[-1]:
                shards.append({})
                size = 0
            shards[-1][hf_name] = piece
            size += nbytes
    for hf_name, t in (extra_tensors or {}).items():
        shards[-1][hf_name] = t.detach().to("cpu", dtype).contiguous()
    n = len(shards)
    if n == 1:
        save_file(shards[0], str(out / "model.safetensors"), metadata={"format": "pt"})
    else:
        weight_map, total = {}, 0
        for i, sh in enumerate(shards):
            fname = f"model-{i + 1:05d}-of-{n:05d}.safetensors"
            save_file(sh, str(out / fname), metadata={"format": "pt"})
            for k, v in sh.items():
                weight_map[k] = fname
                total += v.numel() * v.element_size()
        (out / "model.safetensors.index.json").write_text(
            json.dumps({"metadata": {"total_size": total}, "weight_map": weight_map}, indent=2))
    if tokenizer is not None:
        tokenizer.save_pretrained(str(out))


def _open_shards(model_dir: str):
    from safetensors import safe_open

    d = Path(model_dir)
    idx = d / "model.safetensors.index.json"
    if idx.exists():
        wm = json.loads(idx.read_text())["weight_map"]
        files = sorted(set(wm.values()))
    elif (d / "model.safetensors").exists():
        files = ["model.safetensors"]
    else:
        raise FileNotFoundError(f"no safetensors weights in {model_dir}")
    handles = {f: safe_open(str(d / f), framework="pt", device="cpu") for f in files}
    where = {}
    for f, h in handles.items():
        for k in h.keys():
            where[k] = f
    return handles, where


def load_hf_checkpoint(model_dir: str, flat: torch.Tensor, spec: ModelSpec | None = None, layout: ParamLayout | None = None,
                       strict: bool = True) -> ModelSpec:
    """Fill ``flat`` from a Hugging Face directory; returns the spec read from its config."""
    spec = spec or ModelSpec.from_pretrained(model_dir)
    layout = layout or ParamLayout(spec)
    handles, where = _open_shards(model_dir)
    missing = []
    with torch.no_grad():
        for name in layout.entries:
            dst = layout.view(flat, name)
            names = layout.hf_names(name)
            if any(n not in where for n, _, _ in names) and layout.hf_names_per_expert(name) is not None:
                names = layout.hf_names_per_expert(name)  # experts stored one tensor each
            for hf_name, a, b in names:
                if hf_name not in where and spec.model_type == "olmo_hybrid":
                    # transformers writes the hybrid's layer norms under these names and reads either spelling
                    alt = hf_name.replace("input_layernorm", "attention_layer_norm").replace("post_attention_layernorm", "feedforward_layer_norm")
                    if alt in where:
                        dst[a:b].copy_(handles[where[alt]].get_tensor(alt))
                        continue
                if hf_name not in where:
                    if hf_name == "lm_head.weight" and "model.embed_tokens.weight" in where:
                        src = handles[where["model.embed_tokens.weight"]].get_tensor("model.embed_tokens.weight")
                    else:
                        missing.append(hf_name)
                        continue
                else:
                    src = handles[where[hf_name]].get_tensor(hf_name)
                if src.dim() == 3 and src.numel() == dst[a:b].numel():
                    src = src.reshape(dst[a:b].shape)  # stacked experts [E, rows, cols]
                if tuple(src.shape) != tuple(dst[a:b].shape):
                    if src.shape[0] < dst[a:b].shape[0] and name in ("embed", "lm_head"):
                        dst[a : a + src.shape[0]].copy_(src)  # resized vocabulary: extra rows keep their init
                        continue
                    raise ValueError(f"{hf_name}: checkpoint shape {tuple(src.shape)} != model {tuple(dst[a:b].shape)}")
                dst[a:b].copy_(src)
    if missing and strict:
        raise KeyError(f"missing tensors in {model_dir}: {missing[:5]}{'...' if len(missing) > 5 else ''}")
    return spec


def verify_roundtrip_names(spec: ModelSpec) -> list[str]:
    """All HF tensor names this layout writes (used to check exports against a reference listing)."""
    layout = ParamLayout(spec)
    return [n for e in layout.entries for n, _, _ in layout.hf_names(e)]
