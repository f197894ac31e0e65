"""Legacy dict-style dataset mixer (``{name: fraction | count}``) and the two mixing CLIs.

Behaviour of ``get_datasets`` in the reference (``open_instruct/utils.py:377-590``): local json/jsonl/parquet
or hub names; optional seeded shuffle (seed 42); well-known instruction schemas are converted to ``messages``;
an ``id`` column is created when missing; only ``columns_to_keep`` (+ id, + optional ``source``) survive; all
amounts are either fractions in [0, 1] or integer counts (no mixing of the two); test splits are never subsampled.
``python -m open_instruct_b200.data.legacy_mix [sft|preferences] config.yaml`` replaces ``mix_data.py`` and
``mix_data_preferences.py``.
"""

from __future__ import annotations

import dataclasses
import os
import sys


def _to_messages(row: dict) -> dict | None:
    """Schema conversions the legacy mixer knows (alpaca, code-alpaca, sharegpt, orca, codefeedback, metamath)."""
    def two(u, a, system=None):
        msgs = ([{"role": "system", "content": system}] if system else []) + [{"role": "user", "content": u}, {"role": "assistant", "content": a}]
        return {"messages": msgs}

    if "instruction" in row and "output" in row:
        u = row["instruction"] + ("\n\n" + row["input"] if row.get("input") else "")
        return two(u, row["output"])
    if "prompt" in row and "completion" in row:
        return two(row["prompt"], row["completion"])
    if "conversations" in row:
        role = {"human": "user", "user": "user", "gpt": "assistant", "assistant": "assistant", "system": "system"}
        return {"messages": [{"role": role.get(t.get("from", t.get("role")), "user"), "content": t.get("value", t.get("content", ""))}
                             for t in row["conversations"]]}
    if "question" in row and "response" in row:
        return two(row["question"], row["response"], row.get("system_prompt") or None)
    if "query" in row and "answer" in row:
        return two(row["query"], row["answer"])
    if "query" in row and "response" in row:
        return two(row["query"], row["response"])
    if "chosen" in row and "rejected" in row and "reference_completion" in row:
        return {"messages": row["chosen"]}
    return None


def get_datasets(dataset_mixer: dict | list, splits: list[str] | None = None, configs: list | None = None, columns_to_keep: list[str] | None = None,
                 shuffle: bool = True, save_data_dir: str | None = None, need_columns: list[str] | None = None, keep_ids: bool = False,
                 add_source_col: bool = False):
    from datasets import DatasetDict, concatenate_datasets, load_dataset, load_from_disk

    if isinstance(dataset_mixer, list):
        if len(dataset_mixer) % 2:
            raise ValueError(f"Data mixer list length is not even: {dataset_mixer}")
        dataset_mixer = {dataset_mixer[i]: (float(dataset_mixer[i + 1]) if "." in str(dataset_mixer[i + 1]) else int(dataset_mixer[i + 1]))
                         for i in range(0, len(dataset_mixer), 2)}
    splits = splits or ["train", "test"]
    configs = configs or [None] * len(dataset_mixer)
    keep = list(columns_to_keep or [])
    if len(configs) != len(dataset_mixer):
        raise ValueError("The number of given dataset config names must be the same as the given number of datasets.")
    amounts = list(dataset_mixer.values())
    if any(a < 0 for a in amounts):
        raise ValueError("Dataset fractions / lengths cannot be negative.")
    by_count = any(a > 1 for a in amounts)
    if by_count and not all(isinstance(a, int) for a in amounts):
        raise NotImplementedError("Cannot mix fractions and counts, yet.")

    train, test = [], []
    for (name, _), cfg in zip(dataset_mixer.items(), configs):
        for split in splits:
            if name.endswith((".json", ".jsonl")):
                ds = load_dataset("json", data_files=name, split=split)
            elif name.endswith(".parquet"):
                ds = load_dataset("parquet", data_files=name, split=split)
            elif os.path.isdir(os.path.join(name, split)):
                ds = load_from_disk(os.path.join(name, split))
            else:
                ds = load_dataset(name, cfg, split=split)
            if shuffle:
                ds = ds.shuffle(seed=42)
            if need_columns and not all(c in ds.column_names for c in need_columns):
                raise ValueError(f"Needed column {need_columns} not found in dataset {ds.column_names}.")
            if "messages" not in ds.column_names and _to_messages({c: None for c in ds.column_names} | ds[0] if len(ds) else {}) is not None:
                ds = ds.map(_to_messages)
            if "id" not in ds.column_names:
                ds = ds.add_column("id", [f"{name}_{i}" for i in range(len(ds))])
            ds = ds.remove_columns([c for c in ds.column_names if c not in keep + ["id"]])
            if add_source_col:
                ds = ds.add_column("source", [name] * len(ds))
            for c in keep:
                if c not in ds.column_names:
                    ds = ds.add_column(c, [None] * len(ds))
            if "train" in split:
                train.append(ds)
            elif "test" in split:
                test.append(ds)
            else:
                raise ValueError(f"Split type {split} not recognized as one of test or train.")
    if not train and not test:
        raise ValueError("No datasets loaded.")
    features = (train or test)[0].features
    out = DatasetDict()
    if train:
        parts = []
        for ds, amount in zip(train, amounts):
            ds = ds.cast(features)
            parts.append(ds.select(range(amount if by_count else int(amount * len(ds)))))
        out["train"] = concatenate_datasets(parts)
    if test:
        out["test"] = concatenate_datasets([d.cast(features) for d in test])
    if not keep_ids:
        for k in list(out):
            if "id" in out[k].column_names:
                out[k] = out[k].remove_columns("id")
    if save_data_dir:
        os.makedirs(save_data_dir, exist_ok=True)
        for k, d in out.items():
            d.to_json(os.path.join(save_data_dir, f"mixed_ds_{k}.json"))
    return out


@dataclasses.dataclass
class MixDataArguments:
    dataset_mixer: dict | None = None
    dataset_config_name: str | None = None
    dataset_mix_dir: str | None = None
    save_to_hub: str | None = None


def main(argv: list[str] | None = None) -> None:
    from ..config.argparser import ArgumentParserPlus

    argv = list(sys.argv[1:] if argv is None else argv)
    kind = argv.pop(0) if argv and argv[0] in ("sft", "preferences") else "sft"
    args = ArgumentParserPlus((MixDataArguments,)).parse(argv, allow_extra_keys=True) if argv else None
    if args is None or args.dataset_mixer is None:
        raise SystemExit("a config with `dataset_mixer` is required")
    cols = ["messages"] if kind == "sft" else ["chosen", "rejected"]
    raw = get_datasets(args.dataset_mixer, configs=[args.dataset_config_name] * len(args.dataset_mixer) if args.dataset_config_name else None,
                       splits=["train"], save_data_dir=args.dataset_mix_dir, columns_to_keep=cols, keep_ids=True, add_source_col=True)
    for i in range(min(5, len(raw["train"]))):
        print(raw["train"][i])
    if args.save_to_hub:
        raw["train"].push_to_hub(args.save_to_hub, private=True)


if __name__ == "__main__":
    main()
