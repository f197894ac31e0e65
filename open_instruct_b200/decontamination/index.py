"""Fill an Elasticsearch text index with the user turns of a training set (``decontamination/index.py:152-218`` in the
reference): one document per message that passes ``--query_filter``, carrying the row number it came from.

    python -m open_instruct_b200.decontamination.index --es_url http://localhost:9200 --dataset train.jsonl
    python -m open_instruct_b200.decontamination.index --dataset_mixer_config configs/train_configs/tulu3_8b_sft.yaml

``--dataset`` is a local ``.jsonl`` / ``.json`` / ``.parquet`` file or a dataset name the data layer can load;
``--dataset_mixer_config`` indexes every dataset a training recipe mixes (its ``dataset_mixer`` mapping or
``dataset_mixer_list``).  ``--index_type vector`` stores an embedding per message made by ``--model`` (a local Hugging Face
model folder, mean-pooled; the reference's default embedding model is not in this image).
"""

from __future__ import annotations

import argparse

from .es import ElasticClient, Embedder, index_name_for, index_text, index_vectors, messages_to_index


def _rows(dataset: str, split: str) -> list[dict]:
    from ..data.mixer import _load_any

    return list(_load_any(dataset, split, None))


def _mixer_datasets(path: str) -> list[str]:
    import yaml

    cfg = yaml.safe_load(open(path))
    if cfg.get("dataset_mixer"):
        return list(cfg["dataset_mixer"].keys())
    if cfg.get("dataset_mixer_list"):
        return list(cfg["dataset_mixer_list"][0::2])
    raise ValueError(f"{path} has neither dataset_mixer nor dataset_mixer_list")


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--es_url", default="http://localhost:9200")
    ap.add_argument("--dataset")
    ap.add_argument("--dataset_mixer_config", help="a training recipe (yaml) whose datasets are all indexed")
    ap.add_argument("--split", default="train")
    ap.add_argument("--messages_field", default="messages")
    ap.add_argument("--query_filter", default="role:user")
    ap.add_argument("--query_field", default="content")
    ap.add_argument("--index_type", choices=["text", "vector"], default="text")
    ap.add_argument("--text_batch_size", type=int, default=1000)
    ap.add_argument("--model", default=None, help="vector indexes: folder of the Hugging Face model that embeds the messages")
    ap.add_argument("--max_batch_tokens", type=int, default=10000)
    a = ap.parse_args(argv)
    if a.index_type == "vector" and not a.model:
        raise SystemExit("--index_type vector needs --model (a local Hugging Face model folder)")
    embed = Embedder(a.model, a.max_batch_tokens) if a.index_type == "vector" else None
    if a.dataset_mixer_config:
        names = _mixer_datasets(a.dataset_mixer_config)
    elif a.dataset:
        names = [a.dataset]
    else:
        raise SystemExit("give --dataset or --dataset_mixer_config")
    es = ElasticClient(a.es_url)
    added = {}
    for name in names:
        docs = messages_to_index(_rows(name, a.split), a.messages_field, a.query_filter, a.query_field)
        index = index_name_for(name, a.index_type)
        added[index] = index_text(es, index, docs, a.text_batch_size) if embed is None else index_vectors(es, index, docs, embed)
        print(f"{index}: {added[index]} documents added ({len(docs)} messages in {name})")
    return added


if __name__ == "__main__":
    main()
