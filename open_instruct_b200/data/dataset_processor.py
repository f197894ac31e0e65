"""First-generation dataset processors: tokenise whole conversations with the chat template, then filter by length.

The column contract and the filter rules of the reference's ``open_instruct/dataset_processor.py`` (still used by its
reward-model trainer and by tests): a preference row gets ``input_ids_prompt / input_ids_chosen / input_ids_rejected``
(+ attention masks); an SFT row gets ``input_ids_prompt``, ``input_ids``, ``attention_mask`` and ``labels`` (the prompt part
masked with -100 when ``train_only_on_prompt`` is set - the flag's name is historical: it trains on the RESPONSE only); the
ground-truth variant also carries the verifier columns through.  The newer transform-function pipeline lives in
``data/tokenize.py`` / ``data/mixer.py``; both produce columns the collators of ``data/collate.py`` accept.

Written as one processor with three row schemas instead of three classes with copied bodies; the three class names remain.
"""

from __future__ import annotations

import logging
import multiprocessing
import os
from dataclasses import dataclass

from .templates import CHAT_TEMPLATES

INPUT_IDS_CHOSEN_KEY, ATTENTION_MASK_CHOSEN_KEY = "input_ids_chosen", "attention_mask_chosen"
INPUT_IDS_REJECTED_KEY, ATTENTION_MASK_REJECTED_KEY = "input_ids_rejected", "attention_mask_rejected"
INPUT_IDS_PROMPT_KEY, ATTENTION_MASK_PROMPT_KEY = "input_ids_prompt", "attention_mask_prompt"
GROUND_TRUTHS_KEY, VERIFIER_SOURCE_KEY = "ground_truth", "dataset"
SFT_MESSAGE_KEY, INPUT_IDS_KEY, ATTENTION_MASK_KEY, LABELS_KEY = "messages", "input_ids", "attention_mask", "labels"
TOKENIZED_PREFERENCE_DATASET_KEYS = [INPUT_IDS_CHOSEN_KEY, INPUT_IDS_REJECTED_KEY]

# planning constants for ``dataset.map`` / ``dataset.filter`` worker counts (examples per second per CPU)
APPLY_CHAT_TEMPLATE_EXAMPLE_PER_SECOND_PER_CPU = 400
FILTER_EXAMPLE_PER_SECOND_PER_CPU = 1130

logger = logging.getLogger(__name__)


@dataclass
class DatasetConfig:
    chat_template: str | None = None
    preference_chosen_key: str = "chosen"
    preference_rejected_key: str = "rejected"
    sft_messages_key: str = SFT_MESSAGE_KEY
    ground_truths_key: str = GROUND_TRUTHS_KEY
    dataset_source_key: str = VERIFIER_SOURCE_KEY
    max_token_length: int | None = None
    max_prompt_token_length: int | None = None
    sanity_check: bool = False
    sanity_check_max_samples: int = 100
    batched: bool = False
    load_from_cache_file: bool = True
    num_proc: int = int(float(os.environ.get("BEAKER_ASSIGNED_CPU_COUNT", multiprocessing.cpu_count())))
    train_only_on_prompt: bool = False

    def __post_init__(self):
        if self.sanity_check:
            self.num_proc, self.load_from_cache_file = 1, False
        if self.chat_template is not None and self.chat_template not in CHAT_TEMPLATES:
            raise ValueError(f"chat_template must None or one of {list(CHAT_TEMPLATES.keys())}")


def get_num_proc(dataset_len: int, num_available_cpus: int, example_per_second_per_cpu) -> int:
    """Workers for a map/filter pass: one per second of single-CPU work, within what the machine and the data allow."""
    return max(1, min(max(1, dataset_len // example_per_second_per_cpu), num_available_cpus, dataset_len))


class DatasetProcessor:
    def __init__(self, tokenizer, config: DatasetConfig) -> None:
        self.tokenizer, self.config = tokenizer, config
        if tokenizer.pad_token_id == tokenizer.eos_token_id:
            logger.warning("Tokenizer's pad token is the same as EOS token, this might cause the model to not learn to generate EOS tokens.")

    # ---- shared plumbing
    def _ids(self, messages, generation_prompt: bool = False) -> list[int]:
        out = self.tokenizer.apply_chat_template(messages, add_generation_prompt=generation_prompt)
        return list(out["input_ids"]) if hasattr(out, "keys") else list(out)  # newer tokenizers return an encoding object

    def _map(self, dataset, fn, desc: str):
        return dataset.map(fn, num_proc=get_num_proc(len(dataset), self.config.num_proc, APPLY_CHAT_TEMPLATE_EXAMPLE_PER_SECOND_PER_CPU),
                           load_from_cache_file=self.config.load_from_cache_file, desc=desc)

    def _filter(self, dataset, fn, desc: str):
        return dataset.filter(fn, num_proc=get_num_proc(len(dataset), self.config.num_proc, FILTER_EXAMPLE_PER_SECOND_PER_CPU),
                              load_from_cache_file=self.config.load_from_cache_file, desc=desc)

    def tokenize(self, dataset):
        raise NotImplementedError

    def filter(self, dataset):
        raise NotImplementedError


class PreferenceDatasetProcessor(DatasetProcessor):
    def tokenize(self, dataset):
        c = self.config

        def row_fn(row):
            prompt = self._ids(row[c.preference_chosen_key][:-1], generation_prompt=True)
            chosen, rejected = self._ids(row[c.preference_chosen_key]), self._ids(row[c.preference_rejected_key])
            row.update({INPUT_IDS_PROMPT_KEY: prompt, ATTENTION_MASK_PROMPT_KEY: [1] * len(prompt), INPUT_IDS_CHOSEN_KEY: chosen,
                        ATTENTION_MASK_CHOSEN_KEY: [1] * len(chosen), INPUT_IDS_REJECTED_KEY: rejected,
                        ATTENTION_MASK_REJECTED_KEY: [1] * len(rejected)})
            return row

        return self._map(dataset, row_fn, "Tokenizing preference data")

    def filter(self, dataset):
        c = self.config

        def keep(row):
            if c.max_prompt_token_length is not None:  # the prompt limit, when given, is the only rule
                return len(row[INPUT_IDS_PROMPT_KEY]) <= c.max_prompt_token_length
            if c.max_token_length is not None:
                return len(row[INPUT_IDS_CHOSEN_KEY]) <= c.max_token_length and len(row[INPUT_IDS_REJECTED_KEY]) <= c.max_token_length
            return True

        out = self._filter(dataset, keep, "Filtering preference data")
        logger.info("Filtered out %d of %d preference rows", len(dataset) - len(out), len(dataset))
        return out


class SFTDatasetProcessor(DatasetProcessor):
    carry_ground_truth = False

    def tokenize(self, dataset):
        c = self.config

        def row_fn(row):
            msgs = row[c.sft_messages_key]
            prompt = self._ids(msgs if len(msgs) == 1 else msgs[:-1], generation_prompt=True)
            ids = self._ids(msgs)
            labels = list(ids)
            if c.train_only_on_prompt:
                n = min(len(prompt), len(labels))
                labels[:n] = [-100] * n
            row.update({INPUT_IDS_PROMPT_KEY: prompt, INPUT_IDS_KEY: ids, ATTENTION_MASK_KEY: [1] * len(ids), LABELS_KEY: labels})
            if self.carry_ground_truth:
                row[GROUND_TRUTHS_KEY], row[VERIFIER_SOURCE_KEY] = row[c.ground_truths_key], row[c.dataset_source_key]
            return row

        return self._map(dataset, row_fn, "Tokenizing and reformatting SFT data")

    def filter(self, dataset, need_contain_labels: bool = True):
        c = self.config

        def keep(row):
            if c.max_prompt_token_length is not None and len(row[INPUT_IDS_PROMPT_KEY]) > c.max_prompt_token_length:
                return False
            if c.max_token_length is not None and len(row[INPUT_IDS_KEY]) > c.max_token_length:
                return False
            return not need_contain_labels or any(x != -100 for x in row[LABELS_KEY])

        return self._filter(dataset, keep, "Filtering SFT data")


class SFTGroundTruthDatasetProcessor(SFTDatasetProcessor):
    """SFT rows that keep their verifier columns (``ground_truth``, ``dataset``) for RLVR-style evaluation."""

    carry_ground_truth = True
