"""Tokenizer set-up and row-level tokenisation transforms (SFT, preference, RLVR).

Behavioural contract = the reference's ``open_instruct/dataset_transformation.py``:
tokenizer factories and pad-token rules (``:644-866``), ``TokenizerConfig`` (``:874-912``), SFT label
spans (``:1207-1460``), preference (``:1489-1603``) and RLVR (``:1606-1788``) transforms, and the
name -> (function, "map" | "filter") registry (``:1791-1805``).

The SFT labelling rule: render the whole conversation with the chat template, tokenise with
character offsets, and train exactly the assistant turns - from the end of the generation prompt
that precedes a turn to the end of that turn (content + closing tokens).  A token is trainable when
its character range *overlaps* such a span.  When a rendered prefix is not a literal prefix of the
full render (templates that treat the last turn specially) the spans are derived from prefix token
counts instead and then verified against the decoded text; rows that fail verification come back
fully masked and are dropped by ``sft_tulu_filter_v1``.
"""

from __future__ import annotations

import copy
import hashlib
import logging
import os
from dataclasses import dataclass
from functools import cached_property
from typing import Any

import torch

from .templates import CHAT_TEMPLATES

logger = logging.getLogger(__name__)

# column names (the dataset schema shared with the trainers)
INPUT_IDS_KEY = "input_ids"
ATTENTION_MASK_KEY = "attention_mask"
LABELS_KEY = "labels"
DATASET_ORIGIN_KEY = "dataset_source"
TOKENIZED_SFT_DATASET_KEYS = [INPUT_IDS_KEY, ATTENTION_MASK_KEY, LABELS_KEY]
TOKENIZED_SFT_DATASET_KEYS_WITH_SOURCE = [*TOKENIZED_SFT_DATASET_KEYS, DATASET_ORIGIN_KEY]
DEFAULT_SFT_MESSAGES_KEY = "messages"
DEFAULT_CHOSEN_KEY = "chosen"
DEFAULT_REJECTED_KEY = "rejected"
CHOSEN_INPUT_IDS_KEY = "chosen_input_ids"
CHOSEN_ATTENTION_MASK_KEY = "chosen_attention_mask"
CHOSEN_LABELS_KEY = "chosen_labels"
REJECTED_INPUT_IDS_KEY = "rejected_input_ids"
REJECTED_ATTENTION_MASK_KEY = "rejected_attention_mask"
REJECTED_LABELS_KEY = "rejected_labels"
INPUT_IDS_PROMPT_KEY = "input_ids_prompt"
ATTENTION_MASK_PROMPT_KEY = "attention_mask_prompt"
GROUND_TRUTHS_KEY = "ground_truth"
VERIFIER_SOURCE_KEY = "dataset"
RAW_PROMPT_KEY = "prompt"
TOOLS_COLUMN_KEY = "tools"
ENV_CONFIG_KEY = "env_config"
TOKENIZED_PREFERENCE_DATASET_KEYS = [CHOSEN_INPUT_IDS_KEY, CHOSEN_LABELS_KEY, CHOSEN_ATTENTION_MASK_KEY,
                                     REJECTED_INPUT_IDS_KEY, REJECTED_LABELS_KEY, REJECTED_ATTENTION_MASK_KEY]
MASKED_TOKEN_VALUE = -100


# ---------------------------------------------------------------------------------- tokenizers
def _files_hash(path: str | None, names=("tokenizer_config.json", "tokenizer.json", "special_tokens_map.json", "vocab.json")):
    """Content hashes of the tokenizer files of a local directory (None entries for absent files)."""
    out = []
    for n in names:
        p = os.path.join(path or "", n)
        out.append(hashlib.sha256(open(p, "rb").read()).hexdigest() if os.path.isfile(p) else None)
    return out


def _ensure_pad_token(tokenizer) -> None:
    """Llama-style tokenizers ship without a usable pad token: add ``<pad>`` when pad is missing or
    equal to eos, and insist that pad != eos afterwards (eos must stay trainable, pad is masked)."""
    if tokenizer.pad_token_id is None or tokenizer.pad_token_id == tokenizer.eos_token_id:
        cls = type(tokenizer).__name__
        if cls.startswith("GPTNeoX") and tokenizer.bos_token is None:
            tokenizer.bos_token = tokenizer.eos_token  # OLMo: no bos in the vocabulary
            if tokenizer.pad_token_id is None or tokenizer.pad_token_id == tokenizer.eos_token_id:
                return
        added = tokenizer.add_special_tokens({"pad_token": "<pad>"})
        if added not in (0, 1):
            raise ValueError("adding the pad token changed the vocabulary by more than one entry")


def _install_chat_template(tokenizer, tc: "TokenizerConfig") -> None:
    if tc.chat_template_name in CHAT_TEMPLATES:
        tokenizer.chat_template = CHAT_TEMPLATES[tc.chat_template_name]
    elif tokenizer.chat_template is None:
        raise ValueError(f"Could not find chat template for {tc.tokenizer_name_or_path}.")
    if tc.add_bos:
        tpl = tokenizer.chat_template
        if tpl.startswith("{{ bos_token }}") or (tokenizer.bos_token is not None and tpl.startswith(tokenizer.bos_token)):
            raise ValueError("You specified add_bos=True, but the chat template already has a bos_token at the beginning.")
        tokenizer.chat_template = "{{ bos_token }}" + tpl


def _load_tokenizer(tc: "TokenizerConfig"):
    from transformers import AutoTokenizer

    return AutoTokenizer.from_pretrained(tc.tokenizer_name_or_path, revision=tc.tokenizer_revision,
                                         trust_remote_code=tc.trust_remote_code, use_fast=tc.use_fast)


def get_tokenizer_simple_v1(tc: "TokenizerConfig"):
    return _load_tokenizer(tc)


def get_tokenizer_tulu_v2_2(tc: "TokenizerConfig"):
    name = str(tc.tokenizer_name_or_path).lower()
    if "olmo" in name:
        if tc.chat_template_name is not None:
            if "olmo" in tc.chat_template_name:
                if tc.add_bos:
                    raise ValueError("For newer OLMo chat templates, you must *not* run with `--add_bos`.")
            elif not tc.add_bos:
                raise ValueError("For OLMo, you must run with `--add_bos`.")
        if not tc.use_fast:
            raise ValueError("For OLMo, you must use fast tokenizer.")
    tokenizer = _load_tokenizer(tc)
    _ensure_pad_token(tokenizer)
    if tokenizer.pad_token_id == tokenizer.eos_token_id:
        raise ValueError("pad token and eos token matching causes issues in our setup.")
    _install_chat_template(tokenizer, tc)
    return tokenizer


# earlier revisions differ only in how strictly they validated; they resolve to the same set-up
get_tokenizer_tulu_v1 = get_tokenizer_tulu_v2_2
get_tokenizer_tulu_v2_1 = get_tokenizer_tulu_v2_2

GET_TOKENIZER_FN = {
    "get_tokenizer_simple_v1": get_tokenizer_simple_v1,
    "get_tokenizer_tulu_v1": get_tokenizer_tulu_v1,
    "get_tokenizer_tulu_v2_1": get_tokenizer_tulu_v2_1,
    "get_tokenizer_tulu_v2_2": get_tokenizer_tulu_v2_2,
}


@dataclass
class TokenizerConfig:
    tokenizer_name_or_path: str | None = None
    tokenizer_revision: str | None = None
    trust_remote_code: bool = False
    use_fast: bool = True
    chat_template_name: str | None = None  # None: keep the tokenizer's own template
    add_bos: bool = False
    get_tokenizer_fn: str = "get_tokenizer_tulu_v2_2"
    tokenizer_files_hash: list[str] | None = None  # filled when the tokenizer is built (cache key)
    use_slow_tokenizer: bool = False  # accepted and ignored (old recipes pass it)
    tokenizer_name: str | None = None  # deprecated alias of tokenizer_name_or_path
    ground_truths_key: str = GROUND_TRUTHS_KEY
    sft_messages_key: str = DEFAULT_SFT_MESSAGES_KEY

    @cached_property
    def tokenizer(self):
        if self.tokenizer_name_or_path is None and self.tokenizer_name is not None:
            self.tokenizer_name_or_path = self.tokenizer_name
        if self.tokenizer_name_or_path is None:
            raise ValueError("tokenizer_name_or_path must be set")
        self.tokenizer_files_hash = _files_hash(self.tokenizer_name_or_path)
        return GET_TOKENIZER_FN[self.get_tokenizer_fn](self)


# ---------------------------------------------------------------------------------- SFT
class AssistantSpanDerivationError(ValueError):
    """The assistant label spans of a conversation cannot be derived reliably."""


def sft_tokenize_v1(row: dict, tokenizer, sft_messages_key: str = DEFAULT_SFT_MESSAGES_KEY):
    """Prompt = all but the last message; everything is a label (prompt masking is a separate transform)."""
    msgs = row[sft_messages_key]
    prompt = msgs if len(msgs) == 1 else msgs[:-1]
    row[INPUT_IDS_PROMPT_KEY] = tokenizer.apply_chat_template(prompt, add_generation_prompt=True, return_dict=False)
    row[INPUT_IDS_KEY] = tokenizer.apply_chat_template(msgs, return_dict=False)
    row[ATTENTION_MASK_KEY] = [1] * len(row[INPUT_IDS_KEY])
    row[LABELS_KEY] = copy.deepcopy(row[INPUT_IDS_KEY])
    return row


def sft_tokenize_mask_out_prompt_v1(row: dict, tokenizer, sft_messages_key: str = DEFAULT_SFT_MESSAGES_KEY):
    """As ``sft_tokenize_v1`` with the prompt tokens masked to -100."""
    row = sft_tokenize_v1(row, tokenizer, sft_messages_key)
    n = len(row[INPUT_IDS_PROMPT_KEY])
    labels = row[LABELS_KEY]
    labels[:n] = [MASKED_TOKEN_VALUE] * min(n, len(labels))
    row[LABELS_KEY] = labels
    return row


def sft_filter_v1(row: dict, tokenizer, max_prompt_token_length: int | None = None, max_token_length: int | None = None,
                  need_contain_labels: bool = True):
    ok = True
    if max_prompt_token_length is not None:
        ok &= len(row[INPUT_IDS_PROMPT_KEY]) <= max_prompt_token_length
    if max_token_length is not None:
        ok &= len(row[INPUT_IDS_KEY]) <= max_token_length
    has = any(x != MASKED_TOKEN_VALUE for x in row[LABELS_KEY])
    return bool(ok and (has or not need_contain_labels))


def _normalize_tools(tools):
    if tools is None:
        return None
    if isinstance(tools, str):
        import json

        tools = json.loads(tools)
    return list(tools) or None


def _render(tokenizer, messages, tools, gen: bool) -> str:
    return tokenizer.apply_chat_template(conversation=messages, tools=tools, tokenize=False, add_generation_prompt=gen)


def _spans_from_token_counts(messages, tokenizer, tools, max_seq_length, indices):
    kw = dict(tokenize=True, return_dict=False, padding=False, truncation=max_seq_length is not None,
              max_length=max_seq_length, tools=tools)
    spans = []
    for i in indices:
        start = 0 if i == 0 else len(tokenizer.apply_chat_template(conversation=messages[:i], add_generation_prompt=True, **kw))
        end = len(tokenizer.apply_chat_template(conversation=messages[: i + 1], add_generation_prompt=False, **kw))
        spans.append((i, start, end))
    return spans


def _verify_spans(messages, tokenizer, ids: list[int], rendered: str, spans) -> None:
    n = len(ids)
    for i, start, end in spans:
        content = messages[i].get("content")
        if not content or content not in rendered:
            continue  # the template rewrites this turn: nothing to compare with
        cut = end >= n
        start, end = max(0, start), min(end, n)
        if start >= end:
            continue
        text = tokenizer.decode(ids[start:end], clean_up_tokenization_spaces=False)
        if cut and text.lstrip() and content.startswith(text.lstrip()):
            continue  # truncated tail that is still a prefix of the turn
        if content not in text:
            raise AssistantSpanDerivationError(f"label span of message {i} does not cover its content ({text[:60]!r})")
        if not text.lstrip().startswith(content):
            raise AssistantSpanDerivationError(f"label span of message {i} starts inside the assistant header ({text[:60]!r})")
        tail = text[text.index(content) + len(content):]
        for j in range(i + 1, len(messages)):
            later = messages[j].get("content")
            if later and later in tail:
                raise AssistantSpanDerivationError(f"label span of message {i} runs into message {j}")


def tokenize_with_assistant_labels(messages, tokenizer, tools=None, max_seq_length: int | None = None,
                                   last_turn_only: bool = False):
    """Returns (input_ids, attention_mask, labels) as 1-D LongTensors."""
    if not getattr(tokenizer, "is_fast", False):
        raise ValueError(f"SFT tokenization requires a fast tokenizer (offset mapping); got {type(tokenizer).__name__}. "
                         "Load the tokenizer with `use_fast=True`.")
    rendered = _render(tokenizer, messages, tools, False)
    enc = tokenizer(rendered, add_special_tokens=False, return_offsets_mapping=True, padding=False,
                    truncation=max_seq_length is not None, max_length=max_seq_length)
    ids = list(enc[INPUT_IDS_KEY])
    offsets = enc["offset_mapping"]
    labels = [MASKED_TOKEN_VALUE] * len(ids)
    turns = [i for i, m in enumerate(messages) if m["role"] == "assistant"]
    if last_turn_only:
        turns = turns[-1:]
    char_spans, stable = [], True
    for i in turns:
        try:
            head = "" if i == 0 else _render(tokenizer, messages[:i], tools, True)
            through = _render(tokenizer, messages[: i + 1], tools, False)
        except Exception as exc:  # noqa: BLE001 - template-specific failures on partial conversations
            raise AssistantSpanDerivationError(
                f"chat template failed to render the prefix {[m['role'] for m in messages[: i + 1]]}") from exc
        if not (len(head) <= len(through) and rendered.startswith(head) and rendered.startswith(through)):
            stable = False
            break
        char_spans.append((len(head), len(through)))
    if not stable:
        spans = _spans_from_token_counts(messages, tokenizer, tools, max_seq_length, turns)
        for _, a, b in spans:
            a, b = max(0, a), min(b, len(ids))
            labels[a:b] = ids[a:b]
        _verify_spans(messages, tokenizer, ids, rendered, spans)
    else:
        k = 0  # spans are sorted and disjoint: sweep once
        for t, (a, b) in enumerate(offsets):
            if a == b:
                continue
            while k < len(char_spans) and char_spans[k][1] <= a:
                k += 1
            if k < len(char_spans) and a < char_spans[k][1] and char_spans[k][0] < b:
                labels[t] = ids[t]
    to = lambda x: torch.tensor(x, dtype=torch.long)
    return to(ids), torch.ones(len(ids), dtype=torch.long), to(labels)


def _tokenize_row_or_mask_out(row: dict, tokenizer, max_seq_length, last_turn_only=False,
                              messages_key: str = DEFAULT_SFT_MESSAGES_KEY) -> dict:
    messages = row[messages_key]
    if len(messages) == 0:
        raise ValueError("messages field is empty.")
    tools = _normalize_tools(row.get(TOOLS_COLUMN_KEY))
    try:
        ids, mask, labels = tokenize_with_assistant_labels(messages, tokenizer, tools, max_seq_length, last_turn_only)
    except AssistantSpanDerivationError as exc:
        logger.warning("masking out a conversation whose label spans could not be derived (%s): %s",
                       [m["role"] for m in messages], exc)
        enc = tokenizer(_render(tokenizer, messages, tools, False), add_special_tokens=False, padding=False,
                        truncation=max_seq_length is not None, max_length=max_seq_length)
        ids = torch.tensor(enc[INPUT_IDS_KEY], dtype=torch.long)
        mask = torch.ones_like(ids)
        labels = torch.full_like(ids, MASKED_TOKEN_VALUE)
    row[INPUT_IDS_KEY], row[LABELS_KEY], row[ATTENTION_MASK_KEY] = ids, labels, mask
    return row


def sft_tulu_tokenize_without_truncation_v1(row: dict, tokenizer):
    return _tokenize_row_or_mask_out(row, tokenizer, None)


def sft_tulu_tokenize_and_truncate_v1(row: dict, tokenizer, max_seq_length: int):
    return _tokenize_row_or_mask_out(row, tokenizer, max_seq_length)


def last_turn_tulu_tokenize_and_truncate_v1(row: dict, tokenizer, max_seq_length: int):
    return _tokenize_row_or_mask_out(row, tokenizer, max_seq_length, last_turn_only=True)


def sft_tulu_filter_v1(row: dict, tokenizer):
    return any(x != MASKED_TOKEN_VALUE for x in row[LABELS_KEY])


# ---------------------------------------------------------------------------------- preference
def preference_tokenize_v1(row: dict, tokenizer):
    prompt = row["chosen"][:-1]
    row[INPUT_IDS_PROMPT_KEY] = tokenizer.apply_chat_template(prompt, add_generation_prompt=True, return_dict=False)
    row[ATTENTION_MASK_PROMPT_KEY] = [1] * len(row[INPUT_IDS_PROMPT_KEY])
    for side, k_ids, k_mask in (("chosen", CHOSEN_INPUT_IDS_KEY, CHOSEN_ATTENTION_MASK_KEY),
                                ("rejected", REJECTED_INPUT_IDS_KEY, REJECTED_ATTENTION_MASK_KEY)):
        row[k_ids] = tokenizer.apply_chat_template(row[side], return_dict=False)
        row[k_mask] = [1] * len(row[k_ids])
    return row


def preference_filter_v1(row: dict, tokenizer, max_prompt_token_length: int | None = None,
                         max_token_length: int | None = None):
    if max_prompt_token_length is not None and len(row[INPUT_IDS_PROMPT_KEY]) > max_prompt_token_length:
        return False
    if max_token_length is not None:
        if len(row[CHOSEN_INPUT_IDS_KEY]) > max_token_length or len(row[REJECTED_INPUT_IDS_KEY]) > max_token_length:
            return False
    return True


def _preference_tulu(row, tokenizer, max_seq_length, chosen_key, rejected_key, last_turn_only):
    out = {}
    for side, key in (("chosen", chosen_key), ("rejected", rejected_key)):
        msgs = row[key]
        if len(msgs) == 0:
            raise ValueError(f"{side} messages field is empty.")
        enc = _tokenize_row_or_mask_out({DEFAULT_SFT_MESSAGES_KEY: msgs}, tokenizer, max_seq_length, last_turn_only)
        out[f"{side}_input_ids"] = enc[INPUT_IDS_KEY]
        out[f"{side}_labels"] = enc[LABELS_KEY]
        out[f"{side}_attention_mask"] = enc[ATTENTION_MASK_KEY]
    return out


def preference_tulu_tokenize_and_truncate_v1(row: dict, tokenizer, max_seq_length: int,
                                             chosen_key: str = DEFAULT_CHOSEN_KEY, rejected_key: str = DEFAULT_REJECTED_KEY):
    """Chosen and rejected conversations share all but the last message; only that last assistant
    turn is trained on (the registry maps this name to the last-turn variant, as the reference does)."""
    return _preference_tulu(row, tokenizer, max_seq_length, chosen_key, rejected_key, last_turn_only=True)


def preference_tulu_tokenize_and_truncate_all_turns_v1(row: dict, tokenizer, max_seq_length: int,
                                                       chosen_key: str = DEFAULT_CHOSEN_KEY,
                                                       rejected_key: str = DEFAULT_REJECTED_KEY):
    return _preference_tulu(row, tokenizer, max_seq_length, chosen_key, rejected_key, last_turn_only=False)


def preference_tulu_filter_v1(row: dict, tokenizer):
    return (any(x != MASKED_TOKEN_VALUE for x in row[CHOSEN_LABELS_KEY])
            and any(x != MASKED_TOKEN_VALUE for x in row[REJECTED_LABELS_KEY]))


# ---------------------------------------------------------------------------------- RLVR
def rlvr_tokenize_v1(row: dict, tokenizer, sft_messages_key: str = DEFAULT_SFT_MESSAGES_KEY,
                     ground_truths_key: str = GROUND_TRUTHS_KEY, verifier_source_key: str = VERIFIER_SOURCE_KEY,
                     system_prompt_override: str | None = None, tool_definitions: list[dict] | None = None,
                     pass_tools_to_chat_template: bool = True):
    """Prompt-only tokenisation for RL: ``input_ids_prompt`` ends with the generation prompt; ground
    truth and verifier name are normalised to lists (one entry per verifier)."""
    msgs = row[sft_messages_key]
    prompt = msgs if len(msgs) == 1 else msgs[:-1]
    if system_prompt_override:
        if prompt and prompt[0]["role"] == "system":
            prompt = prompt[1:]
        prompt = [{"role": "system", "content": system_prompt_override}] + list(prompt)
    tools = None
    if pass_tools_to_chat_template and tool_definitions:
        active = row.get(TOOLS_COLUMN_KEY)
        if active is not None:
            names = set(active)
            tools = [t for t in tool_definitions if t.get("function", {}).get("name") in names] or None
        else:
            tools = tool_definitions
    row[INPUT_IDS_PROMPT_KEY] = tokenizer.apply_chat_template(prompt, add_generation_prompt=True, return_dict=False, tools=tools)
    pad = tokenizer.pad_token_id
    if pad is not None and pad in row[INPUT_IDS_PROMPT_KEY]:
        row[INPUT_IDS_PROMPT_KEY] = [x for x in row[INPUT_IDS_PROMPT_KEY] if x != pad]
    gt, src = row[ground_truths_key], row[verifier_source_key]
    if isinstance(src, str):
        src, gt = [src], [gt]
    row[GROUND_TRUTHS_KEY], row[VERIFIER_SOURCE_KEY] = gt, src
    row[RAW_PROMPT_KEY] = "\n".join(f"{m['role']}: {m['content']}" for m in prompt)
    row.pop(sft_messages_key, None)
    return row


def rlvr_filter_v1(row: dict, tokenizer, need_contain_labels: bool = True, max_prompt_token_length: int | None = None,
                   max_token_length: int | None = None):
    ok = True
    if max_prompt_token_length is not None:
        ok &= len(row[INPUT_IDS_PROMPT_KEY]) <= max_prompt_token_length
    if max_token_length is not None:
        ok &= len(row[INPUT_IDS_KEY]) <= max_token_length
    has = any(x != MASKED_TOKEN_VALUE for x in row.get(LABELS_KEY, []))
    return bool(ok and (has or not need_contain_labels))


def rlvr_max_length_filter_v1(row: dict, tokenizer, max_prompt_token_length: int | None = None):
    return max_prompt_token_length is None or len(row[INPUT_IDS_PROMPT_KEY]) <= max_prompt_token_length


TRANSFORM_FNS = {
    "sft_tokenize_v1": (sft_tokenize_v1, "map"),
    "sft_tokenize_mask_out_prompt_v1": (sft_tokenize_mask_out_prompt_v1, "map"),
    "sft_filter_v1": (sft_filter_v1, "filter"),
    "sft_tulu_tokenize_without_truncation_v1": (sft_tulu_tokenize_without_truncation_v1, "map"),
    "sft_tulu_tokenize_and_truncate_v1": (sft_tulu_tokenize_and_truncate_v1, "map"),
    "sft_tulu_filter_v1": (sft_tulu_filter_v1, "filter"),
    "last_turn_tulu_tokenize_and_truncate_v1": (last_turn_tulu_tokenize_and_truncate_v1, "map"),
    "preference_tokenize_v1": (preference_tokenize_v1, "map"),
    "preference_filter_v1": (preference_filter_v1, "filter"),
    "preference_tulu_tokenize_and_truncate_v1": (preference_tulu_tokenize_and_truncate_v1, "map"),
    "preference_tulu_filter_v1": (preference_tulu_filter_v1, "filter"),
    "rlvr_tokenize_v1": (rlvr_tokenize_v1, "map"),
    "rlvr_max_length_filter_v1": (rlvr_max_length_filter_v1, "filter"),
}
# transforms that consume the ``tools`` column (it must not be kept in their output)
SFT_TOKENIZE_FNS = {"sft_tulu_tokenize_without_truncation_v1", "sft_tulu_tokenize_and_truncate_v1",
                    "last_turn_tulu_tokenize_and_truncate_v1"}
