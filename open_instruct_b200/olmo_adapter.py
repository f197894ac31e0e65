"""Sequence-classification (reward-model) heads for the OLMo families in transformers.

transformers ships ``...ForCausalLM`` for OLMo-2, OLMo-3, OLMoE and OLMo-Hybrid but no ``...ForSequenceClassification``, so a
reward model exported by ``reward_modeling.save_reward_model`` for one of them could not be opened with
``AutoModelForSequenceClassification``.  The reference closes that gap with hand-written classes in
``open_instruct/olmo_adapter/__init__.py``; here the classes are transformers' own generic head (backbone + bias-free ``score``
linear, last-non-pad-token pooling) bound to each family's backbone, registered with the auto class on import:

    import open_instruct_b200.olmo_adapter  # noqa: F401
    rm = transformers.AutoModelForSequenceClassification.from_pretrained(folder)
"""

from __future__ import annotations

import transformers
from transformers.modeling_layers import GenericForSequenceClassification

REGISTERED: dict[str, type] = {}


def _register(prefix: str) -> None:
    base = getattr(transformers, f"{prefix}PreTrainedModel", None)
    cfg = getattr(transformers, f"{prefix}Config", None)
    if base is None or cfg is None or hasattr(transformers, f"{prefix}ForSequenceClassification"):
        return
    cls = type(f"{prefix}ForSequenceClassification", (GenericForSequenceClassification, base), {"__doc__": f"{prefix} backbone with a scalar-per-label head."})
    try:
        transformers.AutoModelForSequenceClassification.register(cfg, cls)
    except ValueError:   # another import registered one already
        return
    REGISTERED[cfg.model_type] = cls


for _prefix in ("Olmo2", "Olmo3", "Olmoe", "OlmoHybrid"):
    _register(_prefix)
