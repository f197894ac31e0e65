"""Model description and flat parameter layout.

A decoder is described by a ``ModelSpec`` (convertible from / to a Hugging Face ``config.json``
for the Llama, Qwen2/2.5/3, Mistral, OLMo-2/3, OLMoE and OLMo-Hybrid families) and
its weights live in ONE flat buffer laid out in consumer order with the fused shapes the
kernels use (``wqkv`` = q|k|v rows, ``w_gate_up`` = gate|up rows).  Hugging Face names are only a
view used for checkpoint I/O.  Parameters that take no weight decay (norm weights, biases) are
grouped at the end of the buffer so that the sharded optimizer sees two contiguous regions.
"""

from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field
from pathlib import Path


def _rope_scaling_of(cfg: dict) -> dict | None:
    """The RoPE scaling rule of a config.json: ``rope_scaling`` (older form), else ``rope_parameters`` when it names a rule
    other than the default (the form transformers 5 writes)."""
    sc = cfg.get("rope_scaling")
    if sc:
        return sc
    rp = cfg.get("rope_parameters") or {}
    if rp.get("rope_type", rp.get("type", "default")) not in ("default", None):
        return {k: v for k, v in rp.items() if k != "rope_theta"}
    return None


@dataclass
class ModelSpec:
    vocab_size: int = 128256
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    rope_scaling: dict | None = None
    max_position_embeddings: int = 131072
    tie_word_embeddings: bool = False
    qk_norm: bool = False  # RMSNorm of q and k before RoPE: per head (Qwen3), or over the whole projection (``qk_norm_full``)
    qk_norm_full: bool = False  # OLMo-2 / OLMo-3: one norm over all heads of q (weight [q_dim]) and one over all heads of k
    post_norm: bool = False     # OLMo-2 / OLMo-3 block: h += norm(attn(h)); h += norm(mlp(h)) instead of norming the inputs
    # mixture of experts (OLMoE): every decoder layer's MLP is ``num_experts`` SwiGLU experts of width ``intermediate_size`` behind
    # a linear router; a token goes to its ``num_experts_per_tok`` best experts, weighted by their softmax probabilities
    num_experts: int = 0
    num_experts_per_tok: int = 0
    norm_topk_prob: bool = False
    router_aux_loss_coef: float = 0.01
    sliding_window: int | None = None  # some layers attend to the last N tokens only (OLMo-3, Mistral v0.1): documents up to N are exact
    attention_bias: bool = False  # Qwen2 style q/k/v bias
    # per-layer kinds: "attention" (attends to the whole document), "sliding" (to the last ``sliding_window`` tokens: three of
    # four layers in OLMo-3), "gdn" (OLMo-Hybrid's gated DeltaNet: a linear-attention layer with a [key_dim, value_dim] state per
    # head instead of a KV cache; a pre-norm block, while the attention layers follow ``post_norm`` / ``qk_norm_full``).
    # None: all layers are attention layers, windowed when ``sliding_window`` is set (Mistral v0.1).
    layer_types: tuple | None = None
    gdn_key_heads: int = 0
    gdn_value_heads: int = 0
    gdn_key_dim: int = 0       # per head
    gdn_value_dim: int = 0     # per head
    gdn_conv: int = 4          # taps of the causal depthwise convolution on q, k and v
    gdn_neg_eigval: bool = True  # beta in (0, 2) instead of (0, 1)
    use_rope: bool = True      # False: attention without positional rotation (OLMo-Hybrid without ``rope_theta``)
    model_type: str = "llama"
    bos_token_id: int | None = None
    eos_token_id: int | None = None
    pad_token_id: int | None = None

    # ---- derived
    @property
    def q_dim(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def qkv_dim(self) -> int:
        return self.q_dim + 2 * self.kv_dim

    @property
    def attn_scale(self) -> float:
        """Softmax scale of the attention layers: ``head_dim ** -0.5``, times the square of the factor YaRN puts on cos / sin
        (q and k both carry it; the rotation itself stays unscaled here)."""
        from ..ops.ref import rope_attention_factor

        return self.head_dim ** -0.5 * rope_attention_factor(self.rope_scaling) ** 2

    def is_gdn(self, i: int) -> bool:
        return self.layer_types is not None and self.layer_types[i] == "gdn"

    @property
    def has_gdn(self) -> bool:
        return self.layer_types is not None and "gdn" in self.layer_types

    def window(self, i: int) -> int | None:
        """How many of the latest tokens (itself included) a token of layer ``i`` attends to; None: all of them."""
        if not self.sliding_window:
            return None
        return self.sliding_window if (self.layer_types is None or self.layer_types[i] == "sliding") else None

    @property
    def min_window(self) -> int | None:
        """The shortest attention window of any layer (None: no layer is windowed)."""
        ws = [w for w in (self.window(i) for i in range(self.num_layers)) if w]
        return min(ws) if ws else None

    @property
    def gdn_k_total(self) -> int:
        return self.gdn_key_heads * self.gdn_key_dim

    @property
    def gdn_v_total(self) -> int:
        return self.gdn_value_heads * self.gdn_value_dim

    @property
    def gdn_in_rows(self) -> int:
        """Rows of the fused input projection of a gdn layer: q | k | v | output gate | a (decay) | b (beta)."""
        return 2 * self.gdn_k_total + 2 * self.gdn_v_total + 2 * self.gdn_value_heads

    def num_params(self) -> int:
        return ParamLayout(self).total

    # ---- HF config.json
    @classmethod
    def from_hf_config(cls, cfg: dict) -> "ModelSpec":
        mt = cfg.get("model_type", "llama")
        heads = cfg["num_attention_heads"]
        hd = cfg.get("head_dim") or cfg["hidden_size"] // heads
        hybrid = {}
        if mt == "olmo_hybrid":
            n = cfg["num_hidden_layers"]
            kinds = cfg.get("layer_types") or [("full_attention" if (i % 4 == 3 or (n < 4 and i == n - 1)) else "linear_attention") for i in range(n)]
            kh = cfg.get("linear_num_key_heads") or heads
            kd = cfg.get("linear_key_head_dim") or int(0.75 * cfg["hidden_size"] / kh)
            rp = cfg.get("rope_parameters") or {}
            hybrid = dict(layer_types=tuple("attention" if k == "full_attention" else "gdn" for k in kinds), gdn_key_heads=kh,
                          gdn_value_heads=cfg.get("linear_num_value_heads") or heads, gdn_key_dim=kd,
                          gdn_value_dim=cfg.get("linear_value_head_dim") or 2 * kd, gdn_conv=cfg.get("linear_conv_kernel_dim", 4),
                          gdn_neg_eigval=bool(cfg.get("linear_allow_neg_eigval", True)),
                          use_rope=(cfg.get("rope_theta") or rp.get("rope_theta")) is not None)
        windowed = cfg.get("sliding_window") and (mt == "olmo3" or cfg.get("use_sliding_window", mt == "mistral"))
        if windowed and mt != "olmo_hybrid":
            # which layers are windowed: the config's own list, else the family's rule (OLMo-3: three of four; Qwen2 / Qwen3: the
            # layers from ``max_window_layers`` up; Mistral v0.1: all, which is what ``layer_types`` None means)
            n = cfg["num_hidden_layers"]
            kinds = cfg.get("layer_types")
            if not kinds and mt == "olmo3":
                kinds = [("sliding_attention" if (i + 1) % 4 else "full_attention") for i in range(n)]
            if not kinds and mt in ("qwen2", "qwen3") and cfg.get("max_window_layers") is not None:
                kinds = [("sliding_attention" if i >= cfg["max_window_layers"] else "full_attention") for i in range(n)]
            if kinds and "sliding_attention" in kinds and "full_attention" in kinds:
                hybrid = dict(layer_types=tuple("sliding" if k == "sliding_attention" else "attention" for k in kinds))
            elif kinds and "sliding_attention" not in kinds:
                windowed = False
        return cls(
            **hybrid,
            vocab_size=cfg["vocab_size"],
            hidden_size=cfg["hidden_size"],
            intermediate_size=cfg["intermediate_size"],
            num_layers=cfg["num_hidden_layers"],
            num_heads=heads,
            num_kv_heads=cfg.get("num_key_value_heads", heads),
            head_dim=hd,
            rms_norm_eps=cfg.get("rms_norm_eps", 1e-5),
            rope_theta=cfg.get("rope_theta") or (cfg.get("rope_parameters") or {}).get("rope_theta") or 10000.0,
            rope_scaling=_rope_scaling_of(cfg),
            max_position_embeddings=cfg.get("max_position_embeddings", 8192),
            tie_word_embeddings=cfg.get("tie_word_embeddings", False),
            qk_norm=mt in ("qwen3", "olmo2", "olmo3", "olmoe", "olmo_hybrid"),
            qk_norm_full=mt in ("olmo2", "olmo3", "olmoe", "olmo_hybrid"),
            num_experts=cfg.get("num_experts", 0) if mt == "olmoe" else 0,
            num_experts_per_tok=cfg.get("num_experts_per_tok", 0) if mt == "olmoe" else 0,
            norm_topk_prob=bool(cfg.get("norm_topk_prob", False)),
            router_aux_loss_coef=cfg.get("router_aux_loss_coef", 0.01),
            post_norm=mt in ("olmo2", "olmo3", "olmo_hybrid"),
            sliding_window=cfg.get("sliding_window") if windowed else None,
            attention_bias=cfg.get("attention_bias", mt == "qwen2"),
            model_type=mt,
            bos_token_id=cfg.get("bos_token_id"),
            eos_token_id=cfg.get("eos_token_id") if not isinstance(cfg.get("eos_token_id"), list) else cfg["eos_token_id"][0],
            pad_token_id=cfg.get("pad_token_id"),
        )

    @classmethod
    def from_pretrained(cls, path: str) -> "ModelSpec":
        return cls.from_hf_config(json.loads((Path(path) / "config.json").read_text()))

    def to_hf_config(self) -> dict:
        arch = {"llama": "LlamaForCausalLM", "qwen2": "Qwen2ForCausalLM", "qwen3": "Qwen3ForCausalLM",
                "mistral": "MistralForCausalLM", "olmo2": "Olmo2ForCausalLM", "olmo3": "Olmo3ForCausalLM",
                "olmoe": "OlmoeForCausalLM", "olmo_hybrid": "OlmoHybridForCausalLM"}.get(self.model_type, "LlamaForCausalLM")
        cfg = {
            "architectures": [arch],
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_layers,
            "num_attention_heads": self.num_heads,
            "num_key_value_heads": self.num_kv_heads,
            "head_dim": self.head_dim,
            "hidden_act": "silu",
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling,
            # the form newer transformers releases read and write (``rope_scaling`` above is what older ones and the hub's
            # Llama-3.1 configs carry)
            "rope_parameters": {"rope_theta": self.rope_theta, **(self.rope_scaling or {"rope_type": "default"})},
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "mlp_bias": False,
            "torch_dtype": "bfloat16",
            "bos_token_id": self.bos_token_id,
            "eos_token_id": self.eos_token_id,
            "pad_token_id": self.pad_token_id,
            "use_cache": True,
        }
        if self.sliding_window:
            cfg["sliding_window"] = self.sliding_window
            if self.model_type not in ("mistral", "olmo3"):
                cfg["use_sliding_window"] = True
        if self.layer_types is not None and not self.has_gdn:
            cfg["layer_types"] = ["sliding_attention" if k == "sliding" else "full_attention" for k in self.layer_types]
        if self.has_gdn:
            cfg.update({"layer_types": ["full_attention" if k == "attention" else "linear_attention" for k in self.layer_types],
                        "linear_num_key_heads": self.gdn_key_heads, "linear_num_value_heads": self.gdn_value_heads,
                        "linear_key_head_dim": self.gdn_key_dim, "linear_value_head_dim": self.gdn_value_dim,
                        "linear_conv_kernel_dim": self.gdn_conv, "linear_allow_neg_eigval": self.gdn_neg_eigval})
            if not self.use_rope:
                cfg.update({"rope_theta": None, "rope_scaling": None, "rope_parameters": {"rope_type": "default", "rope_theta": None}})
        if self.num_experts:
            cfg.update({"num_experts": self.num_experts, "num_experts_per_tok": self.num_experts_per_tok, "norm_topk_prob": self.norm_topk_prob,
                        "router_aux_loss_coef": self.router_aux_loss_coef})
        return cfg

    def replace(self, **kw) -> "ModelSpec":
        return dataclasses.replace(self, **kw)


LLAMA31_SCALING = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                   "original_max_position_embeddings": 8192}

OLMO3_YARN = {"rope_type": "yarn", "factor": 8.0, "original_max_position_embeddings": 8192, "attention_factor": 1.2079441541679836,
              "beta_fast": 32.0, "beta_slow": 1.0}

PRESETS: dict[str, ModelSpec] = {
    # the CPU plumbing configuration: 2 layers, d 64, 4 heads, ffn 256, vocab 512, theta 1e4
    "tiny": ModelSpec(vocab_size=512, hidden_size=64, intermediate_size=256, num_layers=2, num_heads=4,
                      num_kv_heads=4, head_dim=16, rope_theta=1e4, max_position_embeddings=2048),
    # tiny but with head_dim 128 so the tcgen05 attention path is exercised
    # tiny, head_dim 128, heads that divide by 2: the smallest model tensor and sequence parallelism can split
    "tiny128-tp": ModelSpec(vocab_size=512, hidden_size=512, intermediate_size=1024, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=128,
                            rope_theta=10000.0, max_position_embeddings=4096),
    "tiny128": ModelSpec(vocab_size=512, hidden_size=256, intermediate_size=512, num_layers=2, num_heads=2,
                         num_kv_heads=1, head_dim=128, rope_theta=1e4, max_position_embeddings=4096),
    "llama3.2-1b": ModelSpec(vocab_size=128256, hidden_size=2048, intermediate_size=8192, num_layers=16,
                             num_heads=32, num_kv_heads=8, head_dim=64, rope_scaling=dict(LLAMA31_SCALING, factor=32.0),
                             tie_word_embeddings=True),
    "llama3.1-8b": ModelSpec(rope_scaling=dict(LLAMA31_SCALING)),
    "llama3.1-70b": ModelSpec(hidden_size=8192, intermediate_size=28672, num_layers=80, num_heads=64, num_kv_heads=8,
                              rope_scaling=dict(LLAMA31_SCALING)),
    "qwen2.5-7b": ModelSpec(vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_layers=28, num_heads=28,
                            num_kv_heads=4, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, attention_bias=True,
                            model_type="qwen2", max_position_embeddings=32768),
    "qwen2.5-14b": ModelSpec(vocab_size=152064, hidden_size=5120, intermediate_size=13824, num_layers=48, num_heads=40,
                             num_kv_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, attention_bias=True,
                             model_type="qwen2", max_position_embeddings=32768),
    "qwen2.5-32b": ModelSpec(vocab_size=152064, hidden_size=5120, intermediate_size=27648, num_layers=64, num_heads=40,
                             num_kv_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, attention_bias=True,
                             model_type="qwen2", max_position_embeddings=32768),
    "qwen3-0.6b": ModelSpec(vocab_size=151936, hidden_size=1024, intermediate_size=3072, num_layers=28, num_heads=16,
                            num_kv_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, qk_norm=True,
                            model_type="qwen3", tie_word_embeddings=True, max_position_embeddings=40960),
    "olmo2-7b": ModelSpec(vocab_size=100352, hidden_size=4096, intermediate_size=11008, num_layers=32, num_heads=32,
                          num_kv_heads=32, head_dim=128, rms_norm_eps=1e-6, rope_theta=5e5, model_type="olmo2",
                          qk_norm=True, qk_norm_full=True, post_norm=True, max_position_embeddings=4096),
    "qwen3-1.7b": ModelSpec(vocab_size=151936, hidden_size=2048, intermediate_size=6144, num_layers=28, num_heads=16, num_kv_heads=8,
                            head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, qk_norm=True, model_type="qwen3", tie_word_embeddings=True,
                            max_position_embeddings=40960),
    "smollm2-135m": ModelSpec(vocab_size=49152, hidden_size=576, intermediate_size=1536, num_layers=30, num_heads=9, num_kv_heads=3,
                              head_dim=64, rms_norm_eps=1e-5, rope_theta=1e5, tie_word_embeddings=True, max_position_embeddings=8192),
    "olmo2-1b": ModelSpec(vocab_size=100352, hidden_size=2048, intermediate_size=8192, num_layers=16, num_heads=16, num_kv_heads=16,
                          head_dim=128, rms_norm_eps=1e-6, rope_theta=5e5, model_type="olmo2", qk_norm=True, qk_norm_full=True, post_norm=True,
                          max_position_embeddings=4096),
    "olmo2-13b": ModelSpec(vocab_size=100352, hidden_size=5120, intermediate_size=13824, num_layers=40, num_heads=40, num_kv_heads=40,
                           head_dim=128, rms_norm_eps=1e-6, rope_theta=5e5, model_type="olmo2", qk_norm=True, qk_norm_full=True, post_norm=True,
                           max_position_embeddings=4096),
    "olmo2-32b": ModelSpec(vocab_size=100352, hidden_size=5120, intermediate_size=27648, num_layers=64, num_heads=40, num_kv_heads=8,
                           head_dim=128, rms_norm_eps=1e-6, rope_theta=5e5, model_type="olmo2", qk_norm=True, qk_norm_full=True, post_norm=True,
                           max_position_embeddings=4096),
    # OLMo-3: three sliding-window layers (4096 tokens) per full-attention layer, YaRN-extended context
    "olmo3-7b": ModelSpec(vocab_size=100278, hidden_size=4096, intermediate_size=11008, num_layers=32, num_heads=32, num_kv_heads=32,
                          head_dim=128, rms_norm_eps=1e-6, rope_theta=5e5, model_type="olmo3", qk_norm=True, qk_norm_full=True, post_norm=True,
                          sliding_window=4096, layer_types=tuple("attention" if i % 4 == 3 else "sliding" for i in range(32)),
                          rope_scaling=dict(OLMO3_YARN), max_position_embeddings=65536),
    "olmo3-32b": ModelSpec(vocab_size=100278, hidden_size=5120, intermediate_size=27648, num_layers=64, num_heads=40, num_kv_heads=8,
                           head_dim=128, rms_norm_eps=1e-6, rope_theta=5e5, model_type="olmo3", qk_norm=True, qk_norm_full=True, post_norm=True,
                           sliding_window=4096, layer_types=tuple("attention" if i % 4 == 3 else "sliding" for i in range(64)),
                           rope_scaling=dict(OLMO3_YARN), max_position_embeddings=65536),
    "olmoe-1b-7b": ModelSpec(vocab_size=50304, hidden_size=2048, intermediate_size=1024, num_layers=16, num_heads=16, num_kv_heads=16,
                             head_dim=128, rms_norm_eps=1e-5, rope_theta=1e4, model_type="olmoe", qk_norm=True, qk_norm_full=True,
                             num_experts=64, num_experts_per_tok=8, norm_topk_prob=False, max_position_embeddings=4096),
    "qwen3-8b": ModelSpec(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_layers=36, num_heads=32, num_kv_heads=8,
                          head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, qk_norm=True, model_type="qwen3", max_position_embeddings=40960),
    "qwen3-32b": ModelSpec(vocab_size=151936, hidden_size=5120, intermediate_size=25600, num_layers=64, num_heads=64, num_kv_heads=8,
                           head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, qk_norm=True, model_type="qwen3", max_position_embeddings=40960),
    "mistral-7b-v0.3": ModelSpec(vocab_size=32768, hidden_size=4096, intermediate_size=14336, num_layers=32, num_heads=32, num_kv_heads=8,
                                 head_dim=128, rms_norm_eps=1e-5, rope_theta=1e6, model_type="mistral", max_position_embeddings=32768),
    "llama3.2-3b": ModelSpec(vocab_size=128256, hidden_size=3072, intermediate_size=8192, num_layers=28, num_heads=24, num_kv_heads=8,
                             head_dim=128, rope_scaling=dict(LLAMA31_SCALING, factor=32.0), tie_word_embeddings=True),
    # allenai/Olmo-Hybrid-7B: 24 gated-DeltaNet layers and 8 full-attention layers (every fourth), ``open_instruct/olmo_core_hybrid.py:154-175``
    "olmo-hybrid-7b": ModelSpec(vocab_size=100352, hidden_size=3840, intermediate_size=11008, num_layers=32, num_heads=30, num_kv_heads=30,
                                head_dim=128, rms_norm_eps=1e-6, model_type="olmo_hybrid", qk_norm=True, qk_norm_full=True, post_norm=True,
                                layer_types=tuple("attention" if i % 4 == 3 else "gdn" for i in range(32)), gdn_key_heads=30,
                                gdn_value_heads=30, gdn_key_dim=96, gdn_value_dim=192, max_position_embeddings=65536),
}


def get_spec(name_or_path: str) -> ModelSpec:
    """Preset name, or a directory holding a Hugging Face ``config.json``."""
    if name_or_path in PRESETS:
        return dataclasses.replace(PRESETS[name_or_path])
    p = Path(name_or_path)
    if (p / "config.json").exists():
        return ModelSpec.from_pretrained(name_or_path)
    raise ValueError(f"unknown model '{name_or_path}': not a preset {sorted(PRESETS)} nor a directory with config.json")


@dataclass
class ParamEntry:
    name: str
    offset: int
    shape: tuple[int, ...]
    decay: bool

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


class ParamLayout:
    """Offsets of every fused parameter inside the flat buffer.

    Order: embed, then per layer (wqkv, wo, w_gate_up, w_down), then lm_head (absent when tied),
    then the no-decay region: per layer (attn_norm, mlp_norm[, q_norm, k_norm, bqkv]), final_norm.
    Every entry starts on a 128-element boundary (256 bytes in bf16) so TMA bases stay aligned.
    """

    ALIGN = 128

    def __init__(self, spec: ModelSpec, with_lm_head: bool = True):
        self.spec = spec
        self.entries: dict[str, ParamEntry] = {}
        off = 0

        def add(name, shape, decay):
            nonlocal off
            e = ParamEntry(name, off, tuple(shape), decay)
            self.entries[name] = e
            off = (off + e.numel + self.ALIGN - 1) // self.ALIGN * self.ALIGN

        s = spec
        add("embed", (s.vocab_size, s.hidden_size), True)
        for i in range(s.num_layers):
            if s.is_gdn(i):
                add(f"l{i}.gdn_in", (s.gdn_in_rows, s.hidden_size), True)
                add(f"l{i}.gdn_out", (s.hidden_size, s.gdn_v_total), True)
            else:
                add(f"l{i}.wqkv", (s.qkv_dim, s.hidden_size), True)
                add(f"l{i}.wo", (s.hidden_size, s.q_dim), True)
            if s.num_experts:  # experts stacked along the rows: expert e owns rows [e * 2F, (e + 1) * 2F) / [e * D, (e + 1) * D)
                add(f"l{i}.router", (s.num_experts, s.hidden_size), True)
                add(f"l{i}.w_gate_up", (s.num_experts * 2 * s.intermediate_size, s.hidden_size), True)
                add(f"l{i}.w_down", (s.num_experts * s.hidden_size, s.intermediate_size), True)
            else:
                add(f"l{i}.w_gate_up", (2 * s.intermediate_size, s.hidden_size), True)
                add(f"l{i}.w_down", (s.hidden_size, s.intermediate_size), True)
        if with_lm_head and not s.tie_word_embeddings:
            add("lm_head", (s.vocab_size, s.hidden_size), True)
        self.decay_end = off
        for i in range(s.num_layers):
            add(f"l{i}.attn_norm", (s.hidden_size,), False)
            add(f"l{i}.mlp_norm", (s.hidden_size,), False)
            if s.is_gdn(i):
                add(f"l{i}.gdn_conv", (2 * s.gdn_k_total + s.gdn_v_total, s.gdn_conv), False)  # depthwise taps of q | k | v
                add(f"l{i}.gdn_o_norm", (s.gdn_value_dim,), False)
                add(f"l{i}.gdn_A_log", (s.gdn_value_heads,), False)
                add(f"l{i}.gdn_dt_bias", (s.gdn_value_heads,), False)
                continue
            if s.qk_norm:
                add(f"l{i}.q_norm", (s.q_dim if s.qk_norm_full else s.head_dim,), False)
                add(f"l{i}.k_norm", (s.kv_dim if s.qk_norm_full else s.head_dim,), False)
            if s.attention_bias:
                add(f"l{i}.bqkv", (s.qkv_dim,), False)
        add("final_norm", (s.hidden_size,), False)
        self.total = off

    def view(self, flat, name: str):
        e = self.entries[name]
        return flat[e.offset : e.offset + e.numel].view(e.shape)

    def views(self, flat) -> dict:
        return {n: self.view(flat, n) for n in self.entries}

    def hf_names_per_expert(self, name: str) -> list[tuple[str, int, int]] | None:
        """The per-expert spelling of a stacked expert entry (``mlp.experts.<e>.gate_proj.weight`` ...: what checkpoints
        written before transformers 5 carry), or None for every other entry."""
        s = self.spec
        if not s.num_experts or "." not in name:
            return None
        layer, leaf = name.split(".", 1)
        p = f"model.layers.{int(layer[1:])}.mlp.experts."
        F, D = s.intermediate_size, s.hidden_size
        if leaf == "w_gate_up":
            return [x for e in range(s.num_experts) for x in ((f"{p}{e}.gate_proj.weight", e * 2 * F, e * 2 * F + F),
                                                              (f"{p}{e}.up_proj.weight", e * 2 * F + F, (e + 1) * 2 * F))]
        if leaf == "w_down":
            return [(f"{p}{e}.down_proj.weight", e * D, (e + 1) * D) for e in range(s.num_experts)]
        return None

    # ---- Hugging Face tensor names <-> fused entries
    def hf_names(self, name: str) -> list[tuple[str, int, int]]:
        """For a fused entry: list of (hf_name, row_start, row_end) slices that make it up."""
        s = self.spec
        if name == "embed":
            return [("model.embed_tokens.weight", 0, s.vocab_size)]
        if name == "lm_head":
            return [("lm_head.weight", 0, s.vocab_size)]
        if name == "final_norm":
            return [("model.norm.weight", 0, s.hidden_size)]
        layer, leaf = name.split(".", 1)
        li = int(layer[1:])
        p = f"model.layers.{li}."
        if leaf.startswith("gdn_"):
            g, K, V, H = p + "linear_attn.", s.gdn_k_total, s.gdn_v_total, s.gdn_value_heads
            if leaf == "gdn_in":
                cuts = [("q_proj", K), ("k_proj", K), ("v_proj", V), ("g_proj", V), ("a_proj", H), ("b_proj", H)]
            elif leaf == "gdn_conv":   # stored [channels, 1, taps] in checkpoints
                cuts = [("q_conv1d", K), ("k_conv1d", K), ("v_conv1d", V)]
            else:
                return [{"gdn_out": (g + "o_proj.weight", 0, s.hidden_size), "gdn_o_norm": (g + "o_norm.weight", 0, s.gdn_value_dim),
                         "gdn_A_log": (g + "A_log", 0, H), "gdn_dt_bias": (g + "dt_bias", 0, H)}[leaf]]
            out, r = [], 0
            for nm, rows in cuts:
                out.append((g + nm + ".weight", r, r + rows))
                r += rows
            return out
        post = s.post_norm and not s.is_gdn(li)   # the gdn layers of a hybrid are pre-norm blocks
        if leaf == "wqkv" or leaf == "bqkv":
            suf = "weight" if leaf == "wqkv" else "bias"
            return [(p + f"self_attn.q_proj.{suf}", 0, s.q_dim), (p + f"self_attn.k_proj.{suf}", s.q_dim, s.q_dim + s.kv_dim),
                    (p + f"self_attn.v_proj.{suf}", s.q_dim + s.kv_dim, s.qkv_dim)]
        if leaf == "wo":
            return [(p + "self_attn.o_proj.weight", 0, s.hidden_size)]
        if s.num_experts and leaf == "router":
            return [(p + "mlp.gate.weight", 0, s.num_experts)]
        if s.num_experts and leaf == "w_gate_up":   # one stacked tensor [E, 2F, D]: the 2-D entry is its reshape
            return [(p + "mlp.experts.gate_up_proj", 0, s.num_experts * 2 * s.intermediate_size)]
        if s.num_experts and leaf == "w_down":      # [E, D, F]
            return [(p + "mlp.experts.down_proj", 0, s.num_experts * s.hidden_size)]
        if leaf == "w_gate_up":
            return [(p + "mlp.gate_proj.weight", 0, s.intermediate_size),
                    (p + "mlp.up_proj.weight", s.intermediate_size, 2 * s.intermediate_size)]
        if leaf == "w_down":
            return [(p + "mlp.down_proj.weight", 0, s.hidden_size)]
        if leaf == "attn_norm":  # post-norm blocks: the norm applied to the attention output
            return [(p + ("post_attention_layernorm.weight" if post else "input_layernorm.weight"), 0, s.hidden_size)]
        if leaf == "mlp_norm":   # post-norm blocks: the norm applied to the MLP output
            return [(p + ("post_feedforward_layernorm.weight" if post else "post_attention_layernorm.weight"), 0, s.hidden_size)]
        if leaf == "q_norm":
            return [(p + "self_attn.q_norm.weight", 0, s.q_dim if s.qk_norm_full else s.head_dim)]
        if leaf == "k_norm":
            return [(p + "self_attn.k_norm.weight", 0, s.kv_dim if s.qk_norm_full else s.head_dim)]
        raise KeyError(name)
