"""Analytic FLOP and byte counts of a decoder, for MFU / MBU reporting.

Same role and method names as ``ModelDims`` in the reference (``open_instruct/utils.py:1833-2513``) with the
same conventions: 2 FLOPs per multiply-accumulate, ~4 FLOPs per attention score for softmax,
training = 3x forward, GQA handled through the kv-head count, optional sliding window.  Device
peaks come from ``GPU_SPECS`` (the B200 row is the nominal 2.25 PFLOP/s dense bf16 / 8 TB/s the
reference uses as denominator, ``utils.py:1807``).
"""

from __future__ import annotations

import dataclasses

FLOP_PER_MAC = 2
SOFTMAX_FLOPS_PER_SCORE = 4
GDN_RECURRENCE_PASSES = 4   # state-sized multiply-add passes of the gated delta rule per token: read-out, error, decayed state, update

GPU_SPECS = {
    "a100": {"flops": 312e12, "memory_size": 80e9, "memory_bandwidth": 2.0e12},
    "b200": {"flops": 2250e12, "memory_size": 192e9, "memory_bandwidth": 8e12},
    "b300": {"flops": 2250e12, "memory_size": 288e9, "memory_bandwidth": 8e12},
    "h100": {"flops": 990e12, "memory_size": 80e9, "memory_bandwidth": 3.35e12},
    "h200": {"flops": 989e12, "memory_size": 141e9, "memory_bandwidth": 4.8e12},
    "a6000": {"flops": 155e12, "memory_size": 48e9, "memory_bandwidth": 768e9},
    "l40s": {"flops": 362e12, "memory_size": 48e9, "memory_bandwidth": 864e9},
    "gb10": {"flops": 104e12, "memory_size": 128e9, "memory_bandwidth": 273e9},
}


def get_device_name(device_name: str | None = None) -> str:
    """Key of ``GPU_SPECS`` matching a device name string (defaults to the current CUDA device)."""
    if device_name is None:
        import torch

        device_name = torch.cuda.get_device_name(0) if torch.cuda.is_available() else "b200"
    low = device_name.lower()
    for key in sorted(GPU_SPECS, key=len, reverse=True):
        if key in low:
            return key
    raise ValueError(f"unknown device {device_name!r}; known: {sorted(GPU_SPECS)}")


def _keys_seen(prompt: int, response: int, window: int | None) -> int:
    """Sum over the response tokens k = 1..R of the keys token k attends to: ``prompt + k``, capped at ``window``."""
    if not window:
        return response * prompt + response * (response + 1) // 2
    m = max(0, min(response, window - prompt - 1))   # tokens whose context is still shorter than the window
    return m * prompt + m * (m + 1) // 2 + (response - m) * window


@dataclasses.dataclass
class ModelDims:
    num_layers: int
    hidden_size: int
    intermediate_size: int
    vocab_size: int
    num_attn_heads: int
    head_dim: int
    num_kv_heads: int | None = None
    num_params: int | None = None
    device_name: str | None = None
    sliding_window: int | None = None
    num_sliding_window_layers: int = 0
    # hybrid models: layers whose sequence mixer is a gated DeltaNet (cost linear in the tokens, a fixed-size state per head)
    num_linear_attn_layers: int = 0
    linear_attn_num_k_heads: int = 0
    linear_attn_num_v_heads: int = 0
    linear_attn_key_head_dim: int = 0
    linear_attn_value_head_dim: int = 0
    linear_attn_conv_size: int = 4

    def __post_init__(self):
        if self.num_kv_heads is None:
            self.num_kv_heads = self.num_attn_heads
        if self.num_attn_heads % self.num_kv_heads:
            raise ValueError("num_attn_heads must be divisible by num_kv_heads")
        if self.num_sliding_window_layers + self.num_linear_attn_layers > self.num_layers:
            raise ValueError("more sliding-window and linear-attention layers than layers")
        if self.num_params is None:
            self.num_params = self._calculate_num_params()

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_spec(cls, spec, device_name: str | None = None) -> "ModelDims":
        return cls(num_layers=spec.num_layers, hidden_size=spec.hidden_size, intermediate_size=spec.intermediate_size,
                   vocab_size=spec.vocab_size, num_attn_heads=spec.num_heads, head_dim=spec.head_dim,
                   num_kv_heads=spec.num_kv_heads, device_name=device_name, sliding_window=spec.sliding_window,
                   num_sliding_window_layers=sum(1 for i in range(spec.num_layers) if spec.window(i)),
                   num_linear_attn_layers=sum(1 for i in range(spec.num_layers) if spec.is_gdn(i)),
                   linear_attn_num_k_heads=spec.gdn_key_heads, linear_attn_num_v_heads=spec.gdn_value_heads,
                   linear_attn_key_head_dim=spec.gdn_key_dim, linear_attn_value_head_dim=spec.gdn_value_dim,
                   linear_attn_conv_size=spec.gdn_conv)

    @classmethod
    def from_hf_config(cls, model_name_or_path: str) -> "ModelDims":
        from ..models import get_spec

        return cls.from_spec(get_spec(model_name_or_path))

    def _calculate_num_params(self) -> int:
        q = self.num_attn_heads * self.head_dim
        kv = self.num_kv_heads * self.head_dim
        attn = self.hidden_size * (q + 2 * kv) + q * self.hidden_size
        mlp = 3 * self.hidden_size * self.intermediate_size
        norms = 2 * self.hidden_size
        n_attn = self.num_layers - self.num_linear_attn_layers
        return (n_attn * attn + self.num_linear_attn_layers * self._gdn_layer_params() + self.num_layers * (mlp + norms)
                + 2 * self.vocab_size * self.hidden_size + self.hidden_size)

    @property
    def linear_attn_key_dim(self) -> int:
        return self.linear_attn_num_k_heads * self.linear_attn_key_head_dim

    @property
    def linear_attn_value_dim(self) -> int:
        return self.linear_attn_num_v_heads * self.linear_attn_value_head_dim

    def _gdn_layer_params(self) -> int:
        """Parameters of one gated-DeltaNet mixer (q, k, v, gate, output projections; decay and beta projections; the taps)."""
        h, kd, vd = self.hidden_size, self.linear_attn_key_dim, self.linear_attn_value_dim
        return 2 * h * kd + 3 * h * vd + 2 * h * self.linear_attn_num_v_heads + (2 * kd + vd) * self.linear_attn_conv_size

    @property
    def device_flops(self) -> float:
        return GPU_SPECS[get_device_name(self.device_name)]["flops"]

    @property
    def device_memory_bandwidth(self) -> float:
        return GPU_SPECS[get_device_name(self.device_name)]["memory_bandwidth"]

    # ------------------------------------------------------------------ FLOPs (forward)
    def attn_flops(self, query_len: int, kv_len: int, sliding_window: int | None = None) -> int:
        """One layer: projections for ``query_len`` new tokens + scores/values against ``kv_len`` keys."""
        d, h, hd = self.hidden_size, self.num_attn_heads, self.head_dim
        q_dim, kv_dim = h * hd, self.num_kv_heads * hd
        kv_eff = min(kv_len, sliding_window) if sliding_window else kv_len
        proj = FLOP_PER_MAC * query_len * d * (q_dim + 2 * kv_dim) + FLOP_PER_MAC * query_len * q_dim * d
        scores = FLOP_PER_MAC * query_len * kv_eff * hd * h
        softmax = SOFTMAX_FLOPS_PER_SCORE * query_len * kv_eff * h
        values = FLOP_PER_MAC * query_len * kv_eff * hd * h
        return proj + scores + softmax + values

    def linear_attn_flops(self, seq_len: int) -> int:
        """One gated-DeltaNet layer over ``seq_len`` tokens (``open_instruct/utils.py:2014-2042``): projections, convolution and
        ``GDN_RECURRENCE_PASSES`` passes over the [key_dim, value_dim] state of every head per token (read-out, error, decay,
        update).  Independent of the context length, so prefill and decode cost the same per token."""
        m, d, kd, vd, hv = FLOP_PER_MAC, self.hidden_size, self.linear_attn_key_dim, self.linear_attn_value_dim, self.linear_attn_num_v_heads
        proj = m * seq_len * d * (2 * kd + 2 * vd + 2 * hv) + m * seq_len * vd * d
        conv = m * seq_len * self.linear_attn_conv_size * (2 * kd + vd)
        rec = m * GDN_RECURRENCE_PASSES * seq_len * hv * self.linear_attn_key_head_dim * self.linear_attn_value_head_dim
        return proj + conv + rec

    def gdn_state_bytes(self, num_tokens: int, dtype_bytes: int = 2) -> int:
        """Bytes moved for the recurrent state: every decoded token reads and writes each layer's whole state once."""
        return self.num_linear_attn_layers * num_tokens * 2 * self.linear_attn_num_v_heads * self.linear_attn_key_head_dim * self.linear_attn_value_head_dim * dtype_bytes

    def mlp_flops(self, seq_len: int) -> int:
        return 3 * FLOP_PER_MAC * seq_len * self.hidden_size * self.intermediate_size

    def _layer_stack(self, query_len: int, kv_len: int) -> int:
        full = self.num_layers - self.num_sliding_window_layers - self.num_linear_attn_layers
        return (full * self.attn_flops(query_len, kv_len) + self.num_sliding_window_layers * self.attn_flops(query_len, kv_len, self.sliding_window)
                + self.num_linear_attn_layers * self.linear_attn_flops(query_len) + self.num_layers * self.mlp_flops(query_len))

    def prefill_flops(self, prompt_lengths: list[int]) -> int:
        """Causal prefill: token t attends to t+1 keys -> average kv length (L+1)/2."""
        total = 0
        for L in prompt_lengths:
            total += self._layer_stack_causal(L) + FLOP_PER_MAC * L * self.hidden_size * self.vocab_size
        return total

    def _layer_stack_causal(self, L: int) -> int:
        # projections + MLP are linear in L; score/value terms see an average of (L+1)/2 keys
        base = self._layer_stack(L, 0)
        d_scores = self._layer_stack(L, L + 1) - base
        return base + d_scores // 2

    def decode_flops(self, prompt_lengths: list[int], response_lengths: list[int], samples_per_prompt: int = 1) -> int:
        if len(response_lengths) != len(prompt_lengths) * samples_per_prompt:
            raise ValueError("response_lengths must have len(prompt_lengths) * samples_per_prompt entries")
        total = 0
        lin = self._layer_stack(1, 0)   # projections, MLP, linear-attention layers: per token, whatever the context
        full = self.num_layers - self.num_sliding_window_layers - self.num_linear_attn_layers
        per_key = self.attn_flops(1, 1) - self.attn_flops(1, 0)   # one layer, one more key
        for i, P in enumerate(prompt_lengths):
            for R in response_lengths[i * samples_per_prompt:(i + 1) * samples_per_prompt]:
                # token k of the response attends to P + k keys (at most the window in a sliding-window layer)
                keys = full * _keys_seen(P, R, None) + self.num_sliding_window_layers * _keys_seen(P, R, self.sliding_window)
                total += R * lin + per_key * keys
                total += FLOP_PER_MAC * R * self.hidden_size * self.vocab_size
        return total

    def flops(self, prompt_lengths: list[int], response_lengths: list[int] | None = None, samples_per_prompt: int = 1,
              is_training: bool = False) -> int:
        total = self.prefill_flops(prompt_lengths)
        if response_lengths is not None:
            total += self.decode_flops(prompt_lengths, response_lengths, samples_per_prompt)
        return 3 * total if is_training else total

    # ------------------------------------------------------------------ bytes
    def weight_memory_bytes(self, num_tokens: int, dtype_bytes: int = 2) -> int:
        """Weights streamed once per forward pass of ``num_tokens`` decode steps (batch-1 view)."""
        q = self.num_attn_heads * self.head_dim
        kv = self.num_kv_heads * self.head_dim
        attn = self.hidden_size * (q + 2 * kv) + q * self.hidden_size
        mlp = 3 * self.hidden_size * self.intermediate_size
        layers = (self.num_layers - self.num_linear_attn_layers) * attn + self.num_linear_attn_layers * self._gdn_layer_params() + self.num_layers * mlp
        return num_tokens * dtype_bytes * (layers + self.vocab_size * self.hidden_size)

    def kv_cache_write_bytes(self, num_tokens: int, dtype_bytes: int = 2) -> int:
        return num_tokens * (self.num_layers - self.num_linear_attn_layers) * 2 * self.num_kv_heads * self.head_dim * dtype_bytes

    def kv_cache_read_bytes(self, prompt_lengths: list[int], response_lengths: list[int], samples_per_prompt: int = 1,
                            dtype_bytes: int = 2) -> int:
        per_tok = (self.num_layers - self.num_linear_attn_layers) * 2 * self.num_kv_heads * self.head_dim * dtype_bytes
        total = 0
        for i, P in enumerate(prompt_lengths):
            for R in response_lengths[i * samples_per_prompt:(i + 1) * samples_per_prompt]:
                total += per_tok * (R * P + R * (R - 1) // 2)
        return total

    def prefill_memory_bytes(self, prompt_lengths: list[int], dtype_bytes: int = 2) -> int:
        return self.weight_memory_bytes(1, dtype_bytes) * max(1, len(prompt_lengths)) ** 0 + self.kv_cache_write_bytes(sum(prompt_lengths), dtype_bytes)

    def decode_memory_bytes(self, prompt_lengths: list[int], response_lengths: list[int], samples_per_prompt: int = 1,
                            dtype_bytes: int = 2) -> int:
        steps = max(response_lengths) if response_lengths else 0  # one weight pass per batched decode step
        return (self.weight_memory_bytes(steps, dtype_bytes) + self.kv_cache_write_bytes(sum(response_lengths), dtype_bytes)
                + self.kv_cache_read_bytes(prompt_lengths, response_lengths, samples_per_prompt, dtype_bytes)
                + self.gdn_state_bytes(sum(response_lengths), dtype_bytes))

    def memory_bytes(self, prompt_lengths: list[int], response_lengths: list[int] | None = None, samples_per_prompt: int = 1,
                     dtype_bytes: int = 2) -> int:
        total = self.prefill_memory_bytes(prompt_lengths, dtype_bytes)
        if response_lengths is not None:
            total += self.decode_memory_bytes(prompt_lengths, response_lengths, samples_per_prompt, dtype_bytes)
        return total

    # ------------------------------------------------------------------ utilisation
    def calculate_mfu(self, sequence_lengths: list[int], seconds: float, num_gpus: int = 1, is_training: bool = False) -> float:
        fl = self.flops(sequence_lengths, is_training=is_training)
        return 100.0 * fl / max(seconds, 1e-12) / (self.device_flops * num_gpus)

    def calculate_mbu(self, prompt_lengths: list[int], seconds: float, response_lengths: list[int] | None = None,
                      samples_per_prompt: int = 1, num_gpus: int = 1) -> float:
        by = self.memory_bytes(prompt_lengths, response_lengths, samples_per_prompt)
        return 100.0 * by / max(seconds, 1e-12) / (self.device_memory_bandwidth * num_gpus)

    def calculate_actor_utilization(self, prompt_lengths, response_lengths, total_generation_time: float, samples_per_prompt: int,
                                    num_engines: int, num_gpus_per_engine: int) -> dict:
        gpus = num_engines * num_gpus_per_engine
        fl = self.flops(prompt_lengths, response_lengths, samples_per_prompt)
        by = self.memory_bytes(prompt_lengths, response_lengths, samples_per_prompt)
        mfu = 100.0 * fl / total_generation_time / (self.device_flops * gpus)
        mbu = 100.0 * by / total_generation_time / (self.device_memory_bandwidth * gpus)
        return {"mfu": mfu, "mbu": mbu}

    def calculate_learner_utilization(self, prompt_lengths, response_lengths, training_time: float, samples_per_prompt: int,
                                      num_training_gpus: int) -> dict:
        seqs = [p + r for i, p in enumerate(prompt_lengths) for r in response_lengths[i * samples_per_prompt:(i + 1) * samples_per_prompt]]
        return {"mfu": self.calculate_mfu(seqs, training_time, num_training_gpus, is_training=True)}

    def approximate_learner_utilization(self, total_tokens: float, avg_sequence_length: float, training_time: float,
                                        num_training_gpus: int, device_name: str | None = None) -> float:
        """MFU (%) from a token count and a (length-weighted) mean sequence length."""
        if total_tokens <= 0 or training_time <= 0:
            return 0.0
        L = max(1, int(round(avg_sequence_length)))
        n = total_tokens / L
        fl = 3 * self.flops([L]) * n
        return 100.0 * fl / training_time / (self.device_flops * num_training_gpus)
