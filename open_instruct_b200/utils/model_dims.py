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

    def __post_init__(self):
        if self.num_kv_heads is None:
            self.num_kv_heads = self.num_attn_heads
        if self.num_attn_heads % self.num_kv_heads:
            raise ValueError("num_attn_heads must be divisible by num_kv_heads")
        if self.num_sliding_window_layers > self.num_layers:
            raise ValueError("more sliding-window layers than layers")
        if self.num_params is None:
            self.num_params = self._calculate_num_params()

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_spec(cls, spec, device_name: str | None = None) -> "ModelDims":
        return cls(num_layers=spec.num_layers, hidden_size=spec.hidden_size, intermediate_size=spec.intermediate_size,
                   vocab_size=spec.vocab_size, num_attn_heads=spec.num_heads, head_dim=spec.head_dim,
                   num_kv_heads=spec.num_kv_heads, device_name=device_name)

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
        return self.num_layers * (attn + mlp + norms) + 2 * self.vocab_size * self.hidden_size + self.hidden_size

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

    def mlp_flops(self, seq_len: int) -> int:
        return 3 * FLOP_PER_MAC * seq_len * self.hidden_size * self.intermediate_size

    def _layer_stack(self, query_len: int, kv_len: int) -> int:
        full = self.num_layers - self.num_sliding_window_layers
        return (full * self.attn_flops(query_len, kv_len) + self.num_sliding_window_layers * self.attn_flops(query_len, kv_len, self.sliding_window)
                + self.num_layers * self.mlp_flops(query_len))

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
        for i, P in enumerate(prompt_lengths):
            for R in response_lengths[i * samples_per_prompt:(i + 1) * samples_per_prompt]:
                # token k of the response attends to P + k keys: sum over k of one-token layers
                lin = self._layer_stack(1, 0)
                per_key = self._layer_stack(1, 1) - lin
                total += R * lin + per_key * (R * P + R * (R + 1) // 2)
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
        per_layer = self.hidden_size * (q + 2 * kv) + q * self.hidden_size + 3 * self.hidden_size * self.intermediate_size
        return num_tokens * dtype_bytes * (self.num_layers * per_layer + self.vocab_size * self.hidden_size)

    def kv_cache_write_bytes(self, num_tokens: int, dtype_bytes: int = 2) -> int:
        return num_tokens * self.num_layers * 2 * self.num_kv_heads * self.head_dim * dtype_bytes

    def kv_cache_read_bytes(self, prompt_lengths: list[int], response_lengths: list[int], samples_per_prompt: int = 1,
                            dtype_bytes: int = 2) -> int:
        per_tok = self.num_layers * 2 * self.num_kv_heads * self.head_dim * dtype_bytes
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
                + self.kv_cache_read_bytes(prompt_lengths, response_lengths, samples_per_prompt, dtype_bytes))

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
