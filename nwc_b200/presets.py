"""Decoder architectures the decode loop knows by name (plain data: importable without the CUDA library).

The shapes are the ones the benchmark configurations name: Qwen3-0.6B / 4B (per-head q/k RMSNorm) and a Llama-3-70B
style decoder; `tiny` is the 2-layer model of the tests (reference: tests/test_checkpoint.py:12-20 builds one like it).
"""
from dataclasses import dataclass


@dataclass
class DecoderConfig:
    name: str
    layers: int
    hidden: int
    intermediate: int
    n_q: int
    n_kv: int
    head_dim: int
    vocab: int
    tied: bool
    qk_norm: bool
    rope_theta: float = 1e6
    eps: float = 1e-6

    @property
    def qkv_rows(self): return (self.n_q + 2 * self.n_kv) * self.head_dim

    def matrix_shapes(self):
        """(rows, cols) of the five kinds of compressed matrices a decode step multiplies with."""
        return {"qkv": (self.qkv_rows, self.hidden), "o": (self.hidden, self.n_q * self.head_dim), "gate_up": (2 * self.intermediate, self.hidden),
                "down": (self.hidden, self.intermediate), "lm_head": (self.vocab, self.hidden)}


PRESETS = {
    "qwen3-0.6b": DecoderConfig("qwen3-0.6b", 28, 1024, 3072, 16, 8, 128, 151936, True, True),
    "qwen3-4b": DecoderConfig("qwen3-4b", 36, 2560, 9728, 32, 8, 128, 151936, False, True),
    "llama3-70b": DecoderConfig("llama3-70b", 80, 8192, 28672, 64, 8, 128, 128256, False, False, rope_theta=5e5, eps=1e-5),
    "tiny": DecoderConfig("tiny", 2, 256, 1000, 4, 2, 64, 4096, True, True),
}
