"""Throughput accounting: model FLOPs per token, MFU and a JSONL sink.

``flops_per_token`` is ``6·N_active + 3.5·(2·S·d_model)·L`` where ``N_active``
counts attention, the top-k experts, the router and the LM head (the embedding
is excluded) and the 3.5 factor is causal attention forward 1 + backward 2.5.
For the 32-block, d_model 4096, d_ff 14336, 32/8-head, top-2, vocab 32000,
context 8192 model this gives 84.01 GFLOPs per token, the figure the
reference's results table uses (README.md:19).
"""
from __future__ import annotations

import json
import time

__all__ = ["active_params", "flops_per_token", "mfu", "MetricsSink", "PEAK_BF16_DENSE"]

PEAK_BF16_DENSE = 2.25e15


def active_params(d_model: int, d_ff: int, num_heads: int, num_experts: int, vocab: int,
                  layers: int, top_k: int = 2, kv_ratio: int = 4) -> int:
    kv_dim = d_model // kv_ratio
    attention = 2 * d_model * d_model + 2 * d_model * kv_dim
    experts = top_k * 3 * d_model * d_ff
    router = d_model * num_experts
    return layers * (attention + experts + router) + vocab * d_model


def flops_per_token(d_model: int, d_ff: int, num_heads: int, num_experts: int, vocab: int,
                    layers: int, seq: int, top_k: int = 2) -> float:
    dense = 6.0 * active_params(d_model, d_ff, num_heads, num_experts, vocab, layers, top_k)
    attention = 3.5 * (2.0 * seq * d_model) * layers
    return dense + attention


def mfu(tokens_per_s: float, flops_token: float, n_gpus: int, peak: float = PEAK_BF16_DENSE) -> float:
    return tokens_per_s * flops_token / (n_gpus * peak)


class MetricsSink:
    """Append one JSON object per record to a file (or keep them in memory)."""

    def __init__(self, path=None):
        self.path = path
        self.records: list[dict] = []

    def write(self, **record) -> dict:
        record.setdefault("ts", time.time())
        self.records.append(record)
        if self.path:
            with open(self.path, "a", encoding="utf-8") as handle:
                handle.write(json.dumps(record) + "\n")
        return record
