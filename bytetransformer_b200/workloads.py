"""Seeded synthetic workloads with the shapes of the benchmark configurations,
and the algorithmic flop / byte model used for roofline figures.

There is no public dataset behind the reference's benchmark (it draws random
tensors, benchmark/bert_bench.sh:21-56); these generators stand in for it.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch


@dataclass
class ModelShape:
    name: str
    layers: int
    head_num: int
    head_size: int = 64

    @property
    def hidden(self):
        return self.head_num * self.head_size

    @property
    def ffn(self):
        return 4 * self.hidden


BERT_BASE = ModelShape("bert-base", 12, 12)
BERT_LARGE = ModelShape("bert-large", 24, 16)


def lengths_for(config: str, seed: int = 1234) -> np.ndarray:
    """Per-sequence valid lengths of a named configuration.

    single_layer_b16_s64   16 sequences, uniform in [1,64]
    b1_sweep_s<S>          1 sequence of round(0.6*S)
    b16_s512               16 sequences, uniform in [1,512]
    large_b64_s384         64 sequences, normal(230,80) rounded, clipped to [8,384]
    whole_box_1024x1024    1024 sequences, uniform in [16,1024]
    """
    g = torch.Generator().manual_seed(seed)
    if config == "single_layer_b16_s64":
        return torch.randint(1, 65, (16,), generator=g).numpy()
    if config.startswith("b1_sweep_s"):
        S = int(config[len("b1_sweep_s"):])
        return np.array([int(round(0.6 * S))])
    if config == "b16_s512":
        return torch.randint(1, 513, (16,), generator=g).numpy()
    if config == "large_b64_s384":
        return torch.clamp(torch.round(torch.randn(64, generator=g) * 80 + 230), 8, 384).long().numpy()
    if config == "whole_box_1024x1024":
        return torch.randint(16, 1025, (1024,), generator=g).numpy()
    raise ValueError(config)


def make_weights(shape: ModelShape, seed: int = 7, device="cpu", std: float = 0.02):
    """Random-init weights of the architecture: GEMM weights ~ N(0, std) stored
    [in,out], biases and beta 0, gamma 1, fp16."""
    g = torch.Generator().manual_seed(seed)
    H, F = shape.hidden, shape.ffn
    layers = []
    for _ in range(shape.layers):
        w = [
            torch.randn(H, 3 * H, generator=g) * std, torch.zeros(3 * H),
            torch.randn(H, H, generator=g) * std, torch.zeros(H), torch.ones(H), torch.zeros(H),
            torch.randn(H, F, generator=g) * std, torch.zeros(F),
            torch.randn(F, H, generator=g) * std, torch.zeros(H), torch.ones(H), torch.zeros(H),
        ]
        layers.append([t.half().to(device).contiguous() for t in w])
    return layers


def gemm_flops_per_layer(tokens: int, hidden: int) -> float:
    """2*T*(3H^2 + H^2 + 2*H*4H) = 24*T*H^2."""
    return 24.0 * tokens * hidden * hidden


def attention_flops_per_layer(lengths, hidden: int) -> float:
    """QK^T + PV over valid x valid positions, all heads: 4*H*sum(L^2)."""
    l = np.asarray(lengths, dtype=np.float64)
    return 4.0 * hidden * float((l * l).sum())


def total_flops(lengths, shape: ModelShape) -> float:
    T = int(np.asarray(lengths).sum())
    return shape.layers * (gemm_flops_per_layer(T, shape.hidden) + attention_flops_per_layer(lengths, shape.hidden))
