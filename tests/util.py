"""Helpers shared by the parity tests: seeded workloads of the benchmark geometries, error metrics."""

from __future__ import annotations

import torch


def make_tables(gen: torch.Generator, heads: int, stages: int, groups: int, sub: int, scales=None) -> torch.Tensor:
    """fp16 deployed tables [H,S,G,256,d]; stage s drawn N(0, scales[s])."""
    scales = scales or [0.5 * 0.5**s for s in range(stages)]
    return torch.stack([torch.randn(heads, groups, 256, sub, generator=gen) * scales[s] for s in range(stages)], dim=1).half()


def make_states(gen: torch.Generator, shape, dtype=torch.float16, outlier_channels: int = 0) -> torch.Tensor:
    x = torch.randn(*shape, generator=gen)
    if outlier_channels:
        for h in range(shape[1]):
            x[:, h, :, torch.randperm(shape[-1], generator=gen)[:outlier_channels]] *= 8.0
    return x.to(dtype)


def rel_l2(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).norm() / want.norm().clamp_min(1e-30))


def max_rel(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
