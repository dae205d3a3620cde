"""Shared helpers for the parity tests: seeded inputs, bf16 <-> numpy, error measures."""
from __future__ import annotations

import numpy as np
import torch

import oracle as O


def to_bits(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> uint16 numpy (the oracle's weight form)."""
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def from_bits(bits: np.ndarray, device="cuda") -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16).to(device)


def widen(t: torch.Tensor) -> np.ndarray:
    """bf16 or f32 tensor -> float32 numpy, exactly."""
    return t.detach().float().cpu().numpy()


def normal_bf16(rng: np.random.Generator, shape, std=1.0) -> np.ndarray:
    """bf16 bits of N(0, std) samples."""
    return O.bf16_bits((rng.standard_normal(shape, dtype=np.float32) * np.float32(std)))


def rel_error(got: np.ndarray, want: np.ndarray) -> float:
    """max |got - want| over max |want|: the per-op relative error the parity bar is stated in."""
    scale = float(np.max(np.abs(want))) or 1.0
    return float(np.max(np.abs(got.astype(np.float64) - want.astype(np.float64)))) / scale


def u32(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy().view(np.uint32)


def dev_u32(a, device="cuda") -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.uint32).view(np.int32)).to(device)
