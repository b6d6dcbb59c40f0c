"""Rotary position encoding: tables of cos and sin, float32.

inv_freq[i] = theta^(-i / (R/2)), angle = position * inv_freq[i]
(rollout/monkey_patch/qwen3.py:121-127; rollout/utils/test_decode.py:14-17).  The reference
rounds its tables to bfloat16; these stay float32 in both precisions, because the rotation
angles belong to the arithmetic that is kept in 32-bit.  The rotation itself is fused into the
kernel that writes the cache (csrc/rope_cache.cu).
"""
from __future__ import annotations

import math

import torch

from .base import POSITION_ENCODINGS, PositionEncoding

# every layer of a model asks for the same tables: one copy per (rotary width, theta, positions, device)
_TABLES = {}


@POSITION_ENCODINGS.register("rope")
class RotaryEncoding(PositionEncoding):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim={spec.rotary_dim} must be even")
        self._tables = None

    def rotary_tables(self):
        """(cos, sin, rotary_dim); cos and sin are float32 [max_positions, rotary_dim/2] on the device."""
        if self._tables is None:
            s = self.spec
            key = (s.rotary_dim, float(s.theta), s.max_positions, str(self.env.device))
            shared = _TABLES.get(key)
            if shared is None:
                half = s.rotary_dim // 2
                # made on the CPU in float32 so that every device sees the same angles
                inv_freq = 1.0 / (s.theta ** (torch.arange(0, half, dtype=torch.float32) / half))
                ang = torch.outer(torch.arange(s.max_positions, dtype=torch.float32), inv_freq)
                shared = _TABLES[key] = (ang.cos().contiguous().to(self.env.device),
                                         ang.sin().contiguous().to(self.env.device), s.rotary_dim)
            self._tables = shared
        return self._tables

    tables = rotary_tables


@POSITION_ENCODINGS.register("rope_scaled")
class ScaledRotaryEncoding(PositionEncoding):
    """Rotary tables with optional slowing of the long wavelengths (``ScaledRopeSpec``).  Frequencies and angles are
    worked out in float64 on the host and rounded once, to the float32 tables the kernels read."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim={spec.rotary_dim} must be even")
        self._tables = None

    @staticmethod
    def frequencies(rotary_dim: int, theta: float, scaling=None) -> torch.Tensor:
        half = rotary_dim // 2
        f = float(theta) ** (-torch.arange(0, half, dtype=torch.float64) / half)
        if scaling is not None:
            factor, low, high, original = (float(v) for v in scaling)
            wavelength = 2.0 * math.pi / f
            blend = ((original / wavelength - low) / (high - low)).clamp(0.0, 1.0)
            mixed = (1.0 - blend) * f / factor + blend * f
            f = torch.where(wavelength < original / high, f, torch.where(wavelength > original / low, f / factor, mixed))
        return f

    def rotary_tables(self):
        """(cos, sin, rotary_dim) for the kernel that rotates while it writes the cache, which takes widths that are
        multiples of 4; None for any other even width: the attention then calls ``apply``."""
        return self.tables() if self.spec.rotary_dim % 4 == 0 else None

    def apply(self, qkv, batch, num_heads, num_kv_heads, head_dim):
        from ..ext import ops
        cos, sin, rot = self.tables()
        ops.rotary_inplace(qkv, cos, sin, rot, batch.pos, num_heads + num_kv_heads, head_dim)

    def tables(self):
        if self._tables is None:
            s = self.spec
            key = ("scaled", s.rotary_dim, float(s.theta), s.scaling, s.max_positions, str(self.env.device))
            shared = _TABLES.get(key)
            if shared is None:
                f = self.frequencies(s.rotary_dim, s.theta, s.scaling)
                ang = torch.outer(torch.arange(s.max_positions, dtype=torch.float64), f)
                shared = _TABLES[key] = (ang.cos().float().contiguous().to(self.env.device),
                                         ang.sin().float().contiguous().to(self.env.device), s.rotary_dim)
            self._tables = shared
        return self._tables


@POSITION_ENCODINGS.register("rope_ramped")
class RampedRotaryEncoding(PositionEncoding):
    """Rotary tables whose frequencies are stretched along a ramp over the pair index, with one factor on cos and sin
    (``RampedRopeSpec``).  Frequencies and angles are worked out in float64 on the host and rounded once, to the
    float32 tables the kernels read."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.rotary_dim % 2 or spec.rotary_dim <= 0:
            raise ValueError(f"rotary_dim={spec.rotary_dim} must be even and positive")
        self._tables = None

    @staticmethod
    def frequencies(spec):
        """(float64 frequencies [rotary_dim / 2], factor on cos and sin)."""
        dims, theta = spec.rotary_dim, float(spec.theta)
        i = torch.arange(dims // 2, dtype=torch.float64)
        f = theta ** (-2.0 * i / dims)
        if spec.factor is None:
            return f, 1.0
        factor = float(spec.factor)

        def index(turns: float) -> float:
            return dims * math.log(float(spec.original) / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

        lo = max(math.floor(index(float(spec.fast))), 0)
        hi = min(math.ceil(index(float(spec.slow))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        return f / factor * ramp + f * (1.0 - ramp), float(spec.magnitude_slope) * math.log(factor) + 1.0

    def rotary_tables(self):
        """(cos, sin, rotary_dim) for the kernel that rotates while it writes the cache, which takes widths that are
        multiples of 4; None for any other even width: the attention then calls ``apply``."""
        return self.tables() if self.spec.rotary_dim % 4 == 0 else None

    def apply(self, qkv, batch, num_heads, num_kv_heads, head_dim):
        from ..ext import ops
        cos, sin, rot = self.tables()
        ops.rotary_inplace(qkv, cos, sin, rot, batch.pos, num_heads + num_kv_heads, head_dim)

    def tables(self):
        """(cos, sin, rotary_dim); cos and sin are float32 [max_positions, rotary_dim/2] on the device, the factor
        already in them."""
        if self._tables is None:
            s = self.spec
            key = ("ramped", s, str(self.env.device))
            shared = _TABLES.get(key)
            if shared is None:
                f, mag = self.frequencies(s)
                ang = torch.outer(torch.arange(s.max_positions, dtype=torch.float64), f)
                shared = _TABLES[key] = ((ang.cos() * mag).float().contiguous().to(self.env.device),
                                         (ang.sin() * mag).float().contiguous().to(self.env.device), s.rotary_dim)
            self._tables = shared
        return self._tables


def drop_shared_tables() -> None:
    """Forgets the shared tables (models that still hold them keep them alive)."""
    _TABLES.clear()


@POSITION_ENCODINGS.register("rope_interleaved")
class InterleavedRotaryEncoding(PositionEncoding):
    """Tables for a rotation of neighbouring pairs (``InterleavedRopeSpec``): column i of cos and sin belongs to the
    elements 2i and 2i + 1 of a head.  Frequencies and angles are worked out in float64 on the host and rounded once.
    The rotation itself happens in the kernel that prepares an attention's rows (csrc/attention_prep.cu)."""

    interleaved = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.rotary_dim % 2 or spec.rotary_dim <= 0:
            raise ValueError(f"rotary_dim={spec.rotary_dim} must be even and positive")
        self._tables = None

    def tables(self):
        """(cos, sin, rotary_dim); cos and sin are float32 [max_positions, rotary_dim / 2] on the device."""
        if self._tables is None:
            s = self.spec
            key = ("interleaved", s.rotary_dim, float(s.theta), s.max_positions, str(self.env.device))
            shared = _TABLES.get(key)
            if shared is None:
                half = s.rotary_dim // 2
                f = float(s.theta) ** (-2.0 * torch.arange(0, half, dtype=torch.float64) / s.rotary_dim)
                ang = torch.outer(torch.arange(s.max_positions, dtype=torch.float64), f)
                shared = _TABLES[key] = (ang.cos().float().contiguous().to(self.env.device),
                                         ang.sin().float().contiguous().to(self.env.device), s.rotary_dim)
            self._tables = shared
        return self._tables
