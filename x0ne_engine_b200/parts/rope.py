"""Rotary position encoding: the table of inverse frequencies."""
from __future__ import annotations

import math

import numpy as np
import torch

from .base import POSITIONS, PositionEncoding


def inv_freq_f32(rotary_dim: int, theta: float) -> np.ndarray:
    """1 / theta^(2i / d) for i < d/2, computed on the host in float32 with theta narrowed to
    float32 first (x0ne-core/runtime/src/ops.rs:210-214, x0ne-core/runtime/src/engine.rs:351)."""
    t = np.float32(theta)
    d = np.float32(rotary_dim)
    return np.array([np.float32(1.0) / np.power(t, np.float32(2 * i) / d, dtype=np.float32)
                     for i in range(rotary_dim // 2)], dtype=np.float32)


class Rope(PositionEncoding):
    """Rotate-half RoPE over the first `rotary_dim` values of each head: the pair
    (i, i + rotary_dim/2) turns by pos * inv_freq[i] (x0ne-core/kernels/cuda/rope.cu:28-31).
    The rotation itself runs inside the mixer's fused kernel; this part owns the table.
    Parameters: head_dim, rotary_dim, theta, freq_in_double (default False: the frequencies are worked
    out in float32 from a float32 theta; True: in float64, then narrowed once)."""
    replayable = True
    TABLE_POSITIONS = 1 << 16      # the table covers this many positions at most; kernels compute the rest

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.head_dim = int(spec["head_dim"])
        self.rotary_dim = int(spec.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.theta = float(spec["theta"])
        if spec.get("freq_in_double"):
            i = np.arange(self.rotary_dim // 2, dtype=np.float64)
            self.inv_freq = np.power(self.theta, -2.0 * i / self.rotary_dim).astype(np.float32)
        else:
            self.inv_freq = inv_freq_f32(self.rotary_dim, self.theta)
        self.table = torch.from_numpy(self.inv_freq).to(env.device)
        self._cos_sin = None

    def rotary(self):
        return self.table, self.rotary_dim

    def cos_sin_table(self, positions: int):
        """float32 [positions, rotary_dim]: cos then sin of the float32 angle position * inv_freq[i],
        made once on the host; mixers pass it to the fused kernel so that it reads two short rows
        instead of computing the row's sines and cosines for every head."""
        positions = max(1, min(int(positions), self.TABLE_POSITIONS))
        if self._cos_sin is None or self._cos_sin.shape[0] < positions:
            pos = np.arange(positions, dtype=np.float32)[:, None]
            ang = (pos * self.inv_freq[None, :]).astype(np.float32).astype(np.float64)
            tab = np.concatenate([np.cos(ang), np.sin(ang)], axis=1).astype(np.float32)
            self._cos_sin = torch.from_numpy(tab).to(self.env.device)
        return self._cos_sin


def yarn_frequencies(rotary_dim: int, theta: float, scaling) -> tuple:
    """(frequency per pair as float64 [rotary_dim / 2], factor on cos and sin).

    Plain frequencies are f_i = theta^(-2i / rotary_dim).  With `scaling` = {factor, original, fast,
    slow} (YaRN): the pair index at which a wave makes t turns over `original` positions is
    idx(t) = rotary_dim ln(original / (2 pi t)) / (2 ln theta); pairs below lo = max(floor(idx(fast)), 0)
    keep f_i, pairs above hi = min(ceil(idx(slow)), rotary_dim - 1) get f_i / factor, and between them
    the two are blended linearly; cos and sin are multiplied by 0.1 ln(factor) + 1."""
    i = np.arange(rotary_dim // 2, dtype=np.float64)
    f = np.power(float(theta), -2.0 * i / rotary_dim)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def idx(turns: float) -> float:
        return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(theta)))

    lo = max(math.floor(idx(float(scaling["fast"]))), 0)
    hi = min(math.ceil(idx(float(scaling["slow"]))), rotary_dim - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


class YarnRope(PositionEncoding):
    """Rotary encoding over `rotary_dim` values with YaRN-scaled frequencies.  `layout` says which
    values pair up: "interleaved" turns value 2i with value 2i + 1, "half" value i with value
    i + rotary_dim / 2.  The pair (u, v) at position p becomes (u c - v s, v c + u s) with
    c = mag cos(p f_i), s = mag sin(p f_i).  The rotation runs inside the mixer's kernel; this part
    owns the frequencies and the table.  Parameters: rotary_dim, theta, scaling (None or {factor,
    original, fast, slow}), layout, angle_in_float32 (default False: the table's angles are position x
    frequency in float64; True: the float32 product of the float32 position and frequency, what a kernel
    that computes the angle itself gets)."""
    replayable = True
    TABLE_POSITIONS = 1 << 16      # the table covers this many positions at most; kernels compute the rest

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.rotary_dim = int(spec["rotary_dim"])
        if self.rotary_dim % 2 or self.rotary_dim <= 0:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and positive")
        self.theta = float(spec["theta"])
        self.angle_in_float32 = bool(spec.get("angle_in_float32"))
        self.layout = spec.get("layout", "interleaved")
        if self.layout not in ("interleaved", "half"):
            raise ValueError(f"rotary layout {self.layout!r} is neither 'interleaved' nor 'half'")
        self.freq64, self.mag = yarn_frequencies(self.rotary_dim, self.theta, spec.get("scaling"))
        self.inv_freq = self.freq64.astype(np.float32)
        self.table = torch.from_numpy(self.inv_freq).to(env.device)
        self._cos_sin = None

    def rotary(self):
        return self.table, self.rotary_dim

    def cos_sin_table(self, positions: int):
        """float32 [positions, rotary_dim]: mag cos then mag sin of position x frequency, the angle taken
        in float64 on the host."""
        positions = max(1, min(int(positions), self.TABLE_POSITIONS))
        if self._cos_sin is None or self._cos_sin.shape[0] < positions:
            if self.angle_in_float32:
                ang = (np.arange(positions, dtype=np.float32)[:, None] * self.inv_freq[None, :]).astype(np.float32).astype(np.float64)
            else:
                ang = np.arange(positions, dtype=np.float64)[:, None] * self.freq64[None, :]
            tab = (np.concatenate([np.cos(ang), np.sin(ang)], axis=1) * self.mag).astype(np.float32)
            self._cos_sin = torch.from_numpy(tab).to(self.env.device)
        return self._cos_sin


class NoPosition(PositionEncoding):
    """No position encoding: mixers leave q and k unrotated."""
    replayable = True


POSITIONS.register("rope", Rope)
POSITIONS.register("none", NoPosition)
POSITIONS.register("yarn_rope", YarnRope)
