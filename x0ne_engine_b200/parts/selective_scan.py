"""A selective state-space mixer: a short causal convolution, then a linear recurrence whose step size and in- and
output weights depend on the token."""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorNeed
from .base import MIXERS, CacheNeed, Mixer
from .linear import Linear


class SelectiveScan(Mixer):
    """W_in x = [u' | z] of `inner` channels each.  u = silu(conv(u') + b): per channel, `conv` taps over the sequence's
    last inputs (zeros before its first token; the last tap meets the current token).  W_x u = [low: dt_rank | B: state |
    C: state]; dt = softplus(W_dt low + dt_bias), one per channel; A = -exp(A_log) [inner, state].  Per channel c and
    state n, with S zero at a sequence's start:
        S[c, n] = exp(dt_c A[c, n]) S[c, n] + dt_c u_c B_n;     y_c = sum_n S[c, n] C_n + D_c u_c,
    then y * silu(z), projected by W_o.

    What a sequence keeps is one float32 row: S, then the convolution's last `conv` - 1 inputs.  Step sizes, decays,
    B, C, the state and every sum of the recurrence are float32 whatever the run's dtype (the two small products write
    float32); the projections, the convolution's output and z are in the run's dtype.  A sequence's result depends on
    its own rows and state only.

    Parameters: hidden_size, inner, state, conv, dt_rank, names.{in, conv, conv_bias, x, dt, dt_bias, A_log, D, o}.
    """
    replayable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden_size"])
        self.inner = int(spec["inner"])
        self.n = int(spec["state"])
        self.taps = int(spec["conv"])
        self.rank = int(spec["dt_rank"])
        self.conv_off = self.inner * self.n
        self.w_in = self.w_low = self.w_bc = self.w_dt = self.o = None
        self.conv_w = self.conv_b = self.dt_bias = self.A = self.D = None

    @staticmethod
    def state_floats(spec: PartSpec) -> int:
        return int(spec["inner"]) * (int(spec["state"]) + int(spec["conv"]) - 1)

    @staticmethod
    def cache_need(spec: PartSpec) -> CacheNeed:
        return CacheNeed("state", state_shape=(SelectiveScan.state_floats(spec),))

    @staticmethod
    def tensor_needs(spec: PartSpec) -> List[TensorNeed]:
        h, i, s, k, r = (int(spec[key]) for key in ("hidden_size", "inner", "state", "conv", "dt_rank"))
        n = spec["names"]
        return [TensorNeed(n["in"], (2 * i, h)), TensorNeed(n["conv"], (i, k), role="vector", init="linear"),
                TensorNeed(n["conv_bias"], (i,), role="vector", init="linear"), TensorNeed(n["x"], (r + 2 * s, i)),
                TensorNeed(n["dt"], (i, r)), TensorNeed(n["dt_bias"], (i,), role="vector", init="linear"),
                TensorNeed(n["A_log"], (i, s), role="vector", init="linear"), TensorNeed(n["D"], (i,), role="vector", init="norm"),
                TensorNeed(n["o"], (h, i))]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.spec["names"]
        self.w_in, self.o = Linear(tensors[n["in"]]), Linear(tensors[n["o"]])
        wx = tensors[n["x"]]
        # the step size's low-rank part feeds a product and stays in the run's dtype; B and C enter the recurrence and
        # are written in float32 by a product of their own
        self.w_low, self.w_bc = Linear(wx[:self.rank].contiguous()), Linear(wx[self.rank:].contiguous())
        self.w_dt = Linear(tensors[n["dt"]])
        f32 = lambda t: t.to(torch.float32).contiguous()
        self.conv_w, self.conv_b, self.dt_bias, self.D = (f32(tensors[n[s]]) for s in ("conv", "conv_bias", "dt_bias", "D"))
        self.A = (-torch.exp(f32(tensors[n["A_log"]]))).contiguous()

    def weight_bytes(self) -> int:
        return sum(l.weight_bytes() for l in (self.w_in, self.w_low, self.w_bc, self.w_dt, self.o))

    def forward(self, ctx, entry, x, n_rows, cache_entry=None, write_cache=True):
        if cache_entry is not None or not write_cache:
            raise ValueError("a recurrent mixer keeps a state of its own; it cannot read another entry's")
        ws, dt, rows = ctx.ws, self.env.dtype, ctx.ws.max_rows
        state = ctx.cache.state(entry)
        xz = ws.buffer("ssm.xz", (rows, 2 * self.inner), dt)
        u = ws.buffer("ssm.u", (rows, self.inner), dt)
        low = ws.buffer("ssm.low", (rows, self.rank), dt)
        bc = ws.buffer("ssm.bc", (rows, 2 * self.n), torch.float32)
        dt_raw = ws.buffer("ssm.dt", (rows, self.inner), torch.float32)
        y = ws.buffer("ssm.y", (rows, self.inner), dt)
        delta = ws.buffer("delta", (rows, self.hidden), dt)
        self.w_in(x, xz, n_rows)
        ops.causal_conv_silu(xz, self.conv_w, self.conv_b, state, self.conv_off, u, ctx.row_slot, ctx.row_pos, n_rows, self.inner)
        self.w_low(u, low, n_rows)
        self.w_bc(u, bc, n_rows)
        self.w_dt(low, dt_raw, n_rows)
        ops.selective_scan(u, xz, self.inner, dt_raw, self.dt_bias, self.A, bc, 0, self.n, self.D, y, state, self.conv_off, self.taps,
                           ctx.seq_first_row, ctx.seq_slot, ctx.n_seqs, one_token=ctx.decode)
        self.o(y, delta, n_rows)
        return delta


MIXERS.register("selective_scan", SelectiveScan)
