"""A recurrent mixer: a linear recurrence with a matrix state per head, fed through a token shift."""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorNeed
from .base import MIXERS, CacheNeed, Mixer
from .linear import Linear

MIXES = ("r", "k", "v", "g", "w")


class MatrixStateRecurrence(Mixer):
    """Time mixing in the manner of RWKV.  With h the input row and h' the row of the sequence's previous token
    (zeros before the first), each of r, k, v, g, w reads its own blend h + (h' - h) mu_s.  r, k, v = W_r, W_k, W_v of
    their blends, split into `heads` heads of `head_dim` channels; gate = silu(W_g blend_g); the decay
    w = exp(-exp(W_w2 tanh(W_w1 blend_w) + w0)) per head and key channel.  Per head, with the state S [key channel, value
    channel] (zero at a sequence's start):  o_t = (S + diag(u) k_t v_t^T)^T r_t, then S = diag(w_t) S + k_t v_t^T.  Each
    head's o is divided by its root mean square (`eps`), the heads are concatenated, multiplied by `norm` and by the gate,
    and projected by W_o.

    What a sequence keeps is one float32 row: the heads' matrices, then the last input row (for the next token's shift).
    The decay, the state and the scan are float32 whatever the run's dtype; the projections run in the run's dtype.
    A sequence's result depends on its own rows and state only.

    Parameters: hidden_size, heads, head_dim, decay_rank, eps, names.{mu (pattern with {s}), r, k, v, g, w1, w2, w0, u,
    norm, o}.
    """
    replayable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["heads"])
        self.n = int(spec["head_dim"])
        self.rank = int(spec["decay_rank"])
        self.eps = float(spec["eps"])
        self.hn = self.heads * self.n
        self.mu = self.w0 = self.u = self.norm = None
        self.proj = {}
        self.w1 = self.w2 = self.o = None

    @staticmethod
    def state_floats(spec: PartSpec) -> int:
        return int(spec["heads"]) * int(spec["head_dim"]) ** 2 + int(spec["hidden_size"])

    @staticmethod
    def cache_need(spec: PartSpec) -> CacheNeed:
        return CacheNeed("state", state_shape=(MatrixStateRecurrence.state_floats(spec),))

    @staticmethod
    def tensor_needs(spec: PartSpec) -> List[TensorNeed]:
        h, hn, rank, n = int(spec["hidden_size"]), int(spec["heads"]) * int(spec["head_dim"]), int(spec["decay_rank"]), spec["names"]
        needs = [TensorNeed(n["mu"].format(s=s), (h,), role="vector", init="linear") for s in MIXES]
        needs += [TensorNeed(n[s], (hn, h)) for s in ("r", "k", "v", "g")]
        needs += [TensorNeed(n["w1"], (rank, h)), TensorNeed(n["w2"], (hn, rank)),
                  TensorNeed(n["w0"], (hn,), role="vector", init="linear"),
                  TensorNeed(n["u"], (int(spec["heads"]), int(spec["head_dim"])), role="vector", init="linear"),
                  TensorNeed(n["norm"], (hn,), role="vector", init="norm"), TensorNeed(n["o"], (h, hn))]
        return needs

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.spec["names"]
        self.mu = torch.stack([tensors[n["mu"].format(s=s)].to(torch.float32) for s in MIXES]).contiguous()
        self.proj = {s: Linear(tensors[n[s]]) for s in ("r", "k", "v", "g")}
        self.w1, self.w2, self.o = Linear(tensors[n["w1"]]), Linear(tensors[n["w2"]]), Linear(tensors[n["o"]])
        self.w0 = tensors[n["w0"]].to(torch.float32).contiguous()
        self.u = tensors[n["u"]].to(torch.float32).reshape(-1).contiguous()
        self.norm = tensors[n["norm"]].to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return sum(l.weight_bytes() for l in self.proj.values()) + self.w1.weight_bytes() + self.w2.weight_bytes() + self.o.weight_bytes()

    def forward(self, ctx, entry, x, n_rows, cache_entry=None, write_cache=True):
        if cache_entry is not None or not write_cache:
            raise ValueError("a recurrent mixer keeps a state of its own; it cannot read another entry's")
        ws, dt, rows = ctx.ws, self.env.dtype, ctx.ws.max_rows
        state = ctx.cache.state(entry)
        mixes = ws.buffer("wkv.mixes", (len(MIXES), rows, self.hidden), dt)
        ops.token_shift_mix(x, self.mu, mixes, state, self.heads * self.n * self.n, ctx.row_slot, ctx.row_pos, n_rows)
        out = {}
        for i, s in enumerate(("r", "k", "v", "g")):
            out[s] = ws.buffer("wkv." + s, (rows, self.hn), dt)
            self.proj[s](mixes[i], out[s], n_rows)
        low = ws.buffer("wkv.decay_low", (rows, self.rank), torch.float32)
        low_t = ws.buffer("wkv.decay_tanh", (rows, self.rank), dt)
        z = ws.buffer("wkv.decay_z", (rows, self.hn), torch.float32)
        self.w1(mixes[4], low, n_rows)
        ops.tanh_rows(low, low_t, n_rows)
        self.w2(low_t, z, n_rows)
        o = ws.buffer("wkv.o", (rows, self.hn), torch.float32)
        ops.wkv_scan(out["r"], out["k"], out["v"], z, self.w0, self.u, x, o, state, ctx.seq_first_row, ctx.seq_slot, ctx.n_seqs,
                     self.heads, self.n, one_token=ctx.decode)
        gated = ws.buffer("wkv.gated", (rows, self.hn), dt)
        ops.head_norm_gate(o, self.norm, out["g"], gated, n_rows, self.heads, self.n, self.eps)
        delta = ws.buffer("delta", (rows, self.hidden), dt)
        self.o(gated, delta, n_rows)
        return delta


MIXERS.register("matrix_state_recurrence", MatrixStateRecurrence)
