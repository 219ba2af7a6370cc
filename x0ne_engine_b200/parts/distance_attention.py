"""Grouped-query attention without rotation: positions enter through a linear distance bias, a sliding window and a
temperature on the queries."""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorNeed
from .attention import run_attention_ex
from .base import MIXERS, CacheNeed, Mixer
from .linear import Linear


def distance_slopes(heads: int, span: float = 8.0) -> List[float]:
    """2^(-span (h + 1) / heads) for h = 0 .. heads-1: a geometric ladder from just below 1 down to 2^-span."""
    return [2.0 ** (-span * (h + 1) / heads) for h in range(heads)]


class DistanceBiasAttention(Mixer):
    """q, k, v and the output gate from one product on the packed [q; k; v; g] weight.  Queries and keys are normed
    per head (RMS over head_dim, one weight of head_dim values shared by all heads, `qk_norm_eps`); nothing is rotated.
    The query at position p is multiplied by 1 + `temp_coef` ln(floor((p + 1) / `temp_every`) + 1) (`temp_every` None:
    no such factor).  With `v_unit` each head's value is divided by its root mean square (no weight) and is cached so.
    The score of query i and key j is q.k * `scale` - slope_h (i - j) with slope_h = 2^(-`slope_span` (h + 1) / heads)
    (`slope_span` None: no bias); i sees j with 0 <= i - j < `window` (None: every j <= i); ordinary softmax.  The
    concatenated heads are multiplied value by value with sigmoid(W_g x) (`gate`), then projected by W_o.
    q head h reads kv head h // (q_heads // kv_heads); keys of `head_dim`, values of `v_dim`.

    The cache keeps every position (pages); the window bounds what a query reads.

    Parameters: hidden_size, q_heads, kv_heads, head_dim, v_dim, scale, window, qk_norm_eps, temp_coef, temp_every,
    v_unit, slope_span, gate, names.{q, k, v, g, o, q_norm, k_norm}.
    """
    replayable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        g = spec.get
        self.hidden = int(spec["hidden_size"])
        self.q_heads = int(spec["q_heads"])
        self.kv_heads = int(spec["kv_heads"])
        self.head_dim = int(spec["head_dim"])
        self.v_dim = int(g("v_dim") or self.head_dim)
        if self.q_heads % self.kv_heads:
            raise ValueError("q heads are not a multiple of kv heads")
        self.scale = float(spec["scale"])
        self.window = int(g("window") or 0)
        self.eps = float(spec["qk_norm_eps"])
        self.temp_every = int(g("temp_every") or 0)
        self.temp_coef = float(g("temp_coef") or 0.0) if self.temp_every else 0.0
        self.v_unit = bool(g("v_unit"))
        self.slope_span = g("slope_span")
        self.gated = bool(g("gate"))
        self.q_dim = self.q_heads * self.head_dim
        self.k_dim = self.kv_heads * self.head_dim
        self.kv_v_dim = self.kv_heads * self.v_dim
        self.out_dim = self.q_heads * self.v_dim
        self.g_col = self.q_dim + self.k_dim + self.kv_v_dim
        self.width = self.g_col + (self.out_dim if self.gated else 0)
        self.slopes = None
        if self.slope_span is not None:
            self.slopes = torch.tensor(distance_slopes(self.q_heads, float(self.slope_span)), dtype=torch.float32, device=env.device)
        self.proj = self.o = self.q_norm = self.k_norm = None

    @staticmethod
    def cache_need(spec: PartSpec) -> CacheNeed:
        hd = int(spec["head_dim"])
        vd = int(spec.get("v_dim") or hd)
        return CacheNeed("kv", int(spec["kv_heads"]), hd, None, v_dim=None if vd == hd else vd)

    @staticmethod
    def tensor_needs(spec: PartSpec) -> List[TensorNeed]:
        h, hd = int(spec["hidden_size"]), int(spec["head_dim"])
        vd, n = int(spec.get("v_dim") or hd), spec["names"]
        qh, kvh = int(spec["q_heads"]), int(spec["kv_heads"])
        needs = [TensorNeed(n["q"], (qh * hd, h)), TensorNeed(n["k"], (kvh * hd, h)), TensorNeed(n["v"], (kvh * vd, h)),
                 TensorNeed(n["q_norm"], (hd,), role="vector", init="norm"), TensorNeed(n["k_norm"], (hd,), role="vector", init="norm")]
        if spec.get("gate"):
            needs.append(TensorNeed(n["g"], (qh * vd, h)))
        needs.append(TensorNeed(n["o"], (h, qh * vd)))
        return needs

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.spec["names"]
        rows = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]] + ([tensors[n["g"]]] if self.gated else [])
        self.proj = Linear(torch.cat(rows, dim=0).contiguous())
        self.q_norm, self.k_norm = tensors[n["q_norm"]], tensors[n["k_norm"]]
        self.o = Linear(tensors[n["o"]])

    def weight_bytes(self) -> int:
        return self.proj.weight_bytes() + self.o.weight_bytes()

    def forward(self, ctx, entry, x, n_rows, cache_entry=None, write_cache=True):
        if cache_entry is not None or not write_cache:
            raise ValueError("this attention keeps keys and values of its own")
        dt, rows = self.env.dtype, ctx.ws.max_rows
        proj = ctx.ws.buffer("dattn.proj", (rows, self.width), dt)
        q = ctx.ws.buffer("dattn.q", (rows, self.q_dim), dt)
        att = ctx.ws.buffer("dattn.out", (rows, self.out_dim), dt)
        out = ctx.ws.buffer("delta", (rows, self.hidden), dt)
        self.proj(x, proj, n_rows)
        view = ctx.cache.kv_view(entry)
        if view.kv_heads != self.kv_heads or view.head_dim != self.head_dim or view.value_dim != self.v_dim:
            raise ValueError("the cache this layer reads does not have its key and value heads")
        ops.head_norm_kv_write(proj, self.q_dim, self.q_dim + self.k_dim, self.q_norm, self.k_norm, self.eps, self.temp_coef,
                               self.temp_every, self.v_unit, q, self.q_heads, view, ctx.row_slot, ctx.row_pos, n_rows)
        gate = proj[:, self.g_col:] if self.gated else None
        extra = ops.attn_extra(gate=gate, gate_ld=self.width, gate_wide=self.gated, slope=self.slopes)
        run_attention_ex(ctx, q, att, view, n_rows, self.q_heads, self.scale, self.window, extra)
        self.o(att, out, n_rows)
        return out


MIXERS.register("distance_bias_attention", DistanceBiasAttention)
