"""Differential attention: two softmax maps per head over the same values, one taken off the other."""
from __future__ import annotations

import math
from typing import List, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorNeed
from .attention import run_attention_ex
from .base import MIXERS, CacheNeed, Mixer
from .linear import Linear


class DifferentialAttention(Mixer):
    """q, k, v and the output gate from one product on the packed [q; k; v; g] weight.  Every query head holds two
    queries of `head_dim` values side by side (map 1, map 2) and every kv head two keys; both maps read the kv head's
    one value of `v_dim` values.  Queries and keys turn by the model's position encoding (`position`, interleaved
    pairs, over the first rotary_dim values of every map).  Each map is a causal softmax attention with the scores
    q.k * `scale`; with a1, a2 the maps' results of a head,
        o = a1 - lambda a2,   lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + `lambda_init`    (one number per layer),
    then o / sqrt(mean(o^2) + `eps`) over the head's values, times 1 - `lambda_init`.  The concatenated heads are
    multiplied value by value with sigmoid(W_g x) (`gate`), then projected by W_o.  q head h reads kv head
    h // (q_heads // kv_heads).

    The cache keeps a kv head's two keys as one row of 2 head_dim values beside its value.  The two maps run as
    2 q_heads query heads of the general attention kernels: a map's query is placed in its half of a row of 2 head_dim
    values with zeros in the other half, so its product with the whole key row is its product with its own key.
    Scores, softmax, the maps' results (the attention kernels write them as float32: the difference of two like maps,
    brought back to unit size, would multiply the rounding of 16-bit results), the difference, the norm and the gate
    are float32; lambda is worked out once at bind, in double precision.

    Parameters: hidden_size, q_heads, kv_heads, head_dim, v_dim, scale, lambda_init, eps, position, gate,
    names.{q, k, v, g, o, lq1, lk1, lq2, lk2}.
    """
    replayable = True
    MAPS = 2

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
        self.lambda_init = float(spec["lambda_init"])
        self.eps = float(spec["eps"])
        self.gated = bool(g("gate"))
        pos = g("position")
        self.position = env.positions[pos] if pos is not None else None
        if self.position is not None and getattr(self.position, "layout", None) != "interleaved":
            raise ValueError("this attention rotates interleaved pairs; its position encoding has another layout")
        m = self.MAPS
        self.q_dim = self.q_heads * m * self.head_dim
        self.k_dim = self.kv_heads * m * self.head_dim
        self.kv_v_dim = self.kv_heads * self.v_dim
        self.out_dim = self.q_heads * self.v_dim
        self.g_col = self.q_dim + self.k_dim + self.kv_v_dim
        self.width = self.g_col + (self.out_dim if self.gated else 0)
        self.lam = 0.0
        self.proj = self.o = None

    @staticmethod
    def cache_need(spec: PartSpec) -> CacheNeed:
        hd = DifferentialAttention.MAPS * int(spec["head_dim"])
        vd = int(spec.get("v_dim") or spec["head_dim"])
        return CacheNeed("kv", int(spec["kv_heads"]), hd, None, v_dim=None if vd == hd else vd)

    @staticmethod
    def tensor_needs(spec: PartSpec) -> List[TensorNeed]:
        h, hd, m = int(spec["hidden_size"]), int(spec["head_dim"]), DifferentialAttention.MAPS
        vd, n = int(spec.get("v_dim") or hd), spec["names"]
        qh, kvh = int(spec["q_heads"]), int(spec["kv_heads"])
        needs = [TensorNeed(n["q"], (qh * m * hd, h)), TensorNeed(n["k"], (kvh * m * hd, h)), TensorNeed(n["v"], (kvh * vd, h))]
        needs += [TensorNeed(n[s], (hd,), role="vector", init="linear") for s in ("lq1", "lk1", "lq2", "lk2")]
        if spec.get("gate"):
            needs.append(TensorNeed(n["g"], (qh * vd, h)))
        needs.append(TensorNeed(n["o"], (h, qh * vd)))
        return needs

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.spec["names"]
        rows = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]] + ([tensors[n["g"]]] if self.gated else [])
        self.proj = Linear(torch.cat(rows, dim=0).contiguous())
        self.o = Linear(tensors[n["o"]])
        lq1, lk1, lq2, lk2 = (tensors[n[s]].detach().to("cpu", torch.float64) for s in ("lq1", "lk1", "lq2", "lk2"))
        self.lam = math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + self.lambda_init

    def weight_bytes(self) -> int:
        return self.proj.weight_bytes() + self.o.weight_bytes()

    def forward(self, ctx, entry, x, n_rows, cache_entry=None, write_cache=True):
        if cache_entry is not None or not write_cache:
            raise ValueError("this attention keeps keys and values of its own")
        dt, rows, m = self.env.dtype, ctx.ws.max_rows, self.MAPS
        proj = ctx.ws.buffer("diffattn.proj", (rows, self.width), dt)
        q = ctx.ws.buffer("diffattn.q", (rows, self.q_heads * m * m * self.head_dim), dt)
        maps = ctx.ws.buffer("diffattn.maps", (rows, self.q_heads * m * self.v_dim), torch.float32)
        att = ctx.ws.buffer("diffattn.out", (rows, self.out_dim), dt)
        out = ctx.ws.buffer("delta", (rows, self.hidden), dt)
        self.proj(x, proj, n_rows)
        view = ctx.cache.kv_view(entry)
        if view.kv_heads != self.kv_heads or view.head_dim != m * self.head_dim or view.value_dim != self.v_dim:
            raise ValueError("the cache this layer reads does not have its key and value heads")
        freq, rot = self.position.rotary() if self.position is not None else (None, 0)
        table = self.position.cos_sin_table(self.env.max_positions) if rot and self.env.max_positions else None
        ops.rope_pairs_kv_write(proj, self.q_dim, self.q_dim + self.k_dim, freq, table, rot, m, self.head_dim, None, q, self.q_heads,
                                True, view, ctx.row_slot, ctx.row_pos, n_rows)
        run_attention_ex(ctx, q, maps, view, n_rows, self.q_heads * m, self.scale, 0, ops.attn_extra(out_f32=True))
        gate = proj[:, self.g_col:] if self.gated else None
        ops.diff_heads(maps, gate, self.width, att, n_rows, self.q_heads, self.v_dim, self.lam, self.eps, 1.0 - self.lambda_init)
        self.o(att, out, n_rows)
        return out


MIXERS.register("differential_attention", DifferentialAttention)
