"""Grouped-query attention with a mask of its own, free key and value widths, and value blending."""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorNeed
from .attention import run_attention_ex
from .base import MIXERS, CacheNeed, Mixer
from .linear import Linear


class MaskedAttention(Mixer):
    """q, k, v from one product on the packed [q; k; v] weight; keys of `head_dim` and
    values of `v_dim` per kv head written to the cache; softmax attention of every query over the
    keys j <= i it may see: all of them, the last `window`, or (with `chunk` = c) those with
    floor(j / c) = floor(i / c), chunks counted from the sequence's first position; q head h reads kv
    head h // (q_heads // kv_heads); output projection.

    Without `position` nothing is rotated.  With it (the name of a position encoding of the model whose pairs are
    interleaved) queries and keys turn by their positions, and with `qk_unit_eps` each head's query and key is then
    divided by its root mean square (no weight).  `sink_zero` adds one term of score zero to every softmax
    denominator: exp(s_j) / (1 + sum exp(s)).

    Value blending (`v_blend`): the first layer of a model that says "source" keeps its values of the
    pass's rows; a layer that says "blend" replaces its own by (1 - a) v + a v_source with its learned
    scalar a (`names.v_blend`), and caches the blended values.  All blending layers share the
    source's kv_heads x v_dim.

    Parameters: hidden_size, q_heads, kv_heads, head_dim, v_dim, scale, chunk (None: no chunks), window
    (None: all keys), v_blend (None | "source" | "blend"), position, qk_unit_eps, sink_zero, names.{q, k, v, o, v_blend}.
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
        self.chunk = int(g("chunk") or 0)
        self.window = int(g("window") or 0)
        self.v_blend = g("v_blend")
        if self.v_blend not in (None, "source", "blend"):
            raise ValueError(f"v_blend {self.v_blend!r} is not None, 'source' or 'blend'")
        pos = g("position")
        self.position = env.positions[pos] if pos is not None else None
        if self.position is not None and getattr(self.position, "layout", None) != "interleaved":
            raise ValueError("this attention rotates interleaved pairs; its position encoding has another layout")
        self.qk_unit_eps = g("qk_unit_eps")
        self.prepared = self.position is not None or self.qk_unit_eps is not None    # queries and keys change on their way
        if self.prepared and self.v_blend is not None:
            raise ValueError("value blending together with rotated or normed queries and keys is not served")
        self.sink = torch.zeros(self.q_heads, dtype=torch.float32, device=env.device) if g("sink_zero") else None
        self.q_dim = self.q_heads * self.head_dim
        self.k_dim = self.kv_heads * self.head_dim
        self.kv_v_dim = self.kv_heads * self.v_dim
        self.qkv = self.o = self.blend = None

    @staticmethod
    def cache_need(spec: PartSpec) -> CacheNeed:
        hd = int(spec["head_dim"])
        vd = int(spec.get("v_dim") or hd)
        return CacheNeed("kv", int(spec["kv_heads"]), hd, spec.get("window"), v_dim=None if vd == hd else vd)

    @staticmethod
    def tensor_needs(spec: PartSpec) -> List[TensorNeed]:
        h, hd = int(spec["hidden_size"]), int(spec["head_dim"])
        vd, n = int(spec.get("v_dim") or hd), spec["names"]
        qh, kvh = int(spec["q_heads"]), int(spec["kv_heads"])
        needs = [TensorNeed(n["q"], (qh * hd, h)), TensorNeed(n["k"], (kvh * hd, h)), TensorNeed(n["v"], (kvh * vd, h)),
                 TensorNeed(n["o"], (h, qh * vd))]
        if spec.get("v_blend") is not None:
            # every blending layer of a checkpoint carries the scalar; the source's is not read
            needs.append(TensorNeed(n["v_blend"], (), role="vector", init="norm"))
        return needs

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.spec["names"]
        self.qkv = Linear(torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]], dim=0).contiguous())
        self.o = Linear(tensors[n["o"]])
        if self.v_blend == "blend":
            self.blend = tensors[n["v_blend"]].reshape(1).contiguous()

    def weight_bytes(self) -> int:
        return self.qkv.weight_bytes() + self.o.weight_bytes()

    def forward(self, ctx, entry, x, n_rows, cache_entry=None, write_cache=True):
        dt, rows = self.env.dtype, ctx.ws.max_rows
        width = self.q_dim + self.k_dim + self.kv_v_dim
        qkv = ctx.ws.buffer("mattn.qkv", (rows, width), dt)
        att = ctx.ws.buffer("mattn.out", (rows, self.q_heads * self.v_dim), dt)
        out = ctx.ws.buffer("delta", (rows, self.hidden), dt)
        self.qkv(x, qkv, n_rows)
        view = ctx.cache.kv_view(entry if cache_entry is None else cache_entry)
        if self.prepared:
            q = ctx.ws.buffer("mattn.q", (rows, self.q_dim), dt)
            freq, rot = self.position.rotary() if self.position is not None else (None, 0)
            table = self.position.cos_sin_table(self.env.max_positions) if rot and self.env.max_positions else None
            ops.rope_pairs_kv_write(qkv, self.q_dim, self.q_dim + self.k_dim, freq, table, rot, 1, self.head_dim,
                                    None if self.qk_unit_eps is None else float(self.qk_unit_eps), q, self.q_heads, False, view,
                                    ctx.row_slot, ctx.row_pos, n_rows, write_cache)
            extra = ops.attn_extra(chunk=self.chunk, sink=self.sink)
            run_attention_ex(ctx, q, att, view, n_rows, self.q_heads, self.scale, self.window, extra)
            self.o(att, out, n_rows)
            return out
        if write_cache:
            mode = {None: 0, "source": 1, "blend": 2}[self.v_blend]
            first = ctx.ws.buffer("mattn.v_source", (rows, self.kv_v_dim), dt) if mode else None
            ops.kv_write_blend(qkv, self.q_dim, self.q_dim + self.k_dim, view, ctx.row_slot, ctx.row_pos, n_rows, mode,
                               first, self.blend)
        extra = ops.attn_extra(chunk=self.chunk, q_ld=width, sink=self.sink)
        run_attention_ex(ctx, qkv, att, view, n_rows, self.q_heads, self.scale, self.window, extra)
        self.o(att, out, n_rows)
        return out


MIXERS.register("masked_attention", MaskedAttention)
