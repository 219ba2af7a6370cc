"""Retuvik restated in plain PyTorch on the CPU, one function per mechanism.

Nothing here is shared with the package: the functions take a config.json as a dict and the
checkpoint tensors by name (any dtype; they are widened to the working precision), run a whole
sequence with explicit loops over tokens (the recurrence) or full T x T score matrices (the
attention), and return the logits of every position.

Notation: T tokens, width W.  Recurrent mixer: H heads of N channels, state S[h] of N x N (key channel
by value channel).  Attention: H query heads, G key/value heads, key width D, value width Dv, window n.
Routed feed-forward: E experts, k chosen per token.
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional

import torch
import torch.nn.functional as F

PRECISION = torch.float32      # the tests set float64: the same equations, as a sharper reference


def f32(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to("cpu", PRECISION)


# ------------------------------------------------------------------------------------------ norms
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def group_norm(x: torch.Tensor, w: torch.Tensor, eps: float, groups: int) -> torch.Tensor:
    """The last axis in `groups` equal consecutive parts, each brought to unit root mean square by itself;
    the whole times w."""
    parts = x.reshape(*x.shape[:-1], groups, x.shape[-1] // groups)
    return unit_rms(parts, eps).reshape(x.shape) * w


# ------------------------------------------------------------------------------------------ recurrent mixer
def shifted(h: torch.Tensor, before: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row t holds h[t-1]; row 0 holds `before` (what the sequence saw last), or zeros."""
    first = torch.zeros_like(h[:1]) if before is None else before.reshape(1, -1).to(h.dtype)
    return torch.cat([first, h[:-1]], dim=0)


def decay(mix_w: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, w0: torch.Tensor) -> torch.Tensor:
    """exp(-exp(w0 + W2 tanh(W1 x))): one number in (0, 1) per head and key channel."""
    return torch.exp(-torch.exp(torch.tanh(mix_w @ w1.T) @ w2.T + w0))


def wkv_scan(r, k, v, w, u, S):
    """r, k, v, w [T, H, N]; u [H, N]; S [H, N, N] is changed in place.  Token by token:
    out[t, h, j] = sum_i r[t, h, i] (S[h, i, j] + u[h, i] k[t, h, i] v[t, h, j]), then
    S[h, i, j] = w[t, h, i] S[h, i, j] + k[t, h, i] v[t, h, j]."""
    T = r.shape[0]
    out = torch.zeros_like(v)
    for t in range(T):
        kv = k[t, :, :, None] * v[t, :, None, :]
        out[t] = torch.einsum("hi,hij->hj", r[t], S + u[:, :, None] * kv)
        S.mul_(w[t, :, :, None]).add_(kv)
    return out


def wkv_mixer(h: torch.Tensor, mixer: Mapping, t: Mapping[str, torch.Tensor], p: str, eps: float,
              state: Optional[Dict] = None) -> torch.Tensor:
    """The recurrent mixer over the rows of h [T, W].  `state` (a dict with "S" and "last", or empty / None for a
    sequence's start) is read and left as the rows leave it."""
    H, N = mixer["heads"], mixer["dim"]
    T = h.shape[0]
    before = state.get("last") if state else None
    d = shifted(h, before) - h
    mixes = {s: h + d * f32(t[p + "mu." + s]) for s in "rkvgw"}
    r = (mixes["r"] @ f32(t[p + "r"]).T).view(T, H, N)
    k = (mixes["k"] @ f32(t[p + "k"]).T).view(T, H, N)
    v = (mixes["v"] @ f32(t[p + "v"]).T).view(T, H, N)
    gate = F.silu(mixes["g"] @ f32(t[p + "g"]).T)
    w = decay(mixes["w"], f32(t[p + "w1"]), f32(t[p + "w2"]), f32(t[p + "w0"])).view(T, H, N)
    S = state["S"] if state and "S" in state else torch.zeros(H, N, N, dtype=PRECISION)
    o = wkv_scan(r, k, v, w, f32(t[p + "u"]).view(H, N), S)
    if state is not None:
        state["S"], state["last"] = S, h[-1].clone()
    o = unit_rms(o, eps).reshape(T, H * N) * f32(t[p + "norm"]) * gate
    return o @ f32(t[p + "o"]).T


# ------------------------------------------------------------------------------------------ attention
def slopes(H: int) -> torch.Tensor:
    """2^(-8 (h + 1) / H) for h = 0 .. H-1."""
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=PRECISION)


def query_temperature(positions: torch.Tensor, coef: float, every: int) -> torch.Tensor:
    """1 + coef ln(floor((p + 1) / every) + 1)."""
    return 1.0 + coef * torch.log((torch.div(positions + 1, every, rounding_mode="floor") + 1).to(PRECISION))


def window_mask(T: int, size: Optional[int]) -> torch.Tensor:
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if size is not None:
        ok = ok & (i - j < size)
    return ok


def attention_mixer(h: torch.Tensor, mixer: Mapping, t: Mapping[str, torch.Tensor], p: str, eps: float,
                    start: int = 0, past: Optional[Dict] = None) -> torch.Tensor:
    """Grouped-query attention over the rows of h [T, W], positions start .. start + T - 1.  `past` (a dict)
    holds the keys and values of the positions before `start` and gets those of these rows appended."""
    H, D = mixer["heads"], mixer["dim"]
    G, Dv = mixer.get("kv_heads") or H, mixer.get("vdim") or D
    T = h.shape[0]
    pos = torch.arange(start, start + T)
    q = unit_rms((h @ f32(t[p + "q"]).T).view(T, H, D), eps) * f32(t[p + "q.norm"])
    k = unit_rms((h @ f32(t[p + "k"]).T).view(T, G, D), eps) * f32(t[p + "k.norm"])
    v = unit_rms((h @ f32(t[p + "v"]).T).view(T, G, Dv), eps)
    qt = mixer.get("q_temp")
    if qt:
        q = q * query_temperature(pos, qt["coef"], qt["every"])[:, None, None]
    if past is not None:
        if "k" in past:
            k, v = torch.cat([past["k"], k]), torch.cat([past["v"], v])
        past["k"], past["v"] = k, v
    L = k.shape[0]                                   # keys 0 .. L-1; the rows are the last T of them
    size = (mixer.get("mask") or {}).get("size")
    i = pos[:, None]
    j = torch.arange(L)[None, :]
    ok = (j <= i) & ((i - j < size) if size is not None else True)
    dist = (i - j).to(PRECISION)
    out = torch.zeros(T, H, Dv, dtype=PRECISION)
    sl = slopes(H)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * mixer["scale"] - sl[head] * dist
        s = s.masked_fill(~ok, float("-inf"))
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, g]
    gate = torch.sigmoid(h @ f32(t[p + "g"]).T)
    return (out.reshape(T, H * Dv) * gate) @ f32(t[p + "o"]).T


# ------------------------------------------------------------------------------------------ feed-forwards
def xielu(z: torch.Tensor, p: float, q: float) -> torch.Tensor:
    """z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2."""
    sp = lambda a: math.log1p(math.exp(a))
    pos = sp(p) * z * z + 0.5 * z
    neg = (0.5 + sp(q)) * (torch.expm1(z) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def dense_ff(h: torch.Tensor, t: Mapping[str, torch.Tensor], p: str) -> torch.Tensor:
    a = f32(t[p + "act"])
    z = h @ f32(t[p + "up"]).T + f32(t[p + "up.b"])
    return xielu(z, float(a[0]), float(a[1])) @ f32(t[p + "down"]).T + f32(t[p + "down.b"])


def router_logits(h: torch.Tensor, t: Mapping[str, torch.Tensor], p: str) -> torch.Tensor:
    return h @ f32(t[p + "router"]).T + f32(t[p + "router.b"])


def choose(z: torch.Tensor, top: int):
    """The `top` largest logits of every row (the lowest index among equals), and the softmax over them alone."""
    order = torch.sort(z, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.softmax(torch.gather(z, 1, order), dim=-1)


def expert(h: torch.Tensor, t: Mapping[str, torch.Tensor], p: str) -> torch.Tensor:
    return (F.silu(h @ f32(t[p + "gate"]).T) * (h @ f32(t[p + "up"]).T)) @ f32(t[p + "down"]).T


def moe_ff(h: torch.Tensor, mlp: Mapping, t: Mapping[str, torch.Tensor], p: str, margins: Optional[List] = None,
           forced: Optional[torch.Tensor] = None, own: Optional[List] = None) -> torch.Tensor:
    """`margins` collects, per row, the gap between the last chosen logit and the first one left out, `own` the
    choice made here.  `forced` [T, top] replaces the choice (the weights are then the softmax over the forced
    experts' logits)."""
    top = mlp["router"]["top"]
    z = router_logits(h, t, p)
    idx, wt = choose(z, top)
    if own is not None:
        own.append(idx.clone())
    if margins is not None:
        s = torch.sort(z, dim=-1, descending=True).values
        margins.append((s[:, top - 1] - s[:, top]) if z.shape[1] > top else torch.full((z.shape[0],), float("inf")))
    if forced is not None:
        idx = forced.to(torch.int64)
        wt = torch.softmax(torch.gather(z, 1, idx), dim=-1)
    out = torch.zeros(h.shape[0], t[p + "e0.down"].shape[0], dtype=PRECISION)
    for row in range(h.shape[0]):
        for c in range(top):
            e = int(idx[row, c])
            out[row] += wt[row, c] * expert(h[row:row + 1], t, f"{p}e{e}.")[0]
    return out


# ------------------------------------------------------------------------------------------ the model
def run_order(cfg: Mapping):
    """(layer, pass number or None, first of its pass) for every layer run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    order = [(i, None, False) for i in range(loop["start"])]
    for rep in range(loop["times"]):
        order += [(i, rep, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None, False) for i in range(loop["stop"], n)]


def forward(cfg: Mapping, t: Mapping[str, torch.Tensor], ids, layers_out: Optional[List] = None, margins=None, forced=None,
            states: Optional[List[Dict]] = None, start: int = 0, own=None) -> torch.Tensor:
    """Logits [T, vocab] of the tokens `ids` at positions start ..; `states` (one dict per layer run, kept by the
    caller) carries a sequence from one call to the next.  `forced`, `margins` and `own` count the routed feed-forwards
    in the order they run (a repeated layer counts each time)."""
    eps, groups = cfg["norm"]["eps"], cfg["norm"].get("groups", 1)
    ids = torch.as_tensor(list(ids), dtype=torch.int64)
    emb = f32(t["embed"])[ids] * (cfg.get("embedding") or {}).get("scale", 1.0)
    x = emb.clone()
    order = run_order(cfg)
    if states is None:
        states = [{} for _ in order]
    moe_at = 0
    for run, (i, rep, first) in enumerate(order):
        if first:
            if rep > 0:
                x = x + emb
            x = x + f32(t["loop.step"])[rep]
        layer, p = cfg["layers"][i], f"l{i}."
        h = group_norm(x, f32(t[p + "norm1"]), eps, groups)
        if layer["type"] == "wkv":
            x = x + wkv_mixer(h, layer["mixer"], t, p + "mix.", eps, states[run])
        else:
            x = x + attention_mixer(h, layer["mixer"], t, p + "mix.", eps, start, states[run])
        mlp = layer.get("mlp")
        if mlp is not None:
            h = group_norm(x, f32(t[p + "norm2"]), eps, groups)
            if mlp["kind"] == "dense":
                x = x + dense_ff(h, t, p + "mlp.")
            else:
                x = x + moe_ff(h, mlp, t, p + "mlp.", margins, None if forced is None else forced[moe_at], own)
                moe_at += 1
        if layers_out is not None:
            layers_out.append(x.clone())
    return group_norm(x, f32(t["final.norm"]), eps, groups) @ f32(t["head"]).T
