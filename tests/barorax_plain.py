"""Barorax restated in plain PyTorch on the CPU, one function per mechanism.

Nothing here is shared with the package: the functions take a config.json as a dict and the checkpoint tensors by
name (any dtype; they are widened to the working precision), run a whole sequence with explicit loops over tokens
(the selective scan, the convolution) or full T x T score matrices (the attentions), and return the logits of every
position.

Notation: T tokens, width W.  Attention: H query heads, G key/value heads, key width D, value width Dv.  Selective
scan: I channels, N state values per channel, K convolution taps, R the rank of the step size's projection.  Routed
feed-forward: E experts in groups, k chosen per token.
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional

import torch

PRECISION = torch.float32      # the tests set float64: the same equations, as a sharper reference


def f32(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to("cpu", PRECISION)


# ------------------------------------------------------------------------------------------ norms
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


# ------------------------------------------------------------------------------------------ rotation
def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, D]: the first `dims` values of every head are pairs (2i, 2i + 1) that turn by the angle
    position * base^(-2i / dims); the other values stay."""
    if dims == 0:
        return x
    i = torch.arange(dims // 2, dtype=PRECISION)
    ang = positions.to(PRECISION)[:, None] * torch.pow(torch.tensor(float(base), dtype=PRECISION), -2.0 * i / dims)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------------ attention
def softmax_attention(q, k, v, scale: float, positions: torch.Tensor, chunk: int = 0, sink_one: bool = False):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] of ONE sequence whose rows lie at `positions` (ascending, all of the
    sequence from its first token).  Query head h reads key/value head h // (H / G).  Query i sees key j when
    pos_j <= pos_i and, with `chunk` = c > 0, floor(pos_i / c) = floor(pos_j / c).  Weights exp(s_j) / (sum exp(s) +
    (1 if sink_one)).  Returns [T, H, Dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    pi, pj = positions[:, None], positions[None, :]
    seen = pj <= pi
    if chunk:
        seen = seen & (torch.div(pi, chunk, rounding_mode="floor") == torch.div(pj, chunk, rounding_mode="floor"))
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // rep
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~seen, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        if sink_one:
            m = torch.clamp(m, min=0.0)
        e = torch.exp(s - m)
        den = e.sum(dim=-1, keepdim=True)
        if sink_one:
            den = den + torch.exp(-m)
        out[:, h] = (e / den) @ v[:, g]
    return out


def diff_lambda(lq1, lk1, lq2, lk2, diff: float) -> float:
    return math.exp(float((f32(lq1) * f32(lk1)).sum())) - math.exp(float((f32(lq2) * f32(lk2)).sum())) + diff


def differential_attention(h, t: Mapping[str, torch.Tensor], p: str, m: Mapping, eps: float, positions):
    """Two softmax maps per head over the same values; the second, times lambda, is taken off the first; each head's
    difference is brought to unit root mean square and multiplied by 1 - diff; a sigmoid gate of the input multiplies
    the concatenated heads before the output product."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = (h @ f32(t[p + ".q"]).T).reshape(T, H, 2, D)
    k = (h @ f32(t[p + ".k"]).T).reshape(T, G, 2, D)
    v = (h @ f32(t[p + ".v"]).T).reshape(T, G, Dv)
    maps = []
    for a in range(2):
        qa = rotate_pairs(q[:, :, a], positions, rot["dims"], rot["base"])
        ka = rotate_pairs(k[:, :, a], positions, rot["dims"], rot["base"])
        maps.append(softmax_attention(qa, ka, v, m["scale"], positions))
    lam = diff_lambda(t[p + ".lq1"], t[p + ".lk1"], t[p + ".lq2"], t[p + ".lk2"], m["diff"])
    o = unit_rms(maps[0] - lam * maps[1], eps) * (1.0 - m["diff"])
    o = o.reshape(T, H * Dv) * torch.sigmoid(h @ f32(t[p + ".g"]).T)
    return o @ f32(t[p + ".o"]).T


def chunked_attention(h, t: Mapping[str, torch.Tensor], p: str, m: Mapping, eps: float, positions):
    """Rotation, then queries and keys brought to unit root mean square per head, a mask of chunks counted from the
    sequence's first position, and a softmax whose denominator holds one more term of score zero."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rotate_pairs((h @ f32(t[p + ".q"]).T).reshape(T, H, D), positions, rot["dims"], rot["base"])
    k = rotate_pairs((h @ f32(t[p + ".k"]).T).reshape(T, G, D), positions, rot["dims"], rot["base"])
    v = (h @ f32(t[p + ".v"]).T).reshape(T, G, Dv)
    o = softmax_attention(unit_rms(q, eps), unit_rms(k, eps), v, m["scale"], positions, chunk=m["mask"]["size"], sink_one=True)
    return o.reshape(T, H * Dv) @ f32(t[p + ".o"]).T


# ------------------------------------------------------------------------------------------ selective scan
def silu(x):
    return x * torch.sigmoid(x)


def causal_conv(x, w, b, before: Optional[torch.Tensor] = None):
    """x [T, I]; w [I, K]; the last column of w meets the current token, the one before it the token before, and so
    on; `before` [K - 1, I] holds the inputs ahead of row 0 (zeros at a sequence's start).  Returns (y [T, I], the last
    K - 1 inputs)."""
    T, I = x.shape
    K = w.shape[1]
    if before is None:
        before = torch.zeros(K - 1, I, dtype=x.dtype)
    ext = torch.cat([before.to(x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for t in range(T):
        y[t] = (ext[t:t + K].T * w).sum(dim=-1) + b
    return y, ext[ext.shape[0] - (K - 1):].clone()


def softplus(x):
    return torch.where(x > 20, x, torch.log1p(torch.exp(torch.clamp(x, max=20.0))))


def selective_scan(x, dt, A, B, C, D, S):
    """x, dt [T, I]; A [I, N]; B, C [T, N]; D [I]; S [I, N] is changed in place.  Token by token:
    S = exp(dt A) S + dt x B;  y = S C + D x."""
    T = x.shape[0]
    y = torch.zeros_like(x)
    for t in range(T):
        S.mul_(torch.exp(dt[t][:, None] * A)).add_((dt[t] * x[t])[:, None] * B[t][None, :])
        y[t] = S @ C[t] + D * x[t]
    return y


def mamba_mixer(h, t: Mapping[str, torch.Tensor], p: str, m: Mapping, state: Optional[dict] = None):
    """state: {"S": [I, N], "conv": [K - 1, I]} carried from call to call (None: a sequence's start, nothing kept)."""
    I, N, R = m["inner"], m["state"], m["dt_rank"]
    xz = h @ f32(t[p + ".in"]).T
    x, z = xz[:, :I], xz[:, I:]
    x, conv_tail = causal_conv(x, f32(t[p + ".conv"]), f32(t[p + ".conv.b"]), None if state is None else state.get("conv"))
    x = silu(x)
    low = x @ f32(t[p + ".x"]).T
    dt = softplus(low[:, :R] @ f32(t[p + ".dt"]).T + f32(t[p + ".dt.b"]))
    A = -torch.exp(f32(t[p + ".A_log"]))
    S = torch.zeros(I, N, dtype=h.dtype) if state is None or "S" not in state else state["S"]
    y = selective_scan(x, dt, A, low[:, R:R + N], low[:, R + N:R + 2 * N], f32(t[p + ".D"]), S)
    if state is not None:
        state["S"], state["conv"] = S, conv_tail
    return (y * silu(z)) @ f32(t[p + ".o"]).T


# ------------------------------------------------------------------------------------------ feed-forward
def gated_expert(h, gate, up, down):
    return (silu(h @ f32(gate).T) * (h @ f32(up).T)) @ f32(down).T


def route(z: torch.Tensor, top: int, groups: int, keep: int, scale: float):
    """z [T, E] router logits.  Scores sigmoid(z); the experts form `groups` equal groups of neighbours, a group is
    worth the sum of its two largest scores, the `keep` best groups stay; of their experts the `top` largest scores
    are chosen.  Weights: the chosen scores over their sum (+ 1e-20), times `scale`.  Returns (chosen [T, top],
    weights [T, top])."""
    T, E = z.shape
    s = torch.sigmoid(z)
    per = E // groups

    def largest(x, k):
        """Indices of the k largest values of each row; of equal values the one with the lower index goes first."""
        return torch.sort(x, dim=-1, descending=True, stable=True).indices[:, :k]

    allowed = torch.ones(T, E, dtype=torch.bool)
    if keep < groups:
        worth = s.reshape(T, groups, per).sort(dim=-1, descending=True).values[:, :, :2].sum(dim=-1)
        gmask = torch.zeros(T, groups, dtype=torch.bool)
        gmask.scatter_(1, largest(worth, keep), True)
        allowed = gmask[:, :, None].expand(T, groups, per).reshape(T, E)
    chosen = largest(s.masked_fill(~allowed, float("-inf")), top)
    w = s.gather(1, chosen)
    return chosen, w / (w.sum(dim=-1, keepdim=True) + 1e-20) * scale


def routed_ffn(h, t: Mapping[str, torch.Tensor], p: str, mlp: Mapping, chosen=None, record=None):
    """`chosen` [T, top]: the experts to take instead of the router's own choice (the weights are still worked out
    from this function's scores); `record`: a list that receives the router's own choice."""
    r = mlp["router"]
    groups = (r.get("groups") or {}).get("count", 1)
    keep = (r.get("groups") or {}).get("keep", groups)
    z = h @ f32(t[p + ".router"]).T
    scale = float(r["scale"]) if r.get("scale") is not None else 1.0
    own, w = route(z, r["top"], groups, keep, scale)
    if record is not None:
        record.append(own.clone())
    if chosen is not None:
        s = torch.sigmoid(z).gather(1, chosen)
        own, w = chosen, s / (s.sum(dim=-1, keepdim=True) + 1e-20) * scale
    out = torch.zeros_like(h)
    for e in range(r["experts"]):
        rows, col = (own == e).nonzero(as_tuple=True)
        if rows.numel():
            y = gated_expert(h[rows], t[f"{p}.e{e}.gate"], t[f"{p}.e{e}.up"], t[f"{p}.e{e}.down"])
            out.index_add_(0, rows, y * w[rows, col][:, None])
    if mlp.get("shared") is not None:
        out = out + gated_expert(h, t[p + ".shared.gate"], t[p + ".shared.up"], t[p + ".shared.down"])
    return out


# ------------------------------------------------------------------------------------------ the model
def run_order(cfg: Mapping) -> List[tuple]:
    """(layer, number of the pass it opens or None) for every layer run."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(lp["start"])]
    for t in range(lp["times"]):
        order += [(i, t if i == lp["start"] else None) for i in range(lp["start"], lp["stop"])]
    return order + [(i, None) for i in range(lp["stop"], n)]


def forward(cfg: Mapping, t: Mapping[str, torch.Tensor], tokens, layers_out: Optional[list] = None, states: Optional[dict] = None,
            pos0: int = 0, kv: Optional[dict] = None, chosen: Optional[Dict[int, torch.Tensor]] = None, record: Optional[dict] = None):
    """Logits [T, vocab] of one sequence's `tokens` at positions pos0 ..; `layers_out` receives the residual stream
    after every layer run.  `states` (recurrent layers) and `kv` (attention layers: the mixer inputs of all earlier
    rows, kept per run) carry a sequence over several calls; None: the call holds the whole sequence."""
    eps = cfg["norm"]["eps"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = f32(t["embed"])[ids]
    T = x.shape[0]
    for run, (i, opens) in enumerate(run_order(cfg)):
        L, p = cfg["layers"][i], f"l{i}"
        if opens is not None:
            x = x + f32(t["loop.step"])[opens]
        h = rms_norm(x, f32(t[p + ".norm1"]), eps)
        if L["type"] == "mamba1":
            st = None if states is None else states.setdefault(run, {})
            x = x + mamba_mixer(h, t, p + ".mix", L["mixer"], st)
        else:
            # attention over everything the sequence has brought so far: earlier inputs are kept as they were
            if kv is not None:
                h_all = torch.cat([kv[run], h], dim=0) if run in kv else h
                kv[run] = h_all
            else:
                h_all = h
            positions = torch.arange(pos0 + T - h_all.shape[0], pos0 + T)
            fn = differential_attention if L["type"] == "attention" else chunked_attention
            x = x + fn(h_all, t, p + ".mix", L["mixer"], eps, positions)[h_all.shape[0] - T:]
        if L.get("mlp") is not None:
            h = rms_norm(x, f32(t[p + ".norm2"]), eps)
            x = x + routed_ffn(h, t, p + ".mlp", L["mlp"], None if chosen is None else chosen.get(run),
                               None if record is None else record.setdefault(run, []))
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, f32(t["final.norm"]), eps) @ f32(t["head"]).T
