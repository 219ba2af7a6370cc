"""Small Retuvik configurations and model folders with random weights for the tests.

Sizes lie away from powers of two and from each other (key width != value width, heads != kv heads, recurrent
heads times channels smaller and larger than the model's width, norm groups of 1, 2, 3 and 5 parts, widths that
are no multiple of 8), windows that do not line up with the pages of 64, repeated stretches that start at layer 0
or later, run once or several times and hold one layer or several, layers without a feed-forward, routers that
choose one expert or all of them.  Weights are drawn here, not by the package's initialiser, so that decays reach
from a few tokens to hundreds, and bonuses, biases, step vectors and activation constants take values that matter.
"""
import json
import os
import tempfile

import numpy as np
import torch

import retuvik_plain as P

P.PRECISION = torch.float64      # the reference of the tests is the plain implementation in double precision


def wkv(dim=10, heads=5, rank=None):
    m = {"dim": dim, "heads": heads}
    if rank:
        m["decay_rank"] = rank
    return m


def attention(dim=20, heads=6, kv_heads=2, vdim=12, window=37, temp=(0.7, 16), scale=None):
    m = {"dim": dim, "heads": heads, "scale": scale or 1.3 * dim ** -0.5}
    if kv_heads:
        m["kv_heads"] = kv_heads
    if vdim:
        m["vdim"] = vdim
    if window:
        m["mask"] = {"size": window}
    if temp:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return m


def dense(ff=100):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=3, ff=40):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def layer(mixer, mlp):
    return {"type": "attention" if "scale" in mixer else "wkv", "mixer": mixer, "mlp": mlp}


def config(layers, loop=None, vocab=211, width=72, eps=1e-5, groups=3, scale=3.5):
    cfg = {"architecture": "Retuvik", "embedding": {"scale": scale}, "layers": layers, "norm": {"eps": eps, "groups": groups},
           "vocab": vocab, "width": width}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


CONFIGS = {
    # both mixers, both feed-forwards and a layer without one; the stretch 1..2 runs twice
    "mixed": lambda: config([layer(wkv(10, 5), dense()), layer(attention(), moe()), layer(wkv(24, 3), moe(5, 2, 24)),
                             layer(attention(dim=16, heads=4, kv_heads=4, vdim=24, window=64, temp=None), None),
                             layer(wkv(12, 4), dense(50))], loop=(1, 3, 2)),
    # widths that are multiples of 16, as served models have; the stretch starts at layer 0 and runs three times
    "even": lambda: config([layer(wkv(32, 4), moe(8, 2, 64)), layer(attention(dim=32, heads=4, kv_heads=2, vdim=32, window=130, temp=(0.25, 32)), dense(128)),
                            layer(wkv(64, 2), dense(256))], loop=(0, 2, 3), vocab=256, width=128, groups=2, scale=1.0),
    # nothing a multiple of 8; one layer repeated four times; a router that takes every expert
    "odd": lambda: config([layer(wkv(9, 3), moe(3, 3, 50)), layer(attention(dim=10, heads=3, kv_heads=3, vdim=6, window=11, temp=(1.5, 7)), dense(50)),
                           layer(wkv(7, 15), None)], loop=(1, 2, 4), vocab=101, width=100, groups=5),
    # what a configuration may leave out or set to one: no repeated stretch, one norm group, no window, no temperature,
    # every query head with its own keys, values as wide as keys, one expert chosen, one recurrent head, scale 1
    "plain": lambda: config([layer(wkv(40, 1), moe(4, 1, 32)), layer(attention(dim=16, heads=4, kv_heads=None, vdim=None, window=None, temp=None, scale=1.0), dense(64)),
                             layer(wkv(16, 2, rank=6), dense(64))], vocab=97, width=64, groups=1, scale=1.0),
    # a stretch that runs once, many query heads on one key head, wide values, heads of more than 128 channels
    "wide": lambda: config([layer(attention(dim=16, heads=20, kv_heads=1, vdim=80, window=70, temp=(0.3, 50)), moe(5, 1, 24)),
                            layer(wkv(136, 1), dense(64)), layer(wkv(96, 2), None)], loop=(0, 3, 1), vocab=97, width=64, groups=4),
    # sizes of a small served model
    "served": lambda: config([layer(wkv(64, 8), dense(1024)), layer(wkv(64, 8), moe(16, 4, 128)),
                              layer(attention(dim=64, heads=8, kv_heads=2, vdim=64, window=128, temp=(0.5, 128), scale=0.125), moe(16, 4, 128)),
                              layer(wkv(64, 8), dense(1024))], loop=(1, 3, 2), vocab=1000, width=512, groups=4, scale=16.0),
    "wkv_only": lambda: config([layer(wkv(), None)]),
    "attention_only": lambda: config([layer(attention(window=9), None)]),
    "dense_only": lambda: config([layer(wkv(8, 2), dense(160))]),
    "experts_only": lambda: config([layer(wkv(8, 2), moe())]),
    "loop_only": lambda: config([layer(wkv(8, 3), None)], loop=(0, 1, 3)),
}

_folders = {}


def make_tensors(cfg: dict, seed: int, sharp: float = 1.0, router_scale: float = 4.0):
    """Random tensors by name (float32 values that bfloat16 holds exactly).  `sharp` scales the query norm weights,
    which makes the softmax peaky: single keys then decide a row.  The decay offsets spread from memories of
    hundreds of tokens to a few; `router_scale` spreads the routers' logits."""
    g = torch.Generator().manual_seed(seed)

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * (s / i ** 0.5)).bfloat16().float()

    def vec(n, mean=1.0, s=0.1):
        return (mean + s * torch.randn(n, generator=g)).bfloat16().float()

    w, t = cfg["width"], {}
    t["embed"] = torch.randn(cfg["vocab"], w, generator=g).bfloat16().float()
    if cfg.get("loop"):
        t["loop.step"] = (0.7 * torch.randn(cfg["loop"]["times"], w, generator=g)).bfloat16().float()
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        t[p + "norm1"] = vec(w)
        if l["type"] == "wkv":
            hn, rank = m["heads"] * m["dim"], m.get("decay_rank") or 5 + i
            for s in "rkvgw":
                t[p + "mix.mu." + s] = torch.rand(w, generator=g).bfloat16().float()
            for s in "kv":
                t[p + "mix." + s] = mat(hn, w, 1.5)
            # r leans towards k and the bonus is positive: the current token's own term r.(u k) then has one sign, so no
            # head's output comes out as a small difference of large terms in the first rows of a sequence, which the
            # head norm would blow up to full size together with bfloat16's rounding
            t[p + "mix.r"] = (t[p + "mix.k"] + mat(hn, w, 0.9)).bfloat16().float()
            t[p + "mix.g"] = mat(hn, w, 2.0)
            t[p + "mix.w1"] = mat(rank, w, 1.5)
            t[p + "mix.w2"] = mat(hn, rank, 1.5)
            t[p + "mix.w0"] = (-6.0 + 7.0 * torch.rand(hn, generator=g)).bfloat16().float()
            t[p + "mix.u"] = (0.2 + 0.8 * torch.rand(m["heads"], m["dim"], generator=g)).bfloat16().float()
            t[p + "mix.norm"] = vec(hn, s=0.3)
            t[p + "mix.o"] = mat(w, hn)
        else:
            H, d = m["heads"], m["dim"]
            G, dv = m.get("kv_heads") or H, m.get("vdim") or d
            t[p + "mix.q"] = mat(H * d, w)
            t[p + "mix.k"] = mat(G * d, w)
            t[p + "mix.v"] = mat(G * dv, w)
            t[p + "mix.g"] = mat(H * dv, w, 2.0)
            t[p + "mix.q.norm"] = vec(d, mean=1.5 * sharp, s=0.3)
            t[p + "mix.k.norm"] = vec(d, mean=1.5, s=0.3)
            t[p + "mix.o"] = mat(w, H * dv, 1.5)
        mlp = l.get("mlp")
        if mlp is None:
            continue
        t[p + "norm2"] = vec(w)
        if mlp["kind"] == "dense":
            t[p + "mlp.up"] = mat(mlp["ff"], w, 1.2)
            t[p + "mlp.up.b"] = vec(mlp["ff"], mean=0.0, s=0.5)
            t[p + "mlp.down"] = mat(w, mlp["ff"], 0.7)
            t[p + "mlp.down.b"] = vec(w, mean=0.0, s=0.5)
            t[p + "mlp.act"] = vec(2, mean=0.0, s=1.0)
        else:
            r = mlp["router"]
            for e in range(r["experts"]):
                t[p + f"mlp.e{e}.gate"] = mat(mlp["expert"]["ff"], w, 1.5)
                t[p + f"mlp.e{e}.up"] = mat(mlp["expert"]["ff"], w, 1.5)
                t[p + f"mlp.e{e}.down"] = mat(w, mlp["expert"]["ff"])
            t[p + "mlp.router"] = mat(r["experts"], w, router_scale)
            t[p + "mlp.router.b"] = (1.0 * torch.randn(r["experts"], generator=g)).bfloat16().float()
    t["final.norm"] = vec(w)
    t["head"] = mat(cfg["vocab"], w)
    return t


def write_folder(cfg, tensors, prefix="x0ne_rtv_"):
    from x0ne_engine_b200.weights import write_file
    d = tempfile.mkdtemp(prefix=prefix)
    write_file(os.path.join(d, "model.safetensors"), {k: v.bfloat16() for k, v in tensors.items()})
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    return d


def folder(name: str, seed: int = 0, sharp: float = 1.0):
    """(folder, config, tensors) of a tiny model written once per (name, seed, sharp)."""
    key = (name, seed, sharp)
    if key not in _folders:
        cfg = CONFIGS[name]()
        tensors = make_tensors(cfg, seed, sharp)
        _folders[key] = (write_folder(cfg, tensors, f"x0ne_rtv_{name}_"), cfg, tensors)
    return _folders[key]


def plain_logits(cfg, tensors, ids, layers_out=None, margins=None, forced=None, own=None):
    return P.forward(cfg, tensors, list(ids), layers_out, margins, forced, own=own).numpy()


def routed_runs(cfg):
    """(layer, how many times it ran before) of every routed feed-forward in the order they run."""
    seen, out = {}, []
    for i, _, _ in P.run_order(cfg):
        mlp = cfg["layers"][i].get("mlp")
        k = seen.get(i, 0)
        seen[i] = k + 1
        if mlp is not None and mlp["kind"] == "moe":
            out.append((i, k))
    return out


class Choices:
    """Records what the routers of an engine choose, per run of a routed layer and (slot, position), while it is
    active.  A bfloat16 run may take another expert than the plain implementation where two logits are within its
    rounding, and from there on the two would differ altogether; the tests give the plain implementation the
    engine's choices (`forced`) and check separately that the choices agree wherever they are clear.  A layer of a
    repeated stretch is called once per pass through the stretch: its calls for one (slot, position) come in that
    order.  (The engine must launch its passes itself, `pass_graphs=False`: a replayed graph calls no Python.)"""

    def __init__(self, eng, cfg):
        self.eng, self.runs = eng, routed_runs(cfg)
        self.layers = sorted({i for i, _ in self.runs})
        self.seen = {i: {} for i in self.layers}

    def __enter__(self):
        for i in self.layers:
            part = self.eng.model.blocks[i].ffn
            assert type(part).__name__ == "RoutedExperts"

            def forward(ctx, x, n_rows, _f=type(part).forward, _p=part, _i=i):
                out = _f(_p, ctx, x, n_rows)
                ch = ctx.ws.buffer("moe.chosen", (ctx.ws.max_rows, _p.top), torch.int32)[:n_rows].cpu()
                slots, pos = ctx.row_slot[:n_rows].cpu().tolist(), ctx.row_pos[:n_rows].cpu().tolist()
                for r, (s, p) in enumerate(zip(slots, pos)):
                    if s >= 0:
                        self.seen[_i].setdefault((s, p), []).append(ch[r].clone())
                return out
            part.forward = forward
        return self

    def __exit__(self, *exc):
        for i in self.layers:
            del self.eng.model.blocks[i].ffn.forward

    def of(self, slot: int, n: int):
        """[run of a routed layer][n, top] for positions 0..n-1 of the sequence that ran in `slot`."""
        return [torch.stack([self.seen[i][(slot, p)][k] for p in range(n)]) for i, k in self.runs]


def agreement(cfg, tensors, ids, forced, clear=0.25):
    """(fraction of (token, routed run) whose engine choice equals the plain choice, the same among those where the
    plain margin is at least `clear`).  The plain run follows the engine's choices, so that every router sees the
    input the engine's router saw."""
    margins, own = [], []
    P.forward(cfg, tensors, list(ids), None, margins, forced, own=own)
    same_all = same_clear = n_clear = n_all = 0
    for m, mine, theirs in zip(margins, own, forced):
        eq = (mine.sort(-1).values == theirs.to(torch.long).sort(-1).values).all(-1)
        ok = m >= clear
        same_all += int(eq.sum()); n_all += eq.numel()
        same_clear += int((eq & ok).sum()); n_clear += int(ok.sum())
    return same_all / max(n_all, 1), (same_clear / n_clear if n_clear else 1.0)


def clear_ids(cfg, tensors, n, seed=0, margin=0.0):
    """n token ids (drawn from `seed`, then seed + 1000, ...) for which no router of the model comes closer than
    `margin` to another choice, by the plain implementation: rounding then cannot flip one."""
    for k in range(200):
        ids = [int(t) for t in np.random.default_rng(seed + 1000 * k).integers(0, cfg["vocab"], n)]
        if margin <= 0:
            return ids
        m = []
        P.forward(cfg, tensors, ids, None, m)
        if not m or min(float(x.min()) for x in m) >= margin:
            return ids
    raise AssertionError("no token sequence with clear routing found")


def plain_greedy(cfg, tensors, prompt, n_new):
    ids, out = list(prompt), []
    for _ in range(n_new):
        t = int(P.forward(cfg, tensors, ids)[-1].argmax())
        out.append(t)
        ids.append(t)
    return out
