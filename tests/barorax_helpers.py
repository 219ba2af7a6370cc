"""Small Barorax configurations and model folders with random weights for the tests.

Sizes lie away from powers of two and from each other (key width != value width, heads != kv heads, rotary widths below
the key width and equal to it, states of 3 to 40 values, 2 to 5 taps, step-size ranks that are no multiple of 8, widths
that are no multiple of 8), chunks that do not line up with the pages of 64, repeated stretches that start at layer 0 or
later, run once or several times and hold one layer or several, layers without a feed-forward, routers with one group,
with groups of one expert and with all groups kept, one expert chosen or all of them, no shared expert.  Weights are drawn
here, not by the package's initialiser, so that the state's memories reach from a few tokens to hundreds, and the numbers
that make lambda, the step vectors and the skip weights take values that matter.
"""
import json
import os
import tempfile

import numpy as np
import torch

import barorax_plain as P

P.PRECISION = torch.float64      # the reference of the tests is the plain implementation in double precision


def mamba(inner=50, state=6, conv=4, dt_rank=5):
    return {"inner": inner, "state": state, "conv": conv, "dt_rank": dt_rank}


def diff_attn(dim=12, heads=4, kv_heads=2, vdim=20, rot=(8, 5000.0), diff=0.3, scale=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim, "diff": diff, "scale": scale or 1.2 * dim ** -0.5}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return m


def chunk_attn(dim=20, heads=6, kv_heads=2, vdim=12, rot=(20, 300.0), chunk=37, scale=None):
    # queries and keys have unit root mean square, so a score reaches dim * scale at most
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim, "scale": scale or 8.0 / dim, "mask": {"size": chunk}}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return m


def moe(experts=6, top=2, ff=24, groups=(3, 2), scale=1.5, shared=40):
    r = {"experts": experts, "top": top, "scale": scale}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r, "shared": {"ff": shared} if shared else None}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(layers, loop=None, vocab=211, width=72, eps=1e-5):
    cfg = {"architecture": "Barorax", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


CONFIGS = {
    # every mixer and a layer without a feed-forward; the stretch 1..2 runs twice
    "mixed": lambda: config([layer("mamba1", mamba(), moe()), layer("attention", diff_attn(), moe(8, 3, 16, (4, 2), 2.5, 24)),
                             layer("attention_2", chunk_attn(), None), layer("mamba1", mamba(36, 10, 3, 7), moe(4, 1, 32, None, 1.0, None))],
                            loop=(1, 3, 2)),
    # the same with chunked attention whose scores reach 40 and 16: single keys decide a row
    "sharp32": lambda: config([layer("mamba1", mamba(), moe()), layer("attention", diff_attn(), moe(8, 3, 16, (4, 2), 2.5, 24)),
                               layer("attention_2", chunk_attn(scale=2.0), None), layer("mamba1", mamba(36, 10, 3, 7), moe(4, 1, 32, None, 1.0, None))],
                              loop=(1, 3, 2)),
    "sharp16": lambda: config([layer("mamba1", mamba(), moe()), layer("attention", diff_attn(), moe(8, 3, 16, (4, 2), 2.5, 24)),
                               layer("attention_2", chunk_attn(scale=0.8), None), layer("mamba1", mamba(36, 10, 3, 7), moe(4, 1, 32, None, 1.0, None))],
                              loop=(1, 3, 2)),
    # widths that are multiples of 16, as served models have; the stretch starts at layer 0 and runs three times
    "even": lambda: config([layer("attention", diff_attn(48, 4, 2, 96, (32, 100000.0), 0.2, 0.15), moe(8, 2, 48, (4, 2), 1.5, 80)),
                            layer("mamba1", mamba(256, 16, 4, 8), moe(8, 2, 48, (4, 2), 1.5, 80)),
                            layer("attention_2", chunk_attn(32, 8, 2, 32, (32, 20000.0), 130, 0.25), moe(8, 4, 32, (2, 2), 1.0, 128))],
                           loop=(0, 2, 3), vocab=256, width=128, eps=1e-6),
    # nothing a multiple of 8; one layer repeated four times; a router that takes every expert; groups of one expert
    "odd": lambda: config([layer("mamba1", mamba(27, 3, 2, 3), moe(3, 3, 50, (3, 3), 0.7, 10)),
                           layer("attention_2", chunk_attn(10, 3, 3, 6, (6, 77.0), 11, 0.9), moe(5, 2, 14, (5, 3), 3.0, None)),
                           layer("attention", diff_attn(9, 3, 1, 7, (4, 19.0), 0.45), None)], loop=(1, 2, 4), vocab=101, width=100),
    # what a configuration may leave out or make equal: no repeated stretch, no rotation, values as wide as keys, every
    # query head with its own keys, one group, one expert chosen, scale 1, state of 40 values (several per thread)
    "plain": lambda: config([layer("attention", diff_attn(16, 2, 2, 16, None, 0.0, 0.25), moe(4, 1, 32, None, 1.0, 32)),
                             layer("mamba1", mamba(64, 40, 5, 16), moe(4, 1, 32, (1, 1), 1.0, 32)),
                             layer("attention_2", chunk_attn(16, 4, 4, 16, None, 64, 0.5), moe(6, 6, 8, (2, 2), 1.0, 8))], vocab=97, width=64),
    # a stretch that runs once, many query heads on one key head, wide values and keys
    "wide": lambda: config([layer("attention_2", chunk_attn(16, 20, 1, 80, (8, 1000.0), 70, 0.6), moe(5, 1, 24, (5, 2), 2.0, 16)),
                            layer("attention", diff_attn(72, 2, 1, 136, (40, 100.0), 0.1), moe()),
                            layer("mamba1", mamba(200, 33, 4, 12), None)], loop=(0, 3, 1), vocab=97, width=64),
    # sizes of a small served model
    "served": lambda: config([layer("mamba1", mamba(1024, 16, 4, 32), moe(16, 4, 128, (4, 2), 2.5, 256)),
                              layer("attention", diff_attn(64, 8, 2, 128, (32, 500000.0), 0.3, 0.125), moe(16, 4, 128, (4, 2), 2.5, 256)),
                              layer("attention_2", chunk_attn(64, 8, 2, 64, (64, 10000.0), 128, 0.125), moe(16, 4, 128, (4, 2), 2.5, 256)),
                              layer("mamba1", mamba(1024, 16, 4, 32), None)], loop=(1, 3, 2), vocab=1000, width=512, eps=1e-6),
    "mamba_only": lambda: config([layer("mamba1", mamba(), None)]),
    "diff_only": lambda: config([layer("attention", diff_attn(), None)]),
    "chunk_only": lambda: config([layer("attention_2", chunk_attn(chunk=9), None)]),
    "experts_only": lambda: config([layer("mamba1", mamba(16, 4, 2, 2), moe())]),
    "loop_only": lambda: config([layer("mamba1", mamba(24, 5, 3, 4), None)], loop=(0, 1, 3)),
}

_folders = {}


def make_tensors(cfg: dict, seed: int, sharp: float = 1.0, router_scale: float = 4.0):
    """Random tensors by name (float32 values that bfloat16 holds exactly).  `sharp` scales the query matrices, which
    makes the softmax peaky: single keys then decide a row.  The decay rates spread from memories of hundreds of tokens
    to a few; `router_scale` spreads the routers' logits."""
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
        if l["type"] == "mamba1":
            I, N, K, R = m["inner"], m["state"], m["conv"], m["dt_rank"]
            t[p + "mix.in"] = mat(2 * I, w, 1.5)
            t[p + "mix.conv"] = (torch.randn(I, K, generator=g) * 0.6).bfloat16().float()
            t[p + "mix.conv.b"] = vec(I, mean=0.0, s=0.3)
            t[p + "mix.x"] = mat(R + 2 * N, I, 1.0)
            t[p + "mix.dt"] = mat(I, R, 1.0)
            t[p + "mix.dt.b"] = (-4.0 + 4.0 * torch.rand(I, generator=g)).bfloat16().float()     # steps of 0.02 to 0.7
            t[p + "mix.A_log"] = (-3.0 + 4.5 * torch.rand(I, N, generator=g)).bfloat16().float()  # rates of 0.05 to 4.5
            t[p + "mix.D"] = vec(I, s=0.5)
            t[p + "mix.o"] = mat(w, I, 0.6 / N ** 0.5)
        else:
            H, d = m["heads"], m["dim"]
            G, dv = m.get("kv_heads") or H, m.get("vdim") or d
            maps = 2 if l["type"] == "attention" else 1
            t[p + "mix.q"] = mat(H * maps * d, w, 1.5 * sharp)
            t[p + "mix.k"] = mat(G * maps * d, w, 1.5)
            t[p + "mix.v"] = mat(G * dv, w)
            t[p + "mix.o"] = mat(w, H * dv, 1.5)
            if maps == 2:
                t[p + "mix.g"] = mat(H * dv, w, 2.0)
                for s in ("lq1", "lk1", "lq2", "lk2"):
                    t[p + "mix." + s] = (0.4 * torch.randn(d, generator=g)).bfloat16().float()
        mlp = l.get("mlp")
        if mlp is None:
            continue
        t[p + "norm2"] = vec(w)
        r = mlp["router"]
        for e in range(r["experts"]):
            t[p + f"mlp.e{e}.gate"] = mat(mlp["expert"]["ff"], w, 1.5)
            t[p + f"mlp.e{e}.up"] = mat(mlp["expert"]["ff"], w, 1.5)
            t[p + f"mlp.e{e}.down"] = mat(w, mlp["expert"]["ff"])
        t[p + "mlp.router"] = mat(r["experts"], w, router_scale)
        if mlp.get("shared"):
            t[p + "mlp.shared.gate"] = mat(mlp["shared"]["ff"], w, 1.5)
            t[p + "mlp.shared.up"] = mat(mlp["shared"]["ff"], w, 1.5)
            t[p + "mlp.shared.down"] = mat(w, mlp["shared"]["ff"])
    t["final.norm"] = vec(w)
    t["head"] = mat(cfg["vocab"], w)
    return t


def write_folder(cfg, tensors, prefix="x0ne_brx_"):
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
        _folders[key] = (write_folder(cfg, tensors, f"x0ne_brx_{name}_"), cfg, tensors)
    return _folders[key]


def routed_runs(cfg):
    """(number of the layer run, layer) of every routed feed-forward in the order they run."""
    return [(run, i) for run, (i, _) in enumerate(P.run_order(cfg)) if cfg["layers"][i].get("mlp") is not None]


class Choices:
    """Records what the routers of an engine choose, per run of a routed layer and (slot, position), while it is active.
    A run may take another expert than the plain implementation where two scores are within its rounding, and from there
    on the two would differ altogether; the tests give the plain implementation the engine's choices and check separately
    that the choices agree nearly everywhere.  A layer of a repeated stretch is called once per pass through the stretch:
    its calls for one (slot, position) come in that order.  (The engine must launch its passes itself,
    `pass_graphs=False`: a replayed graph calls no Python.)"""

    def __init__(self, eng, cfg):
        self.eng, self.runs = eng, routed_runs(cfg)
        self.layers = sorted({i for _, i in self.runs})
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
        """{layer run: [n, top]} for positions 0..n-1 of the sequence that ran in `slot`."""
        count, out = {}, {}
        for run, i in self.runs:
            k = count.get(i, 0)
            count[i] = k + 1
            out[run] = torch.stack([self.seen[i][(slot, p)][k] for p in range(n)]).to(torch.long)
        return out


def plain_logits(cfg, tensors, ids, chosen=None, layers_out=None, record=None):
    return P.forward(cfg, tensors, list(ids), layers_out=layers_out, chosen=chosen, record=record).numpy()


def agreement(cfg, tensors, ids, chosen):
    """The fraction of (token, routed run) at which the plain implementation's router, fed what the engine's choices
    lead to up to there, chooses the same set of experts as the engine did."""
    record = {}
    P.forward(cfg, tensors, list(ids), chosen=chosen, record=record)
    same = total = 0
    for run, theirs in chosen.items():
        own = record[run][0]
        eq = (own.sort(-1).values == theirs.sort(-1).values).all(-1)
        same += int(eq.sum())
        total += eq.numel()
    return same / max(total, 1)


def plain_greedy(cfg, tensors, prompt, n_new):
    ids, out = list(prompt), []
    for _ in range(n_new):
        t = int(P.forward(cfg, tensors, ids)[-1].argmax())
        out.append(t)
        ids.append(t)
    return out


def random_ids(cfg, n, seed=0):
    return [int(t) for t in np.random.default_rng(seed).integers(0, cfg["vocab"], n)]
