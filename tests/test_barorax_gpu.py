"""Barorax on the GPU against the plain implementation (tests/barorax_plain.py), in float32 and bfloat16: every
mechanism alone, whole prompts, token-by-token decoding, portions down to two tokens, unequal batches with slots, pages
and states used again, the chunk's edge in prompts and in decoding, far keys and a far token in the recurrent state, the
first tokens, long decoding, odd sizes and values a configuration may leave out or make equal, and greedy generation
through the entry point.  The plain implementation follows the routers' choices of the run it is compared with (a choice
that flips within rounding changes a row altogether), and the choices must agree with its own nearly everywhere."""
import numpy as np
import pytest
import torch

import barorax_helpers as H
import barorax_plain as P
from helpers import BF16_KL_TOL, BF16_LOGIT_TOL, assert_close_f32, first_difference, kl_rows

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
DEV = "cuda:0"
_engines = {}


def engine(name, dtype, seed=0, sharp=1.0, max_tokens=2048, **kw):
    from x0ne_engine_b200 import Engine
    kw.setdefault("pass_graphs", False)          # the routers' choices are recorded by Python hooks (H.Choices)
    key = (name, dtype, seed, sharp, max_tokens, tuple(sorted(kw.items())))
    if key not in _engines:
        folder, cfg, tensors = H.folder(name, seed, sharp)
        _engines[key] = (Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, max_seq_len=max_tokens, **kw), cfg, tensors)
    return _engines[key]


def close_bf16(got, want, what):
    """Rows within the bfloat16 tolerance of the other tests; of many rows, one in fifty (or one) may reach twice that:
    a differential head is a small difference of two maps brought back to unit size, which amplifies the rounding of
    what went in."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape and np.isfinite(got).all(), what
    err = np.max(np.abs(got - want), axis=-1) / (np.max(np.abs(want), axis=-1) + 1e-30)
    over = int((err > BF16_LOGIT_TOL).sum())
    assert err.max() <= 2 * BF16_LOGIT_TOL and over <= max(1, len(err) // 50), \
        f"{what}: worst logit error {err.max():.3e}, {over} of {len(err)} rows over {BF16_LOGIT_TOL}"
    kl = kl_rows(want, got)
    assert kl.max() <= 2 * BF16_KL_TOL and int((kl > BF16_KL_TOL).sum()) <= max(1, len(err) // 50), f"{what}: worst KL {kl.max():.3e}"


class Run:
    """Logits of one sequence and what its routers chose."""

    def __init__(self, logits, chosen):
        self.logits, self.chosen = logits, chosen


def check(dtype, cfg, t, ids, run, what, rows=None):
    rows = slice(None) if rows is None else rows
    want = H.plain_logits(cfg, t, ids, run.chosen)[rows]
    if dtype == "float32":
        assert_close_f32(run.logits[rows], want, what)
    else:
        close_bf16(run.logits[rows], want, what)
    if run.chosen:
        agree = H.agreement(cfg, t, ids, run.chosen)
        assert agree >= (0.995 if dtype == "float32" else 0.9), f"{what}: the routers agree on {agree:.3f} of all rows"


def same_cut(dtype, cfg, t, ids, run, base, what):
    """Two runs of one sequence cut differently: the same bits in float32; in bfloat16 each is held against the plain
    implementation (a router may choose differently in the two)."""
    if dtype == "float32":
        got, want = np.asarray(run.logits), np.asarray(base.logits)
        assert np.array_equal(got, want), f"{what}: first difference at {first_difference(got, want)}"
    else:
        check(dtype, cfg, t, ids, run, what)


def in_pieces(eng, cfg, ids, cuts):
    """The prompt cut at `cuts` (piece sizes, the last piece takes the rest): logits of all places, and the choices."""
    with H.Choices(eng, cfg) as rec:
        s = eng.new_sequence()
        out, at = [], 0
        try:
            for c in list(cuts) + [len(ids)]:
                piece = ids[at:at + c]
                if not piece:
                    break
                out.append(eng.step([s], [piece], [list(range(len(piece)))]).cpu().numpy())
                at += len(piece)
            chosen = rec.of(s, len(ids))
        finally:
            eng.free_sequence(s)
    return Run(np.concatenate(out), chosen)


def whole(eng, cfg, ids):
    return in_pieces(eng, cfg, ids, [])


i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)      # noqa: E731


# ------------------------------------------------------------------------------------------ the scan mixer's kernels
def scan_inputs(g, rows, inner, n, taps, dtype):
    xz = torch.randn(rows, 2 * inner, generator=g).to(dtype).to(DEV)
    w = (0.6 * torch.randn(inner, taps, generator=g)).to(DEV)
    b = (0.3 * torch.randn(inner, generator=g)).to(DEV)
    dt_raw = (-2.0 + 1.5 * torch.randn(rows, inner, generator=g)).to(DEV)
    dt_bias = (0.5 * torch.randn(inner, generator=g)).to(DEV)
    A = (-torch.exp(-3.0 + 4.5 * torch.rand(inner, n, generator=g))).to(DEV)
    bc = torch.randn(rows, 2 * n + 3, generator=g).to(DEV)          # B at column 3, C behind it
    D = (1 + 0.5 * torch.randn(inner, generator=g)).to(DEV)
    return xz, w, b, dt_raw, dt_bias, A, bc, D


def plain_mixer_rows(xz, w, b, dt_raw, dt_bias, A, bc, D, idx, n, inner, dtype, state=None):
    """The convolution (its output rounded to the activation type, as the kernel hands it on) and the scan of one
    sequence's rows in double precision."""
    d = lambda x: x.double().cpu()      # noqa: E731
    u, tail = P.causal_conv(d(xz[idx, :inner]), d(w), d(b), None if state is None else state["conv"])
    u = P.silu(u).to(dtype).double()
    S = torch.zeros(inner, n, dtype=torch.float64) if state is None else state["S"]
    y = P.selective_scan(u, P.softplus(d(dt_raw[idx]) + d(dt_bias)), d(A), d(bc[idx, 3:3 + n]), d(bc[idx, 3 + n:3 + 2 * n]), d(D), S)
    return u, y * P.silu(d(xz[idx, inner:])), {"S": S, "conv": tail}


def run_mixer(ops, xz, w, b, dt_raw, dt_bias, A, bc, D, state, rows, slots_of_rows, pos_of_rows, first, seq_slot, n_seqs, inner, n, taps):
    u = torch.zeros((rows.stop - rows.start, inner), dtype=xz.dtype, device=DEV)
    y = torch.zeros_like(u)
    sub = lambda x: x[rows].contiguous()        # noqa: E731
    ops.causal_conv_silu(sub(xz), w, b, state, inner * n, u, i32(slots_of_rows), i32(pos_of_rows), u.shape[0], inner)
    ops.selective_scan(u, sub(xz), inner, sub(dt_raw), dt_bias, A, sub(bc), 3, 3 + n, D, y, state, inner * n, taps, i32(first), i32(seq_slot), n_seqs)
    return u, y


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inner,n,taps", [(50, 6, 4), (33, 3, 2), (64, 16, 4), (40, 24, 1), (96, 40, 5), (20, 70, 3), (7, 1, 3)])
def test_convolution_and_scan_over_unequal_sequences_and_again_from_the_state(dtype, inner, n, taps):
    """Three sequences of 1, 37 and 20 rows in one launch, then 5, 1 and 2 more rows of each from the state the first
    launch left (fewer rows than taps: the kept inputs move up), in slots that are not in order, with a padding sequence
    at the end; against the plain functions over each sequence's rows; a slot that no sequence names stays as it was."""
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(100 * n + taps)
    lens1, lens2, slots = [1, 37, 20], [5, 1, 2], [3, 0, 2]
    rows = sum(lens1) + sum(lens2)
    xz, w, b, dt_raw, dt_bias, A, bc, D = scan_inputs(g, rows, inner, n, taps, dtype)
    stride = inner * (n + taps - 1)
    state = torch.zeros((5, stride), device=DEV)
    state[1] = 7.0
    a, bb = slice(0, 58), slice(58, rows)
    row_slots1 = sum(([s] * k for s, k in zip(slots, lens1)), [])
    row_pos1 = sum((list(range(k)) for k in lens1), [])
    u1, y1 = run_mixer(ops, xz, w, b, dt_raw, dt_bias, A, bc, D, state, a, row_slots1, row_pos1, [0, 1, 38, 58, 58], slots + [-1], 4, inner, n, taps)
    row_slots2 = sum(([s] * k for s, k in zip(slots, lens2)), [])
    row_pos2 = sum((list(range(l1, l1 + k)) for l1, k in zip(lens1, lens2)), [])
    u2, y2 = run_mixer(ops, xz, w, b, dt_raw, dt_bias, A, bc, D, state, bb, row_slots2, row_pos2, [0, 5, 6, 8, 8], slots + [-1], 4, inner, n, taps)
    y = torch.cat([y1, y2])
    tol = 2e-5 if dtype == torch.float32 else 2 ** -7
    at1, at2 = 0, 58
    for s, (n1, n2) in enumerate(zip(lens1, lens2)):
        idx = list(range(at1, at1 + n1)) + list(range(at2, at2 + n2))
        u_want, want, st = plain_mixer_rows(xz, w, b, dt_raw, dt_bias, A, bc, D, idx, n, inner, dtype)
        got = y[idx].double().cpu()
        assert (got - want).abs().max() <= tol * want.abs().max(), f"sequence {s}"
        assert (state[slots[s], :inner * n].double().cpu().view(inner, n) - st["S"]).abs().max() <= 2e-5 * st["S"].abs().max()
        if taps > 1:
            assert torch.equal(state[slots[s], inner * n:].view(taps - 1, inner).double().cpu(), st["conv"])
        # all of the sequence's rows in one launch: the same bits
        state2 = torch.zeros_like(state)
        pick = lambda x: x[idx].contiguous()        # noqa: E731
        u3 = torch.zeros((len(idx), inner), dtype=dtype, device=DEV)
        y3 = torch.zeros_like(u3)
        ops.causal_conv_silu(pick(xz), w, b, state2, inner * n, u3, i32([4] * len(idx)), i32(list(range(len(idx)))), len(idx), inner)
        ops.selective_scan(u3, pick(xz), inner, pick(dt_raw), dt_bias, A, pick(bc), 3, 3 + n, D, y3, state2, inner * n, taps,
                           i32([0, len(idx)]), i32([4]), 1)
        assert torch.equal(y3, y[idx]) and torch.equal(state2[4], state[slots[s]])
        at1, at2 = at1 + n1, at2 + n2
    assert float((state[1] - 7.0).abs().max()) == 0.0 and float(state[4].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inner,n,taps", [(50, 6, 4), (64, 16, 4), (33, 40, 2)])
def test_one_token_steps_give_the_bits_of_the_scan_over_all_rows(dtype, inner, n, taps):
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(11 + n)
    T, B = 21, 3
    xz, w, b, dt_raw, dt_bias, A, bc, D = scan_inputs(g, B * T, inner, n, taps, dtype)
    state = torch.zeros((4, inner * (n + taps - 1)), device=DEV)
    state2 = state.clone()
    _, y = run_mixer(ops, xz, w, b, dt_raw, dt_bias, A, bc, D, state, slice(0, B * T), sum(([s] * T for s in (2, 0, 1)), []),
                     list(range(T)) * B, [0, T, 2 * T, 3 * T], [2, 0, 1], B, inner, n, taps)
    y2 = torch.zeros_like(y)
    for t in range(T):
        rows = [t, T + t, 2 * T + t]
        pick = lambda x: x[rows].contiguous()               # noqa: E731
        u = torch.zeros((B, inner), dtype=dtype, device=DEV)
        yt = torch.zeros_like(u)
        ops.causal_conv_silu(pick(xz), w, b, state2, inner * n, u, i32([0, 1, 2]), i32([t] * 3), B, inner)
        ops.selective_scan(u, pick(xz), inner, pick(dt_raw), dt_bias, A, pick(bc), 3, 3 + n, D, yt, state2, inner * n, taps,
                           i32([0, 1, 1, 2, 3]), i32([0, -1, 1, 2]), 4, one_token=True)
        y2[rows] = yt
    assert torch.equal(y2, y)
    assert torch.equal(state2[0], state[2]) and torch.equal(state2[1], state[0]) and torch.equal(state2[2], state[1])


def test_scan_keeps_a_token_hundreds_of_rows_back():
    """One state value of channel 5 hardly decays and only the first token writes to it; the last row reads that state
    value alone.  Its output is the first token's input (times the decays), so a state that is lost, reset or mixed with
    another slot's shows."""
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(8)
    inner, n, taps, rows, c, n0 = 24, 6, 1, 601, 5, 2
    xz, w, b, dt_raw, dt_bias, A, bc, D = scan_inputs(g, rows, inner, n, taps, torch.float32)
    A[c, n0] = -1e-3
    bc[1:, 3 + n0] = 0.0
    bc[0, 3 + n0] = 2.0
    bc[-1, 3 + n:] = 0.0
    bc[-1, 3 + n + n0] = 1.0
    D[c] = 0.0
    xz[-1, inner + c] = 30.0             # silu(z) = z
    for cuts in ([rows], [1, 300, 299, 1]):
        state = torch.zeros((2, inner * n), device=DEV)
        at, ys = 0, []
        for k in cuts:
            _, y = run_mixer(ops, xz, w, b, dt_raw, dt_bias, A, bc, D, state, slice(at, at + k), [1] * k, list(range(at, at + k)), [0, k], [1], 1,
                             inner, n, taps)
            ys.append(y)
            at += k
        y = torch.cat(ys)
        dt = P.softplus(dt_raw[:, c].double().cpu() + float(dt_bias[c]))
        u0 = float(P.silu(xz[0, c].double().cpu() * float(w[c, 0]) + float(b[c])))
        want = 30.0 * float(dt[0]) * u0 * 2.0 * float(torch.exp(-1e-3 * dt[1:].sum()))
        assert abs(float(y[-1, c]) - want) <= 600 * 2.0 ** -23 * abs(want), cuts
        _, full, _ = plain_mixer_rows(xz, w, b, dt_raw, dt_bias, A, bc, D, list(range(rows)), n, inner, torch.float32)
        assert (y.double().cpu() - full).abs().max() <= 600 * 2.0 ** -23 * full.abs().max()


# ------------------------------------------------------------------------------------------ row-wise kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,vd", [(4, 20), (3, 7), (2, 64), (1, 136)])
def test_differential_heads(dtype, heads, vd):
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(9)
    rows, eps, lam, post = 9, 1e-5, 0.83, 0.7
    maps = torch.randn(rows, heads, 2, vd, generator=g).to(DEV)
    maps[:, 0] *= 50.0                                      # one head far larger: a norm over the whole row would show
    maps[3] = 0.0                                           # eps alone under the root
    wide = (2 * torch.randn(rows, heads * vd + 5, generator=g)).to(dtype).to(DEV)         # the gate lies inside wider rows
    out = torch.empty((rows, heads * vd), dtype=dtype, device=DEV)
    ops.diff_heads(maps.view(rows, -1), wide[:, 5:], wide.shape[1], out, rows, heads, vd, lam, eps, post)
    m = maps.double().cpu()
    want = (P.unit_rms(m[:, :, 0] - lam * m[:, :, 1], eps) * post).reshape(rows, -1) * torch.sigmoid(wide[:, 5:].double().cpu())
    tol = 3e-6 if dtype == torch.float32 else 2 ** -8
    assert (out.double().cpu() - want).abs().max() <= tol * want.abs().max()
    ops.diff_heads(maps.view(rows, -1), None, 0, out, rows, heads, vd, lam, eps, post)
    want = (P.unit_rms(m[:, :, 0] - lam * m[:, :, 1], eps) * post).reshape(rows, -1)
    assert (out.double().cpu() - want).abs().max() <= tol * want.abs().max()


@pytest.mark.parametrize("n,groups,keep,top", [(16, 2, 1, 2), (9, 3, 1, 2), (9, 3, 2, 3), (8, 8, 3, 2), (6, 1, 1, 6), (12, 4, 4, 5), (40, 5, 2, 7), (5, 5, 5, 1)])
def test_router_with_sigmoid_scores_and_groups_worth_their_two_largest(n, groups, keep, top):
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(n + top)
    rows = 300
    z = (2.0 * torch.randn(rows, n + 2, generator=g))
    z[5:9] = z[5:9].round()                      # equal scores: the lower index goes first
    chosen = torch.zeros((rows, top), dtype=torch.int32, device=DEV)
    weights = torch.zeros((rows, top), dtype=torch.float32, device=DEV)
    ops.moe_route(z.to(DEV), None, n, groups, keep, top, rows, chosen, weights, None, 0, sigmoid=True, group_top=2, normalize=True,
                  weight_scale=2.5)
    want_c, want_w = P.route(z[:, :n].double(), top, groups, keep, 2.5)
    # rows in which float32 cannot tell two scores apart that double precision can are left out (none of the integer rows)
    s = torch.sigmoid(z[:, :n].double())
    gap = (s[:, :, None] - s[:, None, :]).abs() + torch.eye(n, dtype=torch.float64)[None] * 9
    clear = (gap.flatten(1).min(-1).values > 1e-6) | (torch.arange(rows) < 9) & (torch.arange(rows) >= 5)
    got_c = chosen.cpu().long()
    assert torch.equal(got_c.sort(-1).values[clear], want_c.sort(-1).values[clear])
    order = got_c.argsort(-1), want_c.argsort(-1)
    got_w, ww = weights.cpu().double().gather(1, order[0]), want_w.gather(1, order[1])
    assert (got_w - ww)[clear].abs().max() <= 1e-6 * 2.5
    assert (weights.cpu().double().sum(-1) - 2.5).abs().max() <= 1e-5


# ------------------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths", [("mamba_only", [1, 2, 40]), ("diff_only", [1, 2, 40, 130]), ("chunk_only", [1, 2, 9, 10, 40]),
                                          ("experts_only", [1, 3, 70]), ("loop_only", [1, 30]), ("mixed", [1, 2, 37, 38, 65, 150]),
                                          ("even", [64, 131, 300]), ("wide", [5, 71, 141]), ("odd", [1, 12, 90]), ("plain", [1, 100]),
                                          ("served", [7, 300])])
def test_each_request_alone_and_whole(name, lengths, dtype):
    eng, cfg, t = engine(name, dtype)
    for k, n in enumerate(lengths):
        ids = H.random_ids(cfg, n, seed=k)
        check(dtype, cfg, t, ids, whole(eng, cfg, ids), f"{name} len {n}")


def test_residual_stream_after_every_layer_run():
    """The float32 residual after each run of a layer (the pending delta added by hand) against the plain one: a repeated
    layer counts each time, and what opens the next pass is not yet in it."""
    eng, cfg, t = engine("mixed", "float32")
    ids = H.random_ids(cfg, 90, seed=3)
    seen = []
    for b in eng.model.blocks:
        def wrapped(ctx, entry, resid, delta, cache_entry=None, write_cache=True, _f=b.forward):
            out = _f(ctx, entry, resid, delta, cache_entry=cache_entry, write_cache=write_cache)
            seen.append((resid[:ctx.n_rows].double() + out[:ctx.n_rows].double()).cpu())
            return out
        b.forward = wrapped
    try:
        run = whole(eng, cfg, ids)
    finally:
        for b in eng.model.blocks:
            del b.forward
    want = []
    H.plain_logits(cfg, t, ids, run.chosen, layers_out=want)
    assert len(seen) == len(want) == 6
    for i, (a, b) in enumerate(zip(seen, want)):
        assert (a - b.double()).abs().max() <= 1e-4 * b.abs().max(), f"layer run {i}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,n,tail", [("mixed", 120, 60), ("wide", 100, 40), ("even", 160, 40), ("odd", 70, 30), ("plain", 90, 50),
                                         ("served", 330, 140)])
def test_prefill_against_token_by_token(name, n, tail, dtype):
    eng, cfg, t = engine(name, dtype)
    ids = H.random_ids(cfg, n, seed=5)
    base = whole(eng, cfg, ids)
    got = in_pieces(eng, cfg, ids, [n - tail] + [1] * tail)
    same_cut(dtype, cfg, t, ids, got, base, f"{name}: last {tail} one by one")
    check(dtype, cfg, t, ids, got, f"{name} decoded")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "even"])
def test_prompt_in_portions_down_to_two_tokens(name, dtype):
    eng, cfg, t = engine(name, dtype)
    ids = H.random_ids(cfg, 170, seed=6)
    base = whole(eng, cfg, ids)
    for cuts in ([2] * 30, [64, 64], [63, 2, 1, 64], [37, 37, 37, 37], [3, 125, 2], [129]):
        same_cut(dtype, cfg, t, ids, in_pieces(eng, cfg, ids, cuts), base, f"{name} cut {cuts[:4]}")
    check(dtype, cfg, t, ids, base, name)


def test_a_step_cut_into_passes_inside_prompts():
    eng, cfg, t = engine("mixed", "float32", max_step_tokens=64)
    ids = H.random_ids(cfg, 150, seed=7)
    assert np.array_equal(whole(eng, cfg, ids).logits, whole(engine("mixed", "float32")[0], cfg, ids).logits)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_unequal_batches_against_each_alone_with_slots_used_again(name, dtype):
    eng, cfg, t = engine(name, dtype)
    for round_ in range(3):                      # the second and third rounds get slots, pages and states that were used
        lengths, steps = [[1, 30, 77, 140], [66, 2, 129], [140, 5]][round_], [3, 9, 1, 6]
        full = [H.random_ids(cfg, n + steps[k], seed=10 * round_ + k) for k, n in enumerate(lengths)]
        prompts = [f[:n] for f, n in zip(full, lengths)]
        tails = [f[n:] for f, n in zip(full, lengths)]
        with H.Choices(eng, cfg) as rec:
            slots = [eng.new_sequence() for _ in lengths]
            got = [[] for _ in lengths]
            first = eng.step(slots, prompts, [list(range(n)) for n in lengths]).cpu().numpy()
            at = 0
            for k, n in enumerate(lengths):
                got[k].append(first[at:at + n])
                at += n
            live = list(range(len(lengths)))
            for step in range(max(steps)):
                live = [k for k in live if step < steps[k]]         # the shorter requests end earlier
                out = eng.step([slots[k] for k in live], [[tails[k][step]] for k in live]).cpu().numpy()
                for j, k in enumerate(live):
                    got[k].append(out[j:j + 1])
            runs = [Run(np.concatenate(got[k]), rec.of(slots[k], len(full[k]))) for k in range(len(lengths))]
            for s in slots:
                eng.free_sequence(s)
        for k, n in enumerate(lengths):
            alone = whole(eng, cfg, full[k])
            same_cut(dtype, cfg, t, full[k], runs[k], alone, f"{name} round {round_} request {k}")
            if round_ == 0:
                check(dtype, cfg, t, full[k], alone, f"{name} request {k}")


# ------------------------------------------------------------------------------------------ edges, far keys
@pytest.mark.parametrize("dtype", DTYPES)
def test_chunk_edges_that_decide(dtype):
    """Sharp queries make single keys decide a row, so a chunk whose edge is one off, a sink that is left out, or a page
    read wrongly changes the logits by far more than the tolerance.  Chunks of 37 positions against pages of 64; every
    position of a 260-token sequence is checked, in a prompt and decoded alone."""
    eng, cfg, t = engine("sharp32" if dtype == "float32" else "sharp16", dtype, seed=3)
    ids = H.random_ids(cfg, 260, seed=8)
    run = whole(eng, cfg, ids)
    want = H.plain_logits(cfg, t, ids, run.chosen)

    def moved(change):
        layers = [dict(l, mixer=change(dict(l["mixer"]))) if l["type"] == "attention_2" else l for l in cfg["layers"]]
        diff = np.abs(H.plain_logits({**cfg, "layers": layers}, t, ids, run.chosen) - want).max(-1) / np.abs(want).max(-1)
        return (diff > 0.1).sum()
    # the test sees what it is for: a chunk that is one position longer or shorter changes the plain result
    assert moved(lambda m: {**m, "mask": {"size": m["mask"]["size"] + 1}}) > 8
    assert moved(lambda m: {**m, "mask": {"size": m["mask"]["size"] - 1}}) > 8
    real = P.softmax_attention
    try:
        P.softmax_attention = lambda *a, **k: real(*a, **{**k, "sink_one": False})
        no_sink = H.plain_logits(cfg, t, ids, run.chosen)
    finally:
        P.softmax_attention = real
    assert ((np.abs(no_sink - want).max(-1) / np.abs(want).max(-1)) > 0.1).sum() > 8
    check(dtype, cfg, t, ids, run, "prompt")
    check(dtype, cfg, t, ids, in_pieces(eng, cfg, ids, [30] + [1] * 230), "decoded across chunk edges and page borders")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_key_far_back_in_both_maps(dtype):
    """A differential layer over 700 positions: the first token's key is made to dominate the last token's query in
    map 2 of head 3 alone (one embedding feature that only the first token has feeds one key channel of that map, another
    that only the last token has feeds the same query channel), so the last logits hang on a key eleven pages back in one
    map and on nearer keys in the other, read in a prompt and in decoding.  Swapping the maps, or cutting the far key
    off, changes the plain result by more than the tolerance."""
    from x0ne_engine_b200 import Engine
    cfg = H.config([H.layer("attention", H.diff_attn(heads=4, kv_heads=2, rot=(4, 50.0)), None), H.layer("mamba1", H.mamba(), H.moe()),
                    H.layer("attention_2", H.chunk_attn(chunk=45), None)])
    t = H.make_tensors(cfg, seed=4)
    special, late, d = 7, 11, cfg["layers"][0]["mixer"]["dim"]
    t["embed"][:, :2] = 0.0
    t["embed"][special, 0] = 8.0
    t["embed"][late, 1] = 8.0
    kr, qr = (1 * 2 + 1) * d + d - 1, (3 * 2 + 1) * d + d - 1     # kv head 1 / query head 3, map 2, the last channel (not rotated)
    t["l0.mix.k"][kr] = 0.0
    t["l0.mix.k"][kr, 0] = 4.0
    t["l0.mix.q"][qr] = 0.0
    t["l0.mix.q"][qr, 1] = 4.0
    t["l0.mix.o"] *= 3.0
    t = {k: v.bfloat16().float() for k, v in t.items()}
    folder = H.write_folder(cfg, t, "x0ne_brx_far_")
    ids = [12 + x % (cfg["vocab"] - 12) for x in H.random_ids(cfg, 700, 9)]
    ids[0], ids[-1] = special, late
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_seq_len=1024, pass_graphs=False)
    run = whole(eng, cfg, ids)
    want = H.plain_logits(cfg, t, ids, run.chosen)[-1]
    cut = H.plain_logits(cfg, t, [13] + ids[1:], run.chosen)[-1]            # another first token: the far key is gone
    assert np.abs(cut - want).max() > 0.07 * np.abs(want).max()
    swapped = dict(t)
    for name, heads in (("l0.mix.q", 4), ("l0.mix.k", 2)):
        swapped[name] = t[name].view(heads, 2, d, -1).flip(1).reshape(t[name].shape)
    assert np.abs(H.plain_logits(cfg, swapped, ids, run.chosen)[-1] - want).max() > 0.07 * np.abs(want).max()
    check(dtype, cfg, t, ids, run, "far key in a prompt", rows=slice(-3, None))
    check(dtype, cfg, t, ids, in_pieces(eng, cfg, ids, [697, 1, 1]), "far key decoded", rows=slice(-3, None))


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_of_a_sequence(dtype):
    eng, cfg, t = engine("mixed", dtype)
    ids = H.random_ids(cfg, 6, seed=11)
    check(dtype, cfg, t, ids, in_pieces(eng, cfg, ids, [1, 1, 1, 1, 1]), "first tokens one by one")
    check(dtype, cfg, t, ids, in_pieces(eng, cfg, ids, [2, 2]), "first tokens in twos")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype):
    eng, cfg, t = engine("even", dtype)
    ids = H.random_ids(cfg, 420, seed=12)
    check(dtype, cfg, t, ids, in_pieces(eng, cfg, ids, [20] + [1] * 400), "400 decoded tokens")


# ------------------------------------------------------------------------------------------ generation
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", ["graph", "eager"])
def test_greedy_generation_through_the_entry_point(decode, dtype):
    from x0ne_engine_b200 import Model
    folder, cfg, t = H.folder("mixed")
    prompts = [H.random_ids(cfg, n, seed=20 + n) for n in (1, 7, 36, 64)]
    n_new = 14
    m = Model.from_folder(folder, dtype=dtype, max_batch=3, max_ctx=256, decode=decode)
    out = m.generate(prompts, max_tokens=n_new, stop_token_ids=())
    assert out.finish_reasons == ["length"] * len(prompts)
    for p, got in zip(prompts, out.tokens):
        ids = list(p)
        for tok in got:
            record = {}
            row = H.plain_logits(cfg, t, ids, record=record)[-1]
            top = np.sort(row)[-2:]
            if tok != int(np.argmax(row)):
                # the two part only at a close call: of the argmax itself, or of a router somewhere before it (then the
                # engine's own continuation is what the plain implementation gives when it follows the engine's choices)
                tol = 1e-4 if dtype == "float32" else 2 * 0.05
                if top[1] - top[0] > tol * np.abs(row).max():
                    eng_run = whole(engine("mixed", dtype)[0], cfg, ids)
                    assert tok == int(np.argmax(H.plain_logits(cfg, t, ids, eng_run.chosen)[-1])), "a token left a clear argmax"
                break
            ids.append(tok)
    assert m.generate(prompts, max_tokens=n_new, stop_token_ids=()).tokens == out.tokens


def test_random_model_from_a_configuration_generates():
    from x0ne_engine_b200 import Model
    from x0ne_engine_b200.config import config_from_dict
    m = Model.random(config_from_dict(H.CONFIGS["even"]()), seed=1, max_batch=2, max_ctx=128, norm_jitter=0.1)
    out = m.generate([[1, 2, 3], [4]], max_tokens=5, stop_token_ids=())
    assert [len(x) for x in out.tokens] == [5, 5] and all(0 <= x < 256 for row in out.tokens for x in row)


def test_short_prompt_passes_replayed_from_graphs_give_the_same_bits():
    eng, cfg, t = engine("mixed", "bfloat16", pass_graphs=True)
    base, _, _ = engine("mixed", "bfloat16", pass_graphs=False)
    assert eng.replayable and eng.pass_graphs and not base.pass_graphs
    before = eng.pass_graph_replays
    for k, lengths in enumerate([[100], [120], [70], [126], [20], [30], [5], [5], [100, 20], [90, 30], [100]]):
        prompts = [H.random_ids(cfg, n, 100 + 7 * k + j) for j, n in enumerate(lengths)]
        got = []
        for e in (eng, base):
            slots = [e.new_sequence() for _ in lengths]
            first = e.step(slots, prompts).cpu().numpy()
            nxt = e.step(slots, [[int(np.argmax(r))] for r in first]).cpu().numpy()
            for s in slots:
                e.free_sequence(s)
            got.append((first, nxt))
        assert np.array_equal(got[0][0], got[1][0]) and np.array_equal(got[0][1], got[1][1]), lengths
    assert eng.pass_graph_replays - before >= 4
