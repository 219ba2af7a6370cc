"""Retuvik on the GPU against the plain implementation (tests/retuvik_plain.py), in float32 and bfloat16: every
mechanism alone, whole prompts, token-by-token decoding, portions down to two tokens, unequal batches with slots
and pages used again, the window's edge in prompts and in decoding, far keys and a far token in the recurrent
state, the first tokens, long decoding, odd sizes and values a configuration may leave out, and greedy generation
through the entry point.  Token sequences are drawn so that no router is within rounding of another choice (the
margin is checked by the plain implementation), since a choice that flips changes a row altogether."""
import numpy as np
import pytest
import torch

import retuvik_helpers as H
import retuvik_plain as P
from helpers import assert_close_f32, first_difference

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
DEV = "cuda:0"
MARGIN = {"float32": 1e-4, "bfloat16": 0.0}
_engines = {}


def engine(name, dtype, seed=0, sharp=1.0, max_tokens=2048, **kw):
    from x0ne_engine_b200 import Engine
    if dtype == "bfloat16":
        kw.setdefault("pass_graphs", False)          # the routers' choices are recorded by Python hooks (H.Choices)
    key = (name, dtype, seed, sharp, max_tokens, tuple(sorted(kw.items())))
    if key not in _engines:
        folder, cfg, tensors = H.folder(name, seed, sharp)
        _engines[key] = (Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, max_seq_len=max_tokens, **kw), cfg, tensors)
    return _engines[key]


def close_bf16(got, want, what):
    """Rows within the bfloat16 tolerance of the other tests; of many rows, one in fifty (or one) may reach twice
    that: a routed layer's weights are a softmax, and a row in which two of them are close amplifies the rounding
    of its input."""
    from helpers import BF16_KL_TOL, BF16_LOGIT_TOL, kl_rows
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

    def __init__(self, logits, forced):
        self.logits, self.forced = logits, forced


def check(dtype, cfg, t, ids, run, what, rows=None):
    """A run against the plain implementation.  float32: the plain implementation chooses for itself.  bfloat16: it
    follows the run's choices (they may differ where two are within bfloat16's rounding), and the choices must
    agree with the plain ones wherever those are clear."""
    rows = slice(None) if rows is None else rows
    if dtype == "float32":
        assert_close_f32(run.logits[rows], H.plain_logits(cfg, t, ids)[rows], what)
        return
    close_bf16(run.logits[rows], H.plain_logits(cfg, t, ids, None, None, run.forced)[rows], what)
    if run.forced:
        overall, clear = H.agreement(cfg, t, ids, run.forced, clear=0.15)
        assert clear >= 0.98 and overall >= 0.85, f"{what}: routers agree on {overall:.3f} of all rows, {clear:.3f} of the clear ones"


def same_cut(dtype, cfg, t, ids, run, base, what):
    """Two runs of one sequence cut differently: the same bits in float32; in bfloat16 each is held against the
    plain implementation (a router may choose differently in the two)."""
    if dtype == "float32":
        got, want = np.asarray(run.logits), np.asarray(base.logits)
        assert np.array_equal(got, want), f"{what}: first difference at {first_difference(got, want)}"
    else:
        check(dtype, cfg, t, ids, run, what)


def ids_for(cfg, t, n, dtype, seed=0):
    return H.clear_ids(cfg, t, n, seed, MARGIN[dtype])


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
            forced = rec.of(s, len(ids))
        finally:
            eng.free_sequence(s)
    return Run(np.concatenate(out), forced)


def whole(eng, cfg, ids):
    return in_pieces(eng, cfg, ids, [])


# ------------------------------------------------------------------------------------------ row-wise kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,groups", [(72, 3), (100, 5), (128, 1), (1000, 4), (4096, 2), (66, 66)])
def test_add_then_norm_in_groups(dtype, hidden, groups):
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(2)
    rows, eps = 6, 1e-5
    resid = torch.randn(rows, hidden, generator=g).to(DEV)
    resid[:, : hidden // groups] *= 30.0                 # one part far larger than the others: a norm over the whole row would show
    d = (3 * torch.randn(rows, hidden, generator=g)).to(dtype).to(DEV)
    w = (1 + 0.2 * torch.randn(hidden, generator=g)).to(DEV)
    out = torch.empty((rows, hidden), dtype=dtype, device=DEV)
    before = resid.clone()
    ops.add_rmsnorm(resid, d, w, out, rows, eps, groups=groups)
    want_r = before.double() + d.double()
    assert (resid.double() - want_r).abs().max() <= 2e-6 * want_r.abs().max()
    want = P.group_norm(want_r.cpu(), w.double().cpu(), eps, groups)
    tol = 3e-6 if dtype == torch.float32 else 2 ** -8
    assert (out.double().cpu() - want).abs().max() <= tol * want.abs().max()
    if groups > 1:
        assert (P.group_norm(want_r.cpu(), w.double().cpu(), eps, 1) - want).abs().max() > 0.1 * want.abs().max()
    # gathered rows (the final norm of the wanted rows only), no delta
    rows_t = torch.tensor([4, 1], dtype=torch.int32, device=DEV)
    out2 = torch.empty((2, hidden), dtype=dtype, device=DEV)
    ops.add_rmsnorm(resid, None, w, out2, 2, eps, rows_t, groups=groups)
    assert torch.equal(out2, out[[4, 1]])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pass_opener(dtype):
    """resid = ((resid + delta) + scale * table[token]) + step, each term optional."""
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(3)
    rows, hidden = 5, 72
    table = torch.randn(50, hidden, generator=g).to(dtype).to(DEV)
    tok = torch.tensor([3, 49, 0, 7, 7], dtype=torch.int32, device=DEV)
    step = torch.randn(hidden, generator=g).to(DEV)
    delta = torch.randn(rows, hidden, generator=g).to(dtype).to(DEV)
    base = torch.randn(rows, hidden, generator=g).to(DEV)
    for use_delta, use_table, use_step in [(True, True, True), (False, False, True), (True, False, True), (False, True, False)]:
        resid = base.clone()
        ops.open_pass(resid, delta if use_delta else None, table if use_table else None, tok if use_table else None, 3.25,
                      step if use_step else None, rows)
        want = base.double()
        if use_delta:
            want = want + delta.double()
        if use_table:
            want = want + 3.25 * table.double()[tok.long()]
        if use_step:
            want = want + step.double()
        assert (resid.double() - want).abs().max() <= 1e-6 * want.abs().max(), (use_delta, use_table, use_step)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_bias_and_two_branch_activation(dtype):
    from x0ne_engine_b200.csrc import ops
    from x0ne_engine_b200.parts.mlp import _softplus
    g = torch.Generator().manual_seed(5)
    rows, width, p, q = 7, 100, 0.8, -0.3
    x = (3 * torch.randn(rows, width, generator=g)).to(dtype).to(DEV)
    x[0, :4] = torch.tensor([0.0, -0.0, 1e-3, -1e-3]).to(dtype)
    bias = torch.randn(width, generator=g).to(DEV)
    bias[:4] = 0.0
    out = torch.empty_like(x)
    ops.bias_act(x, bias, out, rows, ops.ACT_QUAD_EXP, _softplus(p), 0.5 + _softplus(q))
    want = P.xielu(x.double().cpu() + bias.double().cpu(), p, q)
    tol = 3e-6 if dtype == torch.float32 else 2 ** -8
    assert ((out.double().cpu() - want).abs() <= tol * want.abs() + 1e-7).all()
    ops.bias_act(x, bias, out, rows)
    assert ((out.double().cpu() - (x.double().cpu() + bias.double().cpu())).abs() <= tol * (want.abs() + 4)).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H_,G,D,Dv,temp", [(6, 2, 20, 12, (0.7, 16)), (4, 4, 32, 32, None), (3, 1, 10, 6, (1.5, 1)), (8, 2, 64, 128, (0.5, 64))])
def test_head_norms_temperature_and_cache_write(dtype, H_, G, D, Dv, temp):
    from x0ne_engine_b200.cache import SequenceCache
    from x0ne_engine_b200.csrc import ops
    from x0ne_engine_b200.parts.base import CacheNeed
    g = torch.Generator().manual_seed(4)
    rows, eps = 6, 1e-5
    cache = SequenceCache([CacheNeed("kv", G, D, None, v_dim=None if Dv == D else Dv)], [None], 512, 512, dtype, DEV)
    slot = cache.acquire(300)
    pos = torch.tensor([0, 14, 15, 63, 64, 255], dtype=torch.int32, device=DEV)
    slots = torch.full((rows,), slot, dtype=torch.int32, device=DEV)
    width = H_ * D + G * D + G * Dv + 5                  # columns after the values (a gate, say) are left alone
    src = (2 * torch.randn(rows, width, generator=g)).to(dtype).to(DEV)
    wq = (1 + 0.3 * torch.randn(D, generator=g)).to(DEV)
    wk = (1 + 0.3 * torch.randn(D, generator=g)).to(DEV)
    q_out = torch.empty((rows, H_ * D), dtype=dtype, device=DEV)
    coef, every = temp or (0.0, 0)
    ops.head_norm_kv_write(src, H_ * D, H_ * D + G * D, wq, wk, eps, coef, every, True, q_out, H_, cache.kv_view(0), slots, pos, rows)
    x, p_cpu = src.double().cpu(), pos.cpu()
    q_want = P.unit_rms(x[:, :H_ * D].view(rows, H_, D), eps) * wq.double().cpu()
    if temp:
        q_want = q_want * P.query_temperature(p_cpu, coef, every)[:, None, None]
    k_want = P.unit_rms(x[:, H_ * D:H_ * D + G * D].view(rows, G, D), eps) * wk.double().cpu()
    v_want = P.unit_rms(x[:, H_ * D + G * D:H_ * D + G * D + G * Dv].view(rows, G, Dv), eps)
    tol = 3e-6 if dtype == torch.float32 else 2 ** -8
    assert (q_out.double().cpu().view(rows, H_, D) - q_want).abs().max() <= tol * q_want.abs().max()
    g0 = cache.groups[0]
    store = g0.storage[0].reshape(g0.n_pages, -1).double().cpu()
    for r in range(rows):
        page = int(g0.table_host[slot, int(p_cpu[r]) // 64])
        at = int(p_cpu[r]) % 64
        keys = store[page, :G * 64 * D].view(G, 64, D)[:, at]
        vals = store[page, G * 64 * D:].view(G, 64, Dv)[:, at]
        assert (keys - k_want[r]).abs().max() <= tol * k_want.abs().max()
        assert (vals - v_want[r]).abs().max() <= tol * v_want.abs().max()


@pytest.mark.parametrize("n,top", [(10, 3), (8, 1), (12, 12), (64, 6), (7, 2), (3, 3)])
def test_router_choice_on_logits(n, top):
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(n)
    rows = 37
    z = torch.randn(rows, n, generator=g) * 3
    z[0, :] = 1.0                                          # equals: the lowest indices win
    bias = torch.randn(n, generator=g) * 2
    bias[:3] = bias[0]
    chosen = torch.empty((rows, top), dtype=torch.int32, device=DEV)
    weights = torch.empty((rows, top), dtype=torch.float32, device=DEV)
    ops.moe_route(z.to(DEV), bias.to(DEV), n, 1, 1, top, rows, chosen, weights, None, 0, on_logits=True)
    want_c, want_w = P.choose((z + bias).double(), top)
    order = chosen.cpu().long().sort(-1)
    want_order = want_c.sort(-1)
    assert torch.equal(order.values, want_order.values)
    got_w = torch.gather(weights.cpu().double(), 1, order.indices)
    assert (got_w - torch.gather(want_w, 1, want_order.indices)).abs().max() <= 1e-6
    assert (weights.sum(-1).cpu() - 1).abs().max() <= 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,E,top,hidden,ff", [(1, 4, 2, 64, 40), (9, 6, 3, 72, 128), (150, 3, 2, 104, 50), (700, 16, 4, 256, 384), (513, 3, 1, 320, 256)])
def test_gated_experts_over_grouped_pairs(dtype, rows, E, top, hidden, ff):
    """down(silu(gate x) * up x) over the listed (row, choice) pairs against a loop over rows and choices: on the CUDA
    cores (float32, and bfloat16 where the tensor-core kernel does not take the shape) and on tcgen05, with gate and up
    rows packed one after the other or in blocks; experts with no pair and with more than a tile of them."""
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, hidden, generator=g).to(dtype)
    gate = (torch.randn(E, ff, hidden, generator=g) * (1.5 / hidden ** 0.5)).to(dtype)
    up = (torch.randn(E, ff, hidden, generator=g) / hidden ** 0.5).to(dtype)
    down = (torch.randn(E, hidden, ff, generator=g) / ff ** 0.5).to(dtype)
    prefer = torch.rand(E, generator=g) ** 3
    if E > top:
        prefer[E - 1] = 0                                  # the last expert gets no pair at all
    chosen = torch.stack([torch.multinomial(prefer + 1e-9 * (torch.arange(E) != E - 1), top, generator=g) for _ in range(rows)]).to(torch.int32)
    weights = torch.rand(rows, top, generator=g)
    pairs = rows * top
    block = ops.MOE_PAIR_BLOCK if ff % ops.MOE_PAIR_BLOCK == 0 else 0
    if block:
        packed = torch.cat([gate.reshape(E, -1, block, hidden), up.reshape(E, -1, block, hidden)], dim=2).reshape(E, 2 * ff, hidden)
    else:
        packed = torch.cat([gate, up], dim=1)
    tc = bool(block) and ops.moe_tc_takes(dtype, pairs, hidden, ff)
    tile = ops.MOE_TC_TILE_ROWS if tc else ops.MOE_TILE_ROWS
    n_tiles = ops.moe_max_tiles(pairs, E, tile)
    i32 = lambda *shape: torch.empty(shape, dtype=torch.int32, device=DEV)
    offsets, listed, tiles, n_real = i32(E + 1), i32(pairs), i32(n_tiles, 3), i32(1)
    act = torch.empty((pairs, ff), dtype=dtype, device=DEV)
    y = torch.empty((pairs, hidden), dtype=torch.float32, device=DEV)
    out = torch.empty((rows, hidden), dtype=dtype, device=DEV)
    xd, ch = x.to(DEV), chosen.to(DEV)
    ops.moe_group(ch, pairs, E, offsets, listed, tiles, tile, n_real)
    if tc:
        xs = torch.full((pairs, hidden), float("nan"), dtype=dtype, device=DEV)
        ops.moe_gather_rows(xd, listed, offsets, E, top, xs, pairs)
        ops.moe_product_tc(2, xs, packed.to(DEV), listed, tiles, n_real, n_tiles, act)
        ops.moe_product_tc(1, act, down.to(DEV), listed, tiles, n_real, n_tiles, y)
        ops.check_tc_status(torch.device(DEV))
    else:
        ops.moe_product(2, xd, packed.to(DEV), listed, tiles, n_tiles, top, act, block)
        ops.moe_product(1, act, down.to(DEV), listed, tiles, n_tiles, top, y)
    ops.moe_combine(y, xd, ch, weights.to(DEV), top, E, None, None, out, rows)
    want = torch.zeros(rows, hidden, dtype=torch.float64)
    for r in range(rows):
        for j in range(top):
            e = int(chosen[r, j])
            a = (torch.nn.functional.silu(gate[e].double() @ x[r].double()) * (up[e].double() @ x[r].double())).to(dtype).double()
            want[r] += weights[r, j].double() * (a @ down[e].double().T)
    tol = 1e-5 if dtype == torch.float32 else 2 ** -7
    assert (out.double().cpu() - want).abs().max() <= tol * want.abs().max()
    if dtype == torch.bfloat16 and rows >= 500:
        assert tc                                          # these shapes are the tensor-core kernel's


SLOPE_CASES = [  # q_heads, kv_heads, dk, dv, window
    (4, 2, 48, None, 100),
    (6, 2, 20, 12, 37),
    (3, 3, 24, 40, 64),
    (20, 1, 16, 80, 9),
    (8, 2, 64, 64, None),
    (2, 1, 128, 128, 300),
]


@pytest.mark.parametrize("case", SLOPE_CASES)
def test_attention_kernels_with_distance_bias_and_a_gate_per_value(case):
    """The general bfloat16 kernels (prompt tiles; decode with one split and with several) and the plain kernel in
    float32, against full score matrices in double precision: slope_h (i - j) off every score, the window, and
    sigmoid gates per (row, head, value) that lie inside a wider buffer."""
    from x0ne_engine_b200.cache import SequenceCache
    from x0ne_engine_b200.csrc import ops
    from x0ne_engine_b200.parts.base import CacheNeed
    H_, G, D, Dv, window = case
    Dv = Dv or D
    g = torch.Generator().manual_seed(H_ * 100 + D)
    T, scale = 330, 1.7 * D ** -0.5
    q = (1.5 * torch.randn(T, H_, D, generator=g)).bfloat16()
    k = torch.randn(T, G, D, generator=g).bfloat16()
    v = torch.randn(T, G, Dv, generator=g).bfloat16()
    gate_ld = H_ * Dv + 24
    gate = (2 * torch.randn(T, gate_ld, generator=g)).bfloat16()
    sl = P.slopes(H_)
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    ok = (j <= i) & ((i - j < window) if window else True)
    want = torch.zeros(T, H_, Dv, dtype=torch.float64)
    for h in range(H_):
        s = (q[:, h].double() @ k[:, h // (H_ // G)].double().T) * scale - sl[h] * (i - j).double()
        want[:, h] = torch.softmax(s.masked_fill(~ok, float("-inf")), -1) @ v[:, h // (H_ // G)].double()
    want = want * torch.sigmoid(gate[:, :H_ * Dv].double().view(T, H_, Dv))
    for dtype in (torch.bfloat16, torch.float32):
        cache = SequenceCache([CacheNeed("kv", G, D, None, v_dim=None if Dv == D else Dv)], [None], 1024, 1024, dtype, DEV)
        slot = cache.acquire(T)
        view = cache.kv_view(0)
        g0 = cache.groups[0]
        store = g0.storage[0].reshape(g0.n_pages, -1)
        for p0 in range(0, T, 64):                        # keys [kv head][64][D], then values [kv head][64][Dv] per page
            page, n = int(g0.table_host[slot, p0 // 64]), min(64, T - p0)
            kp = torch.zeros(G, 64, D, dtype=dtype)
            vp = torch.zeros(G, 64, Dv, dtype=dtype)
            kp[:, :n], vp[:, :n] = k[p0:p0 + n].transpose(0, 1).to(dtype), v[p0:p0 + n].transpose(0, 1).to(dtype)
            store[page] = torch.cat([kp.reshape(-1), vp.reshape(-1)]).to(DEV)
        qd, gd = q.reshape(T, H_ * D).to(dtype).to(DEV), gate.to(dtype).to(DEV)
        slope = sl.float().to(DEV)
        extra = ops.attn_extra(gate=gd, gate_ld=gate_ld, gate_wide=True, slope=slope)
        slots = torch.full((T,), slot, dtype=torch.int32, device=DEV)
        pos = torch.arange(T, dtype=torch.int32, device=DEV)
        tol = 2e-5 if dtype == torch.float32 else 2 ** -6
        out = torch.zeros((T, H_ * Dv), dtype=dtype, device=DEV)
        ops.attention_rows(qd, out, view, slots, pos, T, H_, scale, window or 0, extra)
        assert (out.double().cpu().view(T, H_, Dv) - want).abs().max() <= tol * want.abs().max(), ("plain", dtype)
        if dtype != torch.bfloat16:
            continue
        assert ops.attention_flex_takes(view, dtype, 0, False) and ops.attention_flex_takes(view, dtype, 0, True)
        # prompt tiles of 128 rows: the sequence in two portions (200 rows from position 0, then 130 more)
        out = torch.zeros((T, H_ * Dv), dtype=dtype, device=DEV)
        for first, n in ((0, 200), (200, 130)):
            n_t = -(-n // 128)
            tile_seq = torch.zeros(n_t, dtype=torch.int32, device=DEV)
            tile_row0 = (torch.arange(n_t, dtype=torch.int32, device=DEV) * 128).contiguous()
            ex = ops.attn_extra(gate=gd[first:], gate_ld=gate_ld, gate_wide=True, slope=slope)
            ops.attention_flex_prefill(qd[first:first + n], out[first:first + n], view, tile_seq, tile_row0, n_t,
                                       torch.tensor([0, n], dtype=torch.int32, device=DEV), torch.tensor([slot], dtype=torch.int32, device=DEV),
                                       torch.tensor([first], dtype=torch.int32, device=DEV), H_, scale, window or 0, ex)
        assert (out.double().cpu().view(T, H_, Dv) - want).abs().max() <= tol * want.abs().max(), "prompt tiles"
        # every row as a decode row of its own
        for splits in (1, 3):
            out = torch.zeros((T, H_ * Dv), dtype=dtype, device=DEV)
            scratch = torch.empty(ops.attention_flex_scratch_bytes(T, H_, G, Dv, splits) // 4 + 16, dtype=torch.float32, device=DEV) if splits > 1 else None
            ops.attention_flex_decode(qd, out, view, slots, pos, T, H_, scale, window or 0, extra, splits, scratch)
            assert (out.double().cpu().view(T, H_, Dv) - want).abs().max() <= tol * want.abs().max(), ("decode", splits)


# ------------------------------------------------------------------------------------------ the recurrence's kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_shift_blends(dtype):
    """Rows of three sequences in one pass: one starts (zeros before it), one goes on from the row its state keeps,
    one brings a single row; a padding row (slot -1) is left alone."""
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(6)
    width, n_mix, mats = 72, 5, 40
    h = torch.randn(8, width, generator=g).to(dtype).to(DEV)
    mu = torch.rand(n_mix, width, generator=g).to(DEV)
    state = torch.randn(4, mats + width, generator=g).to(DEV)
    row_slot = torch.tensor([2, 2, 2, 0, 0, 3, -1, -1], dtype=torch.int32, device=DEV)
    row_pos = torch.tensor([0, 1, 2, 9, 10, 4, 0, 0], dtype=torch.int32, device=DEV)
    state[2, mats:] = 0.0                                   # a sequence's start: its state is zero
    mixes = torch.zeros((n_mix, 8, width), dtype=dtype, device=DEV)
    ops.token_shift_mix(h, mu, mixes, state, mats, row_slot, row_pos, 6)
    x, last = h.double().cpu(), state[:, mats:].double().cpu()
    before = torch.stack([torch.zeros(width, dtype=torch.float64), x[0], x[1], last[0], x[3], last[3]])
    want = x[:6][None] + (before - x[:6])[None] * mu.double().cpu()[:, None, :]
    tol = 3e-6 if dtype == torch.float32 else 2 ** -8
    assert (mixes[:, :6].double().cpu() - want).abs().max() <= tol * want.abs().max()
    assert float(mixes[:, 6:].abs().max()) == 0.0


def scan_inputs(g, rows, heads, n, dtype, strong=False):
    hn = heads * n
    r, k, v = ((torch.randn(rows, hn, generator=g)).to(dtype).to(DEV) for _ in range(3))
    z = (torch.randn(rows, hn, generator=g)).to(DEV)
    w0 = (-6.0 + (9.0 if strong else 7.0) * torch.rand(hn, generator=g)).to(DEV)
    u = torch.randn(hn, generator=g).to(DEV)
    return r, k, v, z, w0, u


def plain_scan(r, k, v, z, w0, u, heads, n, S):
    T = r.shape[0]
    w = torch.exp(-torch.exp(z.double().cpu() + w0.double().cpu())).view(T, heads, n)
    return P.wkv_scan(r.double().cpu().view(T, heads, n), k.double().cpu().view(T, heads, n), v.double().cpu().view(T, heads, n), w,
                      u.double().cpu().view(heads, n), S).reshape(T, heads * n)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,n", [(5, 10), (1, 7), (3, 32), (4, 48), (2, 64), (2, 96), (1, 128), (2, 136), (1, 300)])
def test_scan_over_unequal_sequences_and_again_from_the_state(dtype, heads, n):
    """Three sequences of 1, 37 and 20 rows and a padding sequence in one launch, in slots 3, 0 and 2; then 5, 1 and 2
    more rows from the states the first launch left: outputs and states against the token-by-token loop, and the
    same bits as one launch over all rows of a sequence."""
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(7 + n)
    width, hn, mats = 24, heads * n, heads * n * n
    lens1, lens2, slots = [1, 37, 20], [5, 1, 2], [3, 0, 2]
    rows = sum(lens1) + sum(lens2)
    r, k, v, z, w0, u = scan_inputs(g, rows, heads, n, dtype)
    h = torch.randn(rows, width, generator=g).to(dtype).to(DEV)
    state = torch.zeros((5, mats + width), dtype=torch.float32, device=DEV)
    state[1] = 7.0                                          # a slot no sequence of the launch holds
    o = torch.zeros((rows, hn), dtype=torch.float32, device=DEV)
    seq_slot = torch.tensor(slots + [-1], dtype=torch.int32, device=DEV)
    first1 = torch.tensor([0, 1, 38, 58, 58], dtype=torch.int32, device=DEV)
    a = slice(0, 58)
    ops.wkv_scan(r[a], k[a], v[a], z[a], w0, u, h[a], o[a], state, first1, seq_slot, 4, heads, n)
    b = slice(58, rows)
    first2 = torch.tensor([0, 5, 6, 8, 8], dtype=torch.int32, device=DEV)
    ops.wkv_scan(r[b], k[b], v[b], z[b], w0, u, h[b], o[b], state, first2, seq_slot, 4, heads, n)
    tol = 1e-5 if dtype == torch.float32 else 1e-5          # the scan itself is float32 in both; inputs are read exactly
    at1, at2 = 0, 58
    for s, (n1, n2) in enumerate(zip(lens1, lens2)):
        idx = list(range(at1, at1 + n1)) + list(range(at2, at2 + n2))
        S = torch.zeros(heads, n, n, dtype=torch.float64)
        want = plain_scan(r[idx], k[idx], v[idx], z[idx], w0, u, heads, n, S)
        got = o[idx].double().cpu()
        assert (got - want).abs().max() <= tol * want.abs().max(), f"sequence {s}"
        assert (state[slots[s], :mats].double().cpu().view(heads, n, n) - S).abs().max() <= tol * S.abs().max()
        assert torch.equal(state[slots[s], mats:], h[idx[-1]].float())
        # all of the sequence's rows in one launch: the same bits
        state2 = torch.zeros_like(state)
        o2 = torch.zeros((len(idx), hn), dtype=torch.float32, device=DEV)
        ops.wkv_scan(r[idx].contiguous(), k[idx].contiguous(), v[idx].contiguous(), z[idx].contiguous(), w0, u, h[idx].contiguous(), o2,
                     state2, torch.tensor([0, len(idx)], dtype=torch.int32, device=DEV), torch.tensor([4], dtype=torch.int32, device=DEV),
                     1, heads, n)
        assert torch.equal(o2, o[idx]) and torch.equal(state2[4], state[slots[s]])
        at1, at2 = at1 + n1, at2 + n2
    assert float((state[1] - 7.0).abs().max()) == 0.0 and float(state[4].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,n", [(3, 10), (2, 32), (2, 64), (1, 100), (1, 128), (1, 200)])
def test_one_token_steps_give_the_bits_of_the_scan_over_all_rows(dtype, heads, n):
    """Three sequences of 21 rows in one launch, against the same rows fed one per sequence and launch through the
    kernel for decode steps (slots in another order, a padding sequence in the middle): outputs and states bit for bit."""
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(11 + n)
    width, hn, mats, T, B = 16, heads * n, heads * n * n, 21, 3
    r, k, v, z, w0, u = scan_inputs(g, B * T, heads, n, dtype)
    h = torch.randn(B * T, width, generator=g).to(dtype).to(DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)      # noqa: E731
    state = (0.1 * torch.randn((4, mats + width), generator=g)).to(DEV)
    state2 = state[[2, 0, 1, 3]].clone()                  # the same starts, held in slots 2 -> 0, 0 -> 1, 1 -> 2
    o = torch.zeros((B * T, hn), dtype=torch.float32, device=DEV)
    ops.wkv_scan(r, k, v, z, w0, u, h, o, state, i32([0, T, 2 * T, 3 * T]), i32([2, 0, 1]), B, heads, n)
    o2 = torch.zeros_like(o)
    for t in range(T):
        rows = [t, T + t, 2 * T + t]
        pick = lambda x: x[rows].contiguous()               # noqa: E731
        ot = torch.zeros((B, hn), dtype=torch.float32, device=DEV)
        ops.wkv_scan(pick(r), pick(k), pick(v), pick(z), w0, u, pick(h), ot, state2, i32([0, 1, 1, 2, 3]), i32([0, -1, 1, 2]), 4,
                     heads, n, one_token=True)
        o2[rows] = ot
    assert torch.equal(o2, o)
    assert torch.equal(state2[0], state[2]) and torch.equal(state2[1], state[0]) and torch.equal(state2[2], state[1])
    assert torch.equal(state2[3], state[3])


def test_scan_keeps_a_token_hundreds_of_rows_back():
    """One key channel of head 1 hardly decays and only the first token writes to it; a query 600 rows later reads
    that channel alone.  Its output is the first token's value (times the decays), so a state that is lost, reset
    or mixed with another slot's shows; the bonus u enters only for the current token."""
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(8)
    heads, n, rows, width = 2, 48, 601, 8
    hn, mats = heads * n, heads * n * n
    r, k, v, z, w0, u = scan_inputs(g, rows, heads, n, torch.float32, strong=True)
    c = n + 5                                               # head 1, channel 5
    w0[c], z[:, c] = -9.0, 0.0
    k[1:, c], k[0, c] = 0.0, 2.0
    r[-1, n:] = 0.0
    r[-1, c] = 1.0
    h = torch.zeros((rows, width), device=DEV)
    state = torch.zeros((2, mats + width), device=DEV)
    o = torch.zeros((rows, hn), device=DEV)
    for cuts in ([rows], [1, 300, 299, 1]):
        state.zero_()
        at = 0
        for c_ in cuts:
            s = slice(at, at + c_)
            ops.wkv_scan(r[s], k[s], v[s], z[s], w0, u, h[s], o[s], state, torch.tensor([0, c_], dtype=torch.int32, device=DEV),
                         torch.tensor([1], dtype=torch.int32, device=DEV), 1, heads, n)
            at += c_
        want = 2.0 * v[0, n:].double() * np.exp(-np.exp(-9.0)) ** (rows - 2)
        # 600 float32 products with a float32 decay: each may round by 2^-24 twice
        assert (o[-1, n:].double() - want).abs().max() <= 600 * 2.0 ** -23 * want.abs().max(), cuts
        S = torch.zeros(heads, n, n, dtype=torch.float64)
        full = plain_scan(r, k, v, z, w0, u, heads, n, S)
        assert (o.double().cpu() - full).abs().max() <= 600 * 2.0 ** -23 * full.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,n", [(5, 10), (2, 64), (1, 136)])
def test_head_norm_weight_and_gate(dtype, heads, n):
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(9)
    rows, hn, eps = 9, heads * n, 1e-5
    o = torch.randn(rows, hn, generator=g).to(DEV)
    o[:, :n] *= 50.0                                        # one head far larger: a norm over the whole row would show
    o[3] = 0.0                                              # eps alone under the root
    w = (1 + 0.3 * torch.randn(hn, generator=g)).to(DEV)
    gate = (2 * torch.randn(rows, hn, generator=g)).to(dtype).to(DEV)
    out = torch.empty((rows, hn), dtype=dtype, device=DEV)
    ops.head_norm_gate(o, w, gate, out, rows, heads, n, eps)
    want = P.unit_rms(o.double().cpu().view(rows, heads, n), eps).reshape(rows, hn) * w.double().cpu() * torch.nn.functional.silu(gate.double().cpu())
    tol = 3e-6 if dtype == torch.float32 else 2 ** -8
    assert (out.double().cpu() - want).abs().max() <= tol * want.abs().max()


# ------------------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths", [("wkv_only", [1, 2, 40]), ("attention_only", [1, 2, 9, 10, 40]), ("dense_only", [1, 12]),
                                          ("experts_only", [1, 3, 70]), ("loop_only", [1, 30]), ("mixed", [1, 2, 37, 38, 65, 150]),
                                          ("even", [64, 131, 300]), ("wide", [5, 71, 141]), ("odd", [1, 12, 90]), ("plain", [1, 100]),
                                          ("served", [7, 300])])
def test_each_request_alone_and_whole(name, lengths, dtype):
    eng, cfg, t = engine(name, dtype)
    for k, n in enumerate(lengths):
        ids = ids_for(cfg, t, n, dtype, seed=k)
        check(dtype, cfg, t, ids, whole(eng, cfg, ids), f"{name} len {n}")


def test_residual_stream_after_every_layer_run():
    """The float32 residual after each run of a layer (the pending delta added by hand) against the plain one: a
    repeated layer counts each time, and what opens the next pass is not yet in it."""
    eng, cfg, t = engine("mixed", "float32")
    ids = ids_for(cfg, t, 90, "float32", seed=3)
    want = []
    H.plain_logits(cfg, t, ids, want)
    seen = []
    for b in eng.model.blocks:
        def wrapped(ctx, entry, resid, delta, cache_entry=None, write_cache=True, _f=b.forward):
            out = _f(ctx, entry, resid, delta, cache_entry=cache_entry, write_cache=write_cache)
            seen.append((resid[:ctx.n_rows].double() + out[:ctx.n_rows].double()).cpu())
            return out
        b.forward = wrapped
    try:
        whole(eng, cfg, ids)
    finally:
        for b in eng.model.blocks:
            del b.forward
    assert len(seen) == len(want) == 7
    for i, (a, b) in enumerate(zip(seen, want)):
        assert (a - b.double()).abs().max() <= 1e-4 * b.abs().max(), f"layer run {i}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,n,tail", [("mixed", 120, 60), ("wide", 100, 40), ("even", 160, 40), ("odd", 70, 30), ("plain", 90, 50),
                                         ("served", 330, 140)])
def test_prefill_against_token_by_token(name, n, tail, dtype):
    eng, cfg, t = engine(name, dtype)
    ids = ids_for(cfg, t, n, dtype, seed=5)
    base = whole(eng, cfg, ids)
    got = in_pieces(eng, cfg, ids, [n - tail] + [1] * tail)
    same_cut(dtype, cfg, t, ids, got, base, f"{name}: last {tail} one by one")
    check(dtype, cfg, t, ids, got, f"{name} decoded")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "even"])
def test_prompt_in_portions_down_to_two_tokens(name, dtype):
    eng, cfg, t = engine(name, dtype)
    ids = ids_for(cfg, t, 170, dtype, seed=6)
    base = whole(eng, cfg, ids)
    for cuts in ([2] * 30, [64, 64], [63, 2, 1, 64], [37, 37, 37, 37], [3, 125, 2], [129]):
        same_cut(dtype, cfg, t, ids, in_pieces(eng, cfg, ids, cuts), base, f"{name} cut {cuts[:4]}")
    check(dtype, cfg, t, ids, base, name)


def test_a_step_cut_into_passes_inside_prompts():
    eng, cfg, t = engine("mixed", "float32", max_step_tokens=64)
    ids = ids_for(cfg, t, 150, "float32", seed=7)
    assert np.array_equal(whole(eng, cfg, ids).logits, whole(engine("mixed", "float32")[0], cfg, ids).logits)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_unequal_batches_against_each_alone_with_slots_used_again(name, dtype):
    eng, cfg, t = engine(name, dtype)
    for round_ in range(3):                      # the second and third rounds get slots, pages and states that were used
        lengths, steps = [[1, 30, 77, 140], [66, 2, 129], [140, 5]][round_], [3, 9, 1, 6]
        full = [ids_for(cfg, t, n + steps[k], dtype, seed=10 * round_ + k) for k, n in enumerate(lengths)]
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
def test_window_edges_that_decide(dtype):
    """Sharp queries make single keys decide a row, so a window that is one off, or a page read wrongly, changes
    the logits by far more than the tolerance.  Windows of 37 and 64 positions against pages of 64; every position of
    a 260-token sequence is checked, in a prompt and decoded alone."""
    eng, cfg, t = engine("mixed", dtype, seed=3, sharp=4.0 if dtype == "float32" else 2.0)
    ids = ids_for(cfg, t, 260, dtype, seed=8)
    want = H.plain_logits(cfg, t, ids)

    def moved(change):
        layers = [dict(l, mixer=dict(l["mixer"], mask=change(dict(l["mixer"]["mask"])))) if l["type"] == "attention" else l
                  for l in cfg["layers"]]
        diff = np.abs(H.plain_logits({**cfg, "layers": layers}, t, ids) - want).max(-1) / np.abs(want).max(-1)
        return (diff > 0.1).sum()
    # the test sees what it is for: one more key in the window, or one fewer, changes the plain result
    many = 15 if dtype == "float32" else 8
    assert moved(lambda m: {**m, "size": m["size"] + 1}) > many
    assert moved(lambda m: {**m, "size": m["size"] - 1}) > many
    check(dtype, cfg, t, ids, whole(eng, cfg, ids), "prompt")
    check(dtype, cfg, t, ids, in_pieces(eng, cfg, ids, [30] + [1] * 230), "decoded across window edges and page borders")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_key_far_back_and_the_distance_bias(dtype):
    """A layer without a window: the first token's key is made to dominate the last token's query in the head with
    the smallest slope (one embedding feature that only the first token has feeds one key channel, another that only
    the last token has feeds the same query channel), so the last logits hang on a key 700 positions and eleven
    pages back, read in a prompt and in decoding.  Cutting that key off, or leaving the distance bias out, changes
    the plain result by more than the tolerance."""
    from x0ne_engine_b200 import Engine
    cfg = H.config([H.layer(H.attention(heads=4, kv_heads=2, window=None, temp=(0.4, 100)), None), H.layer(H.wkv(12, 3), H.dense(64)),
                    H.layer(H.attention(heads=4, kv_heads=2, window=45), H.moe(4, 2, 24))])
    t = H.make_tensors(cfg, seed=4)
    special, late, d = 7, 11, cfg["layers"][0]["mixer"]["dim"]
    t["embed"][:, :2] = 0.0
    t["embed"][special, 0] = 8.0
    t["embed"][late, 1] = 8.0
    t["l0.mix.k"][d] = 0.0                       # key head 1, channel 0: reads feature 0 only
    t["l0.mix.k"][d, 0] = 4.0
    t["l0.mix.q"][3 * d] = 0.0                   # query head 3, channel 0: reads feature 1 only
    t["l0.mix.q"][3 * d, 1] = 4.0
    t["l0.mix.q.norm"][0] = t["l0.mix.k.norm"][0] = 2.0
    t["l0.mix.o"] *= 3.0
    t = {k: v.bfloat16().float() for k, v in t.items()}
    folder = H.write_folder(cfg, t, "x0ne_rtv_far_")
    ids = [12 + x % (cfg["vocab"] - 12) for x in H.clear_ids(cfg, t, 700, 9)]
    ids[0], ids[-1] = special, late
    want = H.plain_logits(cfg, t, ids)[-3:]

    def with_layer0(**change):
        return {**cfg, "layers": [dict(cfg["layers"][0], mixer={**cfg["layers"][0]["mixer"], **change})] + cfg["layers"][1:]}
    cut_off = H.plain_logits(with_layer0(mask={"size": 650}), t, ids)[-1]
    assert np.abs(cut_off - want[-1]).max() > 0.07 * np.abs(want[-1]).max()
    real = P.slopes
    try:
        P.slopes = lambda heads: 0.0 * real(heads)
        flat = H.plain_logits(cfg, t, ids)
    finally:
        P.slopes = real
    assert (np.abs(flat - H.plain_logits(cfg, t, ids)).max(-1) > 0.07 * np.abs(want).max()).sum() > 100
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_seq_len=1024, pass_graphs=False)
    check(dtype, cfg, t, ids, whole(eng, cfg, ids), "far key in a prompt", rows=slice(-3, None))
    check(dtype, cfg, t, ids, in_pieces(eng, cfg, ids, [697, 1, 1]), "far key decoded", rows=slice(-3, None))


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_of_a_sequence(dtype):
    eng, cfg, t = engine("mixed", dtype)
    ids = ids_for(cfg, t, 6, dtype, seed=11)
    check(dtype, cfg, t, ids, in_pieces(eng, cfg, ids, [1, 1, 1, 1, 1]), "first tokens one by one")
    check(dtype, cfg, t, ids, in_pieces(eng, cfg, ids, [2, 2]), "first tokens in twos")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype):
    eng, cfg, t = engine("even", dtype)
    ids = ids_for(cfg, t, 420, dtype, seed=12)
    check(dtype, cfg, t, ids, in_pieces(eng, cfg, ids, [20] + [1] * 400), "400 decoded tokens")


# ------------------------------------------------------------------------------------------ generation
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", ["graph", "eager"])
def test_greedy_generation_through_the_entry_point(decode, dtype):
    from x0ne_engine_b200 import Model
    folder, cfg, t = H.folder("mixed")
    prompts = [ids_for(cfg, t, n, dtype, seed=20 + n) for n in (1, 7, 36, 64)]
    n_new = 14
    m = Model.from_folder(folder, dtype=dtype, max_batch=3, max_ctx=256, decode=decode)
    out = m.generate(prompts, max_tokens=n_new, stop_token_ids=())
    assert out.finish_reasons == ["length"] * len(prompts)
    for p, got in zip(prompts, out.tokens):
        ids = list(p)
        for tok in got:
            margins = []
            row = H.plain_logits(cfg, t, ids, None, margins)[-1]
            top = np.sort(row)[-2:]
            clear_route = min(float(x.min()) for x in margins) >= (1e-4 if dtype == "float32" else 0.15)
            if tok != int(np.argmax(row)):
                tol = 1e-4 if dtype == "float32" else 2 * 0.05
                assert not clear_route or top[1] - top[0] <= tol * np.abs(row).max(), "a token left a clear argmax"
                break
            if not clear_route:
                break                       # (from a close call of a router on, the two may part)
            ids.append(tok)
    assert m.generate(prompts, max_tokens=n_new, stop_token_ids=()).tokens == out.tokens


def test_random_model_from_a_configuration_generates():
    from x0ne_engine_b200 import Model
    from x0ne_engine_b200.config import config_from_dict
    cfg = H.CONFIGS["even"]()
    for l in cfg["layers"]:
        if l["type"] == "wkv":
            l["mixer"]["decay_rank"] = 8        # no checkpoint to take it from
    m = Model.random(config_from_dict(cfg), seed=1, max_batch=2, max_ctx=128, norm_jitter=0.1)
    out = m.generate([[1, 2, 3], [4]], max_tokens=5, stop_token_ids=())
    assert [len(x) for x in out.tokens] == [5, 5] and all(0 <= x < 256 for row in out.tokens for x in row)


def test_short_prompt_passes_replayed_from_graphs_give_the_same_bits():
    eng, cfg, t = engine("mixed", "bfloat16", pass_graphs=True)
    base, _, _ = engine("mixed", "bfloat16", pass_graphs=False)
    assert eng.replayable and eng.pass_graphs and not base.pass_graphs
    before = eng.pass_graph_replays
    for k, lengths in enumerate([[100], [120], [70], [126], [20], [30], [5], [5], [100, 20], [90, 30], [100]]):
        prompts = [H.clear_ids(cfg, t, n, 100 + 7 * k + j) for j, n in enumerate(lengths)]
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
