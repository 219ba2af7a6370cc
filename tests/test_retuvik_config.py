"""Retuvik on the CPU: the reader of config.json, its refusals, the model as data (parts, tensor names, run order,
what every layer run keeps per sequence), and properties of the plain implementation itself."""
import copy

import numpy as np
import pytest
import torch

import retuvik_helpers as H
import retuvik_plain as P
from x0ne_engine_b200.config import ConfigError, config_from_dict, detect
from x0ne_engine_b200.config.retuvik import RetuvikConfig
from x0ne_engine_b200.engine.model import cache_need_of_layer, step_bytes_of_spec, tensor_needs_of_spec


def shapes_of(cfg, seed=0):
    return {k: tuple(v.shape) for k, v in H.make_tensors(cfg, seed).items()}


def test_config_is_read_and_written_back():
    for name, make in H.CONFIGS.items():
        d = make()
        assert detect(d) == "Retuvik"
        c = config_from_dict(d)
        assert isinstance(c, RetuvikConfig) and c.to_dict() == d, name
        assert config_from_dict(c.to_dict()) == c


@pytest.mark.parametrize("change,word", [
    (lambda d: d["layers"][0]["mixer"].update(extra=1), "extra"),
    (lambda d: d["layers"][1]["mixer"]["mask"].update(left=1), "left"),
    (lambda d: d["layers"][1]["mixer"].update(heads=5), "multiple"),
    (lambda d: d["layers"][0].update(type="conv"), "conv"),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=9), "chooses"),
    (lambda d: d["layers"][0]["mlp"].update(kind="glu"), "glu"),
    (lambda d: d["norm"].pop("eps"), "eps"),
    (lambda d: d["norm"].update(groups=5), "groups"),
    (lambda d: d["loop"].update(stop=9), "loop"),
    (lambda d: d["loop"].update(start=3), "loop"),
    (lambda d: d["loop"].update(times=0), "times"),
    (lambda d: d["layers"][1]["mixer"].pop("scale"), "scale"),
])
def test_refusals_name_the_key(change, word):
    d = copy.deepcopy(H.CONFIGS["mixed"]())
    change(d)
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert word in str(e.value)


def test_run_order_repeats_the_stretch_and_opens_every_pass():
    d = H.CONFIGS["mixed"]()
    c = config_from_dict(d)
    assert [i for i, _ in c.run_layers()] == [0, 1, 2, 1, 2, 3, 4] == [i for i, _, _ in P.run_order(d)]
    spec = c.with_tensor_shapes(shapes_of(d)).to_spec()
    assert [e.layer for e in spec.run_order] == [0, 1, 2, 1, 2, 3, 4]
    openers = [(k, e.before["add_embedding"], e.before["step_row"]) for k, e in enumerate(spec.run_order) if e.before is not None]
    assert openers == [(1, False, 0), (3, True, 1)]
    assert all(e.reads_cache_of is None for e in spec.run_order)           # every pass keeps a cache or state of its own
    # a stretch from layer 0, run three times; one that runs once still adds its step vector; none at all
    even = config_from_dict(H.CONFIGS["even"]())
    assert [i for i, _ in even.run_layers()] == [0, 1, 0, 1, 0, 1, 2]
    spec1 = config_from_dict(H.CONFIGS["wide"]()).with_tensor_shapes(shapes_of(H.CONFIGS["wide"]())).to_spec()
    assert [(e.before is not None) for e in spec1.run_order] == [True, False, False] and spec1.run_order[0].before["add_embedding"] is False
    plain = config_from_dict(H.CONFIGS["plain"]())
    assert plain.loop is None and all(t is None for _, t in plain.run_layers())


def test_spec_parts_tensor_names_and_what_a_sequence_keeps():
    d = H.CONFIGS["mixed"]()
    c = config_from_dict(d)
    assert c.needs_tensor_shapes()
    with pytest.raises(ConfigError):
        c.to_spec()                                   # the decay's inner width is a tensor's shape
    t = H.make_tensors(d, 0)
    spec = c.with_tensor_shapes({k: tuple(v.shape) for k, v in t.items()}).to_spec()
    assert [l.block for l in spec.layers] == ["prenorm", "prenorm", "prenorm", "prenorm_mixer", "prenorm"]
    assert [l.parts["mixer"].kind for l in spec.layers] == ["matrix_state_recurrence", "distance_bias_attention"] * 2 + ["matrix_state_recurrence"]
    assert [l.parts["ffn"].kind for l in spec.layers if "ffn" in l.parts] == ["biased_mlp", "routed_experts", "routed_experts", "biased_mlp"]
    assert spec.layers[0].parts["mixer"]["decay_rank"] == t["l0.mix.w1"].shape[0]
    assert spec.layers[0].parts["mixer_norm"]["groups"] == 3 and spec.final_norm["groups"] == 3
    a1, a3 = spec.layers[1].parts["mixer"], spec.layers[3].parts["mixer"]
    assert (a1["window"], a1["temp_coef"], a1["temp_every"], a1["v_dim"], a1["kv_heads"]) == (37, 0.7, 16, 12, 2)
    assert (a3["window"], a3["temp_every"], a3["v_dim"]) == (64, None, 24)
    names = {n.name: tuple(n.shape) for n in tensor_needs_of_spec(spec)}
    assert names == {k: tuple(v.shape) for k, v in t.items()}
    assert "l3.norm2" not in names and names["loop.step"] == (2, 72) and names["l1.mix.q.norm"] == (20,)
    needs = [cache_need_of_layer(spec.layers[e.layer]) for e in spec.run_order]
    assert [n.kind for n in needs] == ["state", "kv", "state", "kv", "state", "kv", "state"]
    assert needs[0].state_shape == (5 * 10 * 10 + 72,) and needs[2].state_shape == (3 * 24 * 24 + 72,)
    _, cache = step_bytes_of_spec(spec)
    assert cache == 2 * (2 * (2 * (20 + 12))) + 2 * (4 * (16 + 24))      # layer 1 keeps keys and values once per pass


def test_what_a_configuration_may_leave_out():
    d = H.CONFIGS["plain"]()
    spec = config_from_dict(d).with_tensor_shapes(shapes_of(d)).to_spec()
    a = spec.layers[1].parts["mixer"]
    assert (a["kv_heads"], a["v_dim"], a["window"], a["temp_every"]) == (4, 16, None, None)
    assert spec.layers[2].parts["mixer"]["decay_rank"] == 6 and spec.layers[0].parts["mixer"]["decay_rank"] == 5
    assert all(e.before is None for e in spec.run_order) and "loop.step" not in {n.name for n in tensor_needs_of_spec(spec)}
    bare = {k: v for k, v in d.items() if k != "embedding"}
    bare["norm"] = {"eps": 1e-5}
    c = config_from_dict(bare)
    assert c.embedding_scale == 1.0 and c.norm_groups == 1


def test_states_start_at_zero_and_slots_are_used_again():
    from x0ne_engine_b200.cache import SequenceCache
    d = H.CONFIGS["mixed"]()
    spec = config_from_dict(d).with_tensor_shapes(shapes_of(d)).to_spec()
    needs = [cache_need_of_layer(spec.layers[e.layer]) for e in spec.run_order]
    cache = SequenceCache(needs, [None] * len(needs), 512, 512, torch.float32, "cpu", max_slots=3)
    assert sorted(cache.states) == [0, 2, 4, 6] and len(cache.groups) == 2
    assert sorted(g.entries for g in cache.groups) == [[1, 3], [5]]          # the two passes of layer 1 share a pool, not pages
    assert cache.state(2).data_ptr() != cache.state(4).data_ptr()             # one state per pass through the stretch
    a = cache.acquire(100)
    cache.state(2)[a] += 3.0
    cache.state(6)[a] += 1.0
    cache.release(a)
    b = cache.acquire(10)
    assert b == a and float(cache.state(2)[b].abs().max()) == 0.0 and float(cache.state(6)[b].abs().max()) == 0.0


# ---- the plain implementation itself
def test_plain_group_norm_and_unit_values():
    x = torch.tensor([[3.0, 4.0, 0.0, 0.0, 30.0, 40.0]], dtype=torch.float64)
    y = P.group_norm(x, torch.ones(6, dtype=torch.float64), 1e-30, 3)
    assert torch.allclose(y[0, :2], torch.tensor([3.0, 4.0], dtype=torch.float64) / (12.5 ** 0.5)) and torch.equal(y[0, 2:4], torch.zeros(2, dtype=torch.float64))
    assert torch.allclose(y[0, 4:], y[0, :2])
    assert torch.allclose(P.group_norm(x, torch.ones(6, dtype=torch.float64), 1.0, 1), x / ((2500 + 25) / 6 + 1.0) ** 0.5)


def test_plain_window_temperature_and_slopes():
    m = P.window_mask(8, 3)
    assert m[7].tolist() == [False] * 5 + [True] * 3 and m[1].tolist() == [True, True] + [False] * 6
    assert P.window_mask(4, None).tolist() == torch.tril(torch.ones(4, 4, dtype=torch.bool)).tolist()
    f = P.query_temperature(torch.tensor([0, 14, 15, 30, 31, 47]), 0.5, 16)
    assert torch.allclose(f, 1 + 0.5 * torch.log(torch.tensor([1.0, 1.0, 2.0, 2.0, 3.0, 4.0], dtype=torch.float64)))
    s = P.slopes(4)
    assert torch.allclose(s, torch.tensor([0.25, 0.0625, 0.015625, 0.00390625], dtype=torch.float64))
    assert abs(float(P.slopes(6)[0]) - 2 ** (-8 / 6)) < 1e-12


def test_plain_activation_is_smooth_at_zero():
    z = torch.tensor([-1e-6, 0.0, 1e-6, 2.0, -2.0], dtype=torch.float64)
    y = P.xielu(z, 0.3, -0.4)
    assert abs(float(y[1])) == 0.0 and abs(float(y[2] - y[0]) / 2e-6 - 0.5) < 1e-5
    sp = lambda a: float(np.log1p(np.exp(a)))
    assert abs(float(y[3]) - (sp(0.3) * 4 + 1.0)) < 1e-12
    assert abs(float(y[4]) - ((0.5 + sp(-0.4)) * (np.exp(-2.0) - 1 + 2.0) - 1.0)) < 1e-12


def test_plain_scan_by_its_closed_form_and_in_pieces():
    """o_t = sum_{s<t} (r_t * prod_{s<q<t} w_q * k_s) . v_s + (r_t * u * k_t) . v_t, and a sequence run in two calls
    through a kept state equals one call."""
    g = torch.Generator().manual_seed(0)
    T, Hh, N = 9, 2, 5
    r, k, v = (torch.randn(T, Hh, N, generator=g, dtype=torch.float64) for _ in range(3))
    w = torch.rand(T, Hh, N, generator=g, dtype=torch.float64)
    u = torch.randn(Hh, N, generator=g, dtype=torch.float64)
    S = torch.zeros(Hh, N, N, dtype=torch.float64)
    got = P.wkv_scan(r, k, v, w, u, S)
    for t in range(T):
        want = torch.einsum("hi,hj->hj", r[t] * u * k[t], v[t])
        for s in range(t):
            want = want + torch.einsum("hi,hj->hj", r[t] * w[s + 1:t].prod(0) * k[s], v[s])
        assert torch.allclose(got[t], want, atol=1e-12)
    S2 = torch.zeros(Hh, N, N, dtype=torch.float64)
    first = P.wkv_scan(r[:4], k[:4], v[:4], w[:4], u, S2)
    second = P.wkv_scan(r[4:], k[4:], v[4:], w[4:], u, S2)
    assert torch.allclose(torch.cat([first, second]), got, atol=1e-12) and torch.allclose(S, S2, atol=1e-12)


def test_plain_model_in_pieces_through_its_states():
    d = H.CONFIGS["mixed"]()
    t = H.make_tensors(d, 2)
    ids = H.clear_ids(d, t, 50, 1)
    want = P.forward(d, t, ids)
    states = [{} for _ in P.run_order(d)]
    parts = [P.forward(d, t, ids[:20], states=states, start=0), P.forward(d, t, ids[20:21], states=states, start=20),
             P.forward(d, t, ids[21:], states=states, start=21)]
    assert torch.allclose(torch.cat(parts), want, atol=1e-9)


def test_plain_router_takes_the_largest_logits_and_weighs_them_alone():
    z = torch.tensor([[1.0, 3.0, 2.0, 3.0, -1.0]], dtype=torch.float64)
    idx, wt = P.choose(z, 3)
    assert idx[0].tolist() == [1, 3, 2]
    assert torch.allclose(wt[0], torch.softmax(torch.tensor([3.0, 3.0, 2.0], dtype=torch.float64), -1)) and abs(float(wt.sum()) - 1) < 1e-12
