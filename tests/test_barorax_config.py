"""Barorax on the CPU: the reader of config.json, its refusals, the model as data (parts, tensor names, run order, what
every layer run keeps per sequence), and properties of the plain implementation itself."""
import copy

import numpy as np
import pytest
import torch

import barorax_helpers as H
import barorax_plain as P
from x0ne_engine_b200.config import ConfigError, config_from_dict, detect
from x0ne_engine_b200.config.barorax import BaroraxConfig
from x0ne_engine_b200.engine.model import cache_need_of_layer, tensor_needs_of_spec


def test_config_is_read_and_written_back():
    for name, make in H.CONFIGS.items():
        d = make()
        assert detect(d) == "Barorax"
        c = config_from_dict(d)
        assert isinstance(c, BaroraxConfig) and c.to_dict() == d, name
        assert config_from_dict(c.to_dict()) == c


@pytest.mark.parametrize("change,word", [
    (lambda d: d["layers"][0]["mixer"].update(extra=1), "extra"),
    (lambda d: d["layers"][2]["mixer"]["mask"].update(left=1), "left"),
    (lambda d: d["layers"][1]["mixer"].update(heads=5), "multiple"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=14), "rot.dims"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda d: d["layers"][0].update(type="mamba2"), "mamba2"),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=5), "choices"),
    (lambda d: d["layers"][1]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda d: d["layers"][0]["mlp"].update(kind="glu"), "glu"),
    (lambda d: d["norm"].pop("eps"), "eps"),
    (lambda d: d["loop"].update(stop=9), "loop"),
    (lambda d: d["loop"].update(start=3), "loop"),
    (lambda d: d["loop"].update(times=0), "times"),
    (lambda d: d["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda d: d["layers"][1]["mixer"].pop("diff"), "diff"),
    (lambda d: d["layers"][0]["mixer"].update(state=0), "state"),
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
    assert [i for i, _ in c.run_layers()] == [0, 1, 2, 1, 2, 3] == [i for i, _ in P.run_order(d)]
    spec = c.to_spec()
    openers = [(k, e.before["add_embedding"], e.before["step_row"]) for k, e in enumerate(spec.run_order) if e.before is not None]
    assert openers == [(1, False, 0), (3, False, 1)]                        # the first pass gets its step vector too
    assert all(e.reads_cache_of is None for e in spec.run_order)           # every pass keeps a cache or state of its own
    even = config_from_dict(H.CONFIGS["even"]()).to_spec()
    assert [e.layer for e in even.run_order] == [0, 1, 0, 1, 0, 1, 2]
    assert [k for k, e in enumerate(even.run_order) if e.before is not None] == [0, 2, 4]
    once = config_from_dict(H.CONFIGS["wide"]()).to_spec()
    assert [e.before is not None for e in once.run_order] == [True, False, False]
    none = config_from_dict(H.CONFIGS["plain"]()).to_spec()
    assert all(e.before is None for e in none.run_order)


def test_tensor_names_and_shapes_are_the_checkpoints():
    for name, make in H.CONFIGS.items():
        d = make()
        needs = {n.name: tuple(n.shape) for n in tensor_needs_of_spec(config_from_dict(d).to_spec())}
        have = {k: tuple(v.shape) for k, v in H.make_tensors(d, 0).items()}
        assert needs == have, (name, sorted(set(needs) ^ set(have)))


def test_parts_carry_every_constant_of_the_layer():
    d = H.CONFIGS["mixed"]()
    spec = config_from_dict(d).to_spec()
    m = d["layers"][1]["mixer"]
    diff = spec.layers[1].part("mixer")
    assert diff.kind == "differential_attention" and diff["lambda_init"] == m["diff"] and diff["scale"] == m["scale"]
    assert (diff["q_heads"], diff["kv_heads"], diff["head_dim"], diff["v_dim"]) == (m["heads"], m["kv_heads"], m["dim"], m["vdim"])
    rot = spec.positions[diff["position"]]
    assert rot.kind == "yarn_rope" and rot["rotary_dim"] == m["rot"]["dims"] and rot["theta"] == m["rot"]["base"] and rot["layout"] == "interleaved"
    c = d["layers"][2]["mixer"]
    chunk = spec.layers[2].part("mixer")
    assert chunk.kind == "masked_attention" and chunk["chunk"] == c["mask"]["size"] and chunk["sink_zero"] and chunk["qk_unit_eps"] == d["norm"]["eps"]
    assert spec.positions[chunk["position"]]["rotary_dim"] == c["rot"]["dims"]
    s = spec.layers[0].part("mixer")
    assert s.kind == "selective_scan" and (s["inner"], s["state"], s["conv"], s["dt_rank"]) == (50, 6, 4, 5)
    r = d["layers"][1]["mlp"]["router"]
    ffn = spec.layers[1].part("ffn")
    assert ffn.kind == "routed_experts" and ffn["choice"] == "sigmoid" and ffn["group_top"] == 2 and ffn["normalize"]
    assert (ffn["experts"], ffn["top"], ffn["groups"], ffn["keep_groups"], ffn["weight_scale"]) == (8, 3, 4, 2, r["scale"])
    assert ffn["shared_size"] == 24 and spec.layers[3].part("ffn")["shared_size"] is None and spec.layers[3].part("ffn")["groups"] == 1
    assert spec.layers[2].block == "prenorm_mixer" and spec.layers[1].block == "prenorm"
    # layers whose rotations have the same constants share one table; others get their own
    assert len(config_from_dict(H.CONFIGS["served"]()).to_spec().positions) == 2
    assert config_from_dict(H.CONFIGS["plain"]()).to_spec().positions == {}


def test_what_a_layer_run_keeps():
    spec = config_from_dict(H.CONFIGS["mixed"]()).to_spec()
    needs = [cache_need_of_layer(l) for l in spec.layers]
    assert needs[0].kind == "state" and needs[0].state_shape == (50 * (6 + 3),)
    assert needs[1].kind == "kv" and (needs[1].kv_heads, needs[1].head_dim, needs[1].v_dim) == (2, 24, 20)      # two keys side by side
    assert needs[2].kind == "kv" and (needs[2].kv_heads, needs[2].head_dim, needs[2].v_dim, needs[2].window) == (2, 20, 12, None)
    assert needs[3].state_shape == (36 * (10 + 2),)


# ------------------------------------------------------------------------------------------ the plain implementation
def test_plain_rotation_turns_pairs_and_leaves_the_rest():
    x = torch.randn(5, 2, 10, dtype=torch.float64)
    pos = torch.tensor([0, 1, 2, 50, 1000])
    y = P.rotate_pairs(x, pos, 6, 100.0)
    assert torch.equal(y[..., 6:], x[..., 6:]) and torch.equal(y[0], x[0])
    # a rotation keeps each pair's length, and pair i at position p has turned by p * 100^(-2i/6)
    assert torch.allclose(y[..., 0:6:2] ** 2 + y[..., 1:6:2] ** 2, x[..., 0:6:2] ** 2 + x[..., 1:6:2] ** 2)
    a = 50 * 100.0 ** (-2 / 6)
    u, v = x[3, 1, 2], x[3, 1, 3]
    assert abs(float(y[3, 1, 2]) - float(u * np.cos(a) - v * np.sin(a))) < 1e-12 and abs(float(y[3, 1, 3]) - float(v * np.cos(a) + u * np.sin(a))) < 1e-12


def test_plain_chunks_and_sink():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(20, 2, 4, generator=g, dtype=torch.float64) for _ in range(3))
    pos = torch.arange(20)
    o = P.softmax_attention(q, k, v, 0.7, pos, chunk=8, sink_one=True)
    # position 8 opens a chunk: it sees itself alone, with the weight e^s / (1 + e^s)
    s = float((q[8, 0] * k[8, 0]).sum() * 0.7)
    assert torch.allclose(o[8, 0], v[8, 0] * (np.exp(s) / (1 + np.exp(s))))
    # position 7 closes the chunk before: it sees 0..7, and nothing changes for it when later keys change
    k2 = k.clone()
    k2[8:] += 1.0
    assert torch.equal(P.softmax_attention(q, k2, v, 0.7, pos, chunk=8, sink_one=True)[:8], o[:8])
    w = torch.softmax(torch.cat([(q[7, 1] @ k[:8, 1].T) * 0.7, torch.zeros(1, dtype=torch.float64)]), 0)[:8]
    assert torch.allclose(o[7, 1], w @ v[:8, 1])


def test_plain_router_groups_sum_their_two_largest():
    z = torch.logit(torch.tensor([[0.9, 0.1, 0.1, 0.6, 0.55, 0.5, 0.2, 0.2, 0.2]], dtype=torch.float64))
    # groups of three: worth 1.0, 1.15, 0.4; with one group kept the largest single score (0.9) is out of reach
    ch, w = P.route(z, 2, 3, 1, 2.0)
    assert sorted(ch[0].tolist()) == [3, 4] and torch.allclose(w.sum(), torch.tensor(2.0, dtype=torch.float64))
    assert torch.allclose(w[0].sort().values, torch.tensor([0.55, 0.6], dtype=torch.float64) / 1.15 * 2.0)
    ch, _ = P.route(z, 2, 3, 2, 1.0)
    assert sorted(ch[0].tolist()) == [0, 3]
    ch, _ = P.route(z, 3, 1, 1, 1.0)
    assert sorted(ch[0].tolist()) == [0, 3, 4]


def test_plain_scan_in_pieces_is_the_scan():
    cfg = H.CONFIGS["mamba_only"]()
    t = H.make_tensors(cfg, 1)
    ids = H.random_ids(cfg, 40, 3)
    whole = P.forward(cfg, t, ids)
    states, out, at = {}, [], 0
    for n in (1, 2, 17, 20):
        out.append(P.forward(cfg, t, ids[at:at + n], states=states, pos0=at))
        at += n
    assert torch.allclose(torch.cat(out), whole, rtol=0, atol=1e-10)


def test_plain_model_in_pieces_is_the_model():
    cfg = H.CONFIGS["mixed"]()
    t = H.make_tensors(cfg, 2)
    ids = H.random_ids(cfg, 50, 4)
    chosen = {}
    whole = P.forward(cfg, t, ids, record=chosen)
    states, kv, out, at = {}, {}, [], 0
    for n in (3, 1, 36, 10):
        forced = {run: c[0][at:at + n] for run, c in chosen.items()}
        out.append(P.forward(cfg, t, ids[at:at + n], states=states, kv=kv, pos0=at, chosen=forced))
        at += n
    assert torch.allclose(torch.cat(out), whole, rtol=0, atol=1e-9)
