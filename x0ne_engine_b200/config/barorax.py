"""Barorax: the typed configuration, read strictly from config.json, and its ModelSpec.

A Barorax model runs a list of pre-norm layers, `x += mixer(norm1(x))` then (unless the layer has no feed-forward)
`x += ff(norm2(x))`, every norm an RMS norm with a weight.  A stretch of the list (`loop.start` .. `loop.stop` - 1) runs
`loop.times` times in a row with the same weights and a cache or state of its own per pass; right before the first
layer of every pass, the first too, row t of `loop.step` is added to the residual.

The mixer of a layer is one of

  * `attention`: differential attention (`parts/diff_attention.py`): two softmax maps per head over the same values,
    the second taken off the first times a number of the layer; interleaved rotary pairs on the first `rot.dims` values
    of every map; a norm without a weight per head; a sigmoid gate on the concatenated heads;
  * `attention_2`: grouped-query attention over chunks of `mask.size` positions (`parts/masked_attention.py`): rotary
    pairs, then queries and keys brought to unit root mean square per head, and a softmax with one more term of score
    zero in its denominator;
  * `mamba1`: a selective state-space mixer (`parts/selective_scan.py`).

The feed-forward is a mixture of SiLU-gated experts: the router scores with the sigmoid, groups of neighbouring experts
are worth the sum of their two largest scores and only the best `groups.keep` groups give experts, the `top` largest
scores are chosen, and the weights are the chosen scores over their sum times `router.scale`; a shared expert of the
same form runs for every token.

Every size and constant comes from config.json (`layers[i].mixer`, `layers[i].mlp`, `loop`, `norm.eps`, `vocab`,
`width`).  Tensor names: `embed`, `loop.step`, `l<i>.norm1|norm2`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple

from .rovurax import UNBOUNDED_POSITIONS, _get, _num, _only, _pint, _plain
from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry

ARCHITECTURE = "Barorax"
MODEL_TYPE = "barorax"

# fixed by the design: a group of experts is worth the sum of this many of its largest scores
GROUP_TOP = 2

MIXERS = ("attention", "attention_2", "mamba1")


@dataclass(frozen=True)
class BaroraxLayer:
    type: str                       # one of MIXERS
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]


@dataclass(frozen=True)
class BaroraxLoop:
    start: int
    stop: int
    times: int


def _check_rot(mixer: Mapping[str, Any], where: str) -> None:
    rot = mixer.get("rot")
    if rot is None:
        return
    _only(rot, ("base", "dims"), where + ".rot")
    dims = _get(rot, "dims", where + ".rot")
    if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > mixer["dim"]:
        raise ConfigError(f"config.json: {where}.rot.dims is not an even count of at most dim = {mixer['dim']} values")
    _num(rot, "base", where + ".rot")


def _check_heads(mixer: Mapping[str, Any], where: str) -> None:
    _pint(mixer, "dim", where)
    heads = _pint(mixer, "heads", where)
    kv = _pint(mixer, "kv_heads", where) if mixer.get("kv_heads") is not None else heads
    if mixer.get("vdim") is not None:
        _pint(mixer, "vdim", where)
    _num(mixer, "scale", where)
    if heads % kv:
        raise ConfigError(f"config.json: {where}: heads are not a multiple of kv_heads")
    _check_rot(mixer, where)


@dataclass(frozen=True)
class BaroraxConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[BaroraxLayer, ...]
    loop: Optional[BaroraxLoop] = None
    dtype: str = "bfloat16"
    eos_token_ids: tuple = ()
    max_position_embeddings: int = UNBOUNDED_POSITIONS
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    # ---- reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "BaroraxConfig":
        if not isinstance(d, Mapping):
            raise ConfigError("config.json: not a JSON object")
        _only(d, ("architecture", "architectures", "model_type", "layers", "loop", "norm", "vocab", "width", "dtype", "eos_token_id"),
              "the model")
        norm = _get(d, "norm", "the model")
        _only(norm, ("eps",), "norm")
        width = _pint(d, "width", "the model")
        raw_layers = _get(d, "layers", "the model")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: layers is not a list of at least one layer")
        layers: List[BaroraxLayer] = []
        for i, l in enumerate(raw_layers):
            where = f"layers[{i}]"
            _only(l, ("type", "mixer", "mlp"), where)
            kind = _get(l, "type", where)
            mixer = _get(l, "mixer", where)
            mw = where + ".mixer"
            if kind == "mamba1":
                _only(mixer, ("conv", "dt_rank", "inner", "state"), mw)
                for key in ("conv", "dt_rank", "inner", "state"):
                    _pint(mixer, key, mw)
            elif kind == "attention":
                _only(mixer, ("diff", "dim", "heads", "kv_heads", "rot", "scale", "vdim"), mw)
                _check_heads(mixer, mw)
                _num(mixer, "diff", mw, positive=False)
            elif kind == "attention_2":
                _only(mixer, ("dim", "heads", "kv_heads", "mask", "rot", "scale", "vdim"), mw)
                _check_heads(mixer, mw)
                if mixer.get("mask") is not None:
                    _only(mixer["mask"], ("size",), mw + ".mask")
                    _pint(mixer["mask"], "size", mw + ".mask")
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this architecture; it has {list(MIXERS)}")
            mlp = l.get("mlp")
            if mlp is not None:
                cls._check_mlp(mlp, where + ".mlp")
            layers.append(BaroraxLayer(kind, mixer, mlp))
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            _only(lp, ("start", "stop", "times"), "loop")
            start, stop, times = _get(lp, "start", "loop"), _pint(lp, "stop", "loop"), _pint(lp, "times", "loop")
            if isinstance(start, bool) or not isinstance(start, int) or not 0 <= start < stop <= len(layers):
                raise ConfigError(f"config.json: loop runs layers {start!r} .. {stop} - 1 of {len(layers)}")
            loop = BaroraxLoop(start, stop, times)
        dtype = d.get("dtype") or "bfloat16"
        if dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"config.json: dtype {dtype!r}; bfloat16 and float32 checkpoints are served")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(vocab=_pint(d, "vocab", "the model"), width=width, norm_eps=_num(norm, "eps", "norm"), layers=tuple(layers),
                   loop=loop, dtype=dtype, eos_token_ids=eos_ids, raw=dict(d))

    @staticmethod
    def _check_mlp(mlp: Mapping[str, Any], where: str) -> None:
        kind = _get(mlp, "kind", where)
        if kind != "moe":
            raise ConfigError(f"config.json: {where}.kind {kind!r} is not a feed-forward of this architecture; it has 'moe'")
        _only(mlp, ("kind", "expert", "router", "shared"), where)
        expert = _get(mlp, "expert", where)
        _only(expert, ("ff",), where + ".expert")
        _pint(expert, "ff", where + ".expert")
        router = _get(mlp, "router", where)
        rw = where + ".router"
        _only(router, ("experts", "groups", "scale", "top"), rw)
        experts, top = _pint(router, "experts", rw), _pint(router, "top", rw)
        if router.get("scale") is not None:
            _num(router, "scale", rw)
        count = keep = 1
        if router.get("groups") is not None:
            _only(router["groups"], ("count", "keep"), rw + ".groups")
            count = _pint(router["groups"], "count", rw + ".groups")
            keep = _pint(router["groups"], "keep", rw + ".groups") if router["groups"].get("keep") is not None else count
        if experts % count or keep > count or top > keep * (experts // count):
            raise ConfigError(f"config.json: {rw}: {experts} experts in {count} groups of which {keep} stay cannot give {top} choices")
        if mlp.get("shared") is not None:
            _only(mlp["shared"], ("ff",), where + ".shared")
            _pint(mlp["shared"], "ff", where + ".shared")

    def to_dict(self) -> dict:
        """The config.json this configuration is read back from."""
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "layers": [{"type": l.type, "mixer": _plain(l.mixer), "mlp": _plain(l.mlp)} for l in self.layers]}
        if self.loop is not None:
            d["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if self.dtype != "bfloat16":
            d["dtype"] = self.dtype
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ---- the model as data
    def run_layers(self) -> List[Tuple[int, Optional[int]]]:
        """(layer, number of the pass it opens or None) for every layer run, in order."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        lp = self.loop
        order: List[Tuple[int, Optional[int]]] = [(i, None) for i in range(lp.start)]
        for t in range(lp.times):
            order += [(i, t if i == lp.start else None) for i in range(lp.start, lp.stop)]
        return order + [(i, None) for i in range(lp.stop, n)]

    def to_spec(self) -> ModelSpec:
        w, eps = self.width, self.norm_eps

        def norm(name: str) -> PartSpec:
            return PartSpec("rmsnorm", dict(size=w, eps=eps, names=dict(weight=name)))

        positions: Dict[str, PartSpec] = {}

        def position(m: Mapping[str, Any]) -> Optional[str]:
            """The name of the rotary encoding a mixer's `rot` asks for; mixers with the same constants share one."""
            rot = m.get("rot")
            if rot is None or not rot["dims"]:
                return None
            name = f"rot{rot['dims']}@{float(rot['base'])!r}"
            positions.setdefault(name, PartSpec("yarn_rope", dict(rotary_dim=rot["dims"], theta=float(rot["base"]), scaling=None,
                                                                   layout="interleaved", angle_in_float32=True)))
            return name

        layers = []
        for i, l in enumerate(self.layers):
            p, m = f"l{i}", l.mixer
            if l.type == "mamba1":
                mixer = PartSpec("selective_scan", dict(
                    hidden_size=w, inner=m["inner"], state=m["state"], conv=m["conv"], dt_rank=m["dt_rank"],
                    names=dict(**{"in": f"{p}.mix.in"}, conv=f"{p}.mix.conv", conv_bias=f"{p}.mix.conv.b", x=f"{p}.mix.x",
                               dt=f"{p}.mix.dt", dt_bias=f"{p}.mix.dt.b", A_log=f"{p}.mix.A_log", D=f"{p}.mix.D", o=f"{p}.mix.o")))
            elif l.type == "attention":
                mixer = PartSpec("differential_attention", dict(
                    hidden_size=w, q_heads=m["heads"], kv_heads=m.get("kv_heads") or m["heads"], head_dim=m["dim"],
                    v_dim=m.get("vdim") or m["dim"], scale=float(m["scale"]), lambda_init=float(m["diff"]), eps=eps,
                    position=position(m), gate=True,
                    names=dict(q=f"{p}.mix.q", k=f"{p}.mix.k", v=f"{p}.mix.v", g=f"{p}.mix.g", o=f"{p}.mix.o",
                               lq1=f"{p}.mix.lq1", lk1=f"{p}.mix.lk1", lq2=f"{p}.mix.lq2", lk2=f"{p}.mix.lk2")))
            else:
                mixer = PartSpec("masked_attention", dict(
                    hidden_size=w, q_heads=m["heads"], kv_heads=m.get("kv_heads") or m["heads"], head_dim=m["dim"],
                    v_dim=m.get("vdim") or m["dim"], scale=float(m["scale"]), chunk=(m.get("mask") or {}).get("size"), window=None,
                    v_blend=None, position=position(m), qk_unit_eps=eps, sink_zero=True,
                    names=dict(q=f"{p}.mix.q", k=f"{p}.mix.k", v=f"{p}.mix.v", o=f"{p}.mix.o")))
            parts = dict(mixer_norm=norm(f"{p}.norm1"), mixer=mixer)
            if l.mlp is not None:
                r = l.mlp["router"]
                groups = r.get("groups") or {}
                count = groups.get("count", 1)
                shared = l.mlp.get("shared")
                parts["ffn_norm"] = norm(f"{p}.norm2")
                parts["ffn"] = PartSpec("routed_experts", dict(
                    hidden_size=w, experts=r["experts"], identity=0, top=r["top"], groups=count, keep_groups=groups.get("keep") or count,
                    expert_size=l.mlp["expert"]["ff"], activation="swiglu", choice="sigmoid", group_top=GROUP_TOP, normalize=True,
                    weight_scale=float(r["scale"]) if r.get("scale") is not None else 1.0,
                    shared_size=shared["ff"] if shared is not None else None, shared_gate=False,
                    names=dict(router=f"{p}.mlp.router", gate=f"{p}.mlp.e{{e}}.gate", up=f"{p}.mlp.e{{e}}.up", down=f"{p}.mlp.e{{e}}.down",
                               shared_gate_proj=f"{p}.mlp.shared.gate", shared_up=f"{p}.mlp.shared.up",
                               shared_down=f"{p}.mlp.shared.down")))
            layers.append(LayerSpec(block="prenorm" if l.mlp is not None else "prenorm_mixer", parts=parts))
        order = []
        for i, t in self.run_layers():
            before = None
            if t is not None:
                before = PartSpec("pass_opener", dict(hidden_size=w, vocab_size=self.vocab, scale=1.0, add_embedding=False, step_row=t,
                                                      step_rows=self.loop.times, names=dict(table="embed", step="loop.step")))
            order.append(RunEntry(i, before=before))
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=w,
            max_position_embeddings=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", dict(vocab_size=self.vocab, hidden_size=w, names=dict(weight="embed"))),
            positions=positions, layers=tuple(layers), run_order=tuple(order),
            final_norm=norm("final.norm"),
            head=PartSpec("lm_head", dict(vocab_size=self.vocab, hidden_size=w, tied=False, names=dict(weight="head"))),
            stop_token_ids=tuple(self.eos_token_ids), checkpoint_dtype=self.dtype)
        spec.validate()
        return spec
