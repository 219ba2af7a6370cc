"""Retuvik: the typed configuration, read strictly from config.json, and its ModelSpec.

A Retuvik model multiplies its token embedding by a constant and runs a list of pre-norm layers,
`x += mixer(norm1(x))` then (unless the layer has no feed-forward) `x += ff(norm2(x))`; every norm is an RMS norm
over `norm.groups` equal consecutive parts of the row.  A stretch of the list (`loop.start` .. `loop.stop` - 1) runs
`loop.times` times in a row with the same weights and a cache or state of its own per pass; right before the first
layer of a pass the embedding output is added again (not before the first pass) and then row t of `loop.step`.

The mixer of a layer is one of

  * `wkv`: a linear recurrence with a matrix state per head behind a token shift (`parts/recurrent.py`);
  * `attention`: grouped-query attention without rotation: per-head normed queries and keys, unit-norm values, a
    temperature on the queries that grows with the logarithm of the position, a per-head slope times the distance
    taken off every score, a sliding window, and a sigmoid gate on the concatenated heads (`parts/distance_attention.py`).

The feed-forward is dense with biases and an activation with a quadratic positive and an exponential negative branch,
or a mixture of SiLU-gated experts chosen by the largest router logits, weighted by the softmax over the chosen.

Every size and constant comes from config.json (`embedding.scale`, `layers[i].mixer`, `layers[i].mlp`, `loop`,
`norm.eps`, `norm.groups`, `vocab`, `width`); one size is given by a tensor's shape only: the inner width of the decay's
two small products (`l<i>.mix.w1` is [that width, model width]), which `with_tensor_shapes` fills in.  Tensor names:
`embed`, `loop.step`, `l<i>.norm1|norm2`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Any, List, Mapping, Optional, Tuple

from .rovurax import UNBOUNDED_POSITIONS, _get, _num, _only, _pint, _plain
from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry

ARCHITECTURE = "Retuvik"
MODEL_TYPE = "retuvik"

# fixed by the design: the slopes of the distance bias are 2^(-SLOPE_SPAN (h + 1) / heads)
SLOPE_SPAN = 8.0


@dataclass(frozen=True)
class RetuvikLayer:
    type: str                       # "wkv" | "attention"
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]


@dataclass(frozen=True)
class RetuvikLoop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class RetuvikConfig:
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    embedding_scale: float
    layers: Tuple[RetuvikLayer, ...]
    loop: Optional[RetuvikLoop] = None
    dtype: str = "bfloat16"
    eos_token_ids: tuple = ()
    max_position_embeddings: int = UNBOUNDED_POSITIONS
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    # ---- reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "RetuvikConfig":
        if not isinstance(d, Mapping):
            raise ConfigError("config.json: not a JSON object")
        norm = _get(d, "norm", "the model")
        _only(norm, ("eps", "groups"), "norm")
        groups = _pint(norm, "groups", "norm") if norm.get("groups") is not None else 1
        width = _pint(d, "width", "the model")
        if width % groups:
            raise ConfigError(f"config.json: width {width} does not split into norm.groups = {groups} equal parts")
        emb = d.get("embedding") or {}
        _only(emb, ("scale",), "embedding")
        scale = _num(emb, "scale", "embedding") if "scale" in emb else 1.0
        raw_layers = _get(d, "layers", "the model")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: layers is not a list of at least one layer")
        layers: List[RetuvikLayer] = []
        for i, l in enumerate(raw_layers):
            where = f"layers[{i}]"
            _only(l, ("type", "mixer", "mlp"), where)
            kind = _get(l, "type", where)
            mixer = _get(l, "mixer", where)
            mw = where + ".mixer"
            if kind == "wkv":
                _only(mixer, ("dim", "heads", "decay_rank"), mw)
                _pint(mixer, "dim", mw)
                _pint(mixer, "heads", mw)
                if mixer.get("decay_rank") is not None:
                    _pint(mixer, "decay_rank", mw)
            elif kind == "attention":
                _only(mixer, ("dim", "heads", "kv_heads", "mask", "q_temp", "scale", "vdim"), mw)
                _pint(mixer, "dim", mw)
                heads = _pint(mixer, "heads", mw)
                kv = _pint(mixer, "kv_heads", mw) if mixer.get("kv_heads") is not None else heads
                if mixer.get("vdim") is not None:
                    _pint(mixer, "vdim", mw)
                _num(mixer, "scale", mw)
                if heads % kv:
                    raise ConfigError(f"config.json: {mw}: heads are not a multiple of kv_heads")
                if mixer.get("mask") is not None:
                    _only(mixer["mask"], ("size",), mw + ".mask")
                    _pint(mixer["mask"], "size", mw + ".mask")
                if mixer.get("q_temp") is not None:
                    _only(mixer["q_temp"], ("coef", "every"), mw + ".q_temp")
                    _num(mixer["q_temp"], "coef", mw + ".q_temp", positive=False)
                    _pint(mixer["q_temp"], "every", mw + ".q_temp")
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this architecture")
            mlp = l.get("mlp")
            if mlp is not None:
                cls._check_mlp(mlp, where + ".mlp")
            layers.append(RetuvikLayer(kind, mixer, mlp))
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            _only(lp, ("start", "stop", "times"), "loop")
            start, stop, times = _get(lp, "start", "loop"), _pint(lp, "stop", "loop"), _pint(lp, "times", "loop")
            if isinstance(start, bool) or not isinstance(start, int) or not 0 <= start < stop <= len(layers):
                raise ConfigError(f"config.json: loop runs layers {start!r} .. {stop} - 1 of {len(layers)}")
            loop = RetuvikLoop(start, stop, times)
        dtype = d.get("dtype") or "bfloat16"
        if dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"config.json: dtype {dtype!r}; bfloat16 and float32 checkpoints are served")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(vocab=_pint(d, "vocab", "the model"), width=width, norm_eps=_num(norm, "eps", "norm"), norm_groups=groups,
                   embedding_scale=scale, layers=tuple(layers), loop=loop, dtype=dtype, eos_token_ids=eos_ids, raw=dict(d))

    @staticmethod
    def _check_mlp(mlp: Mapping[str, Any], where: str) -> None:
        kind = _get(mlp, "kind", where)
        if kind == "dense":
            _only(mlp, ("ff", "kind"), where)
            _pint(mlp, "ff", where)
            return
        if kind != "moe":
            raise ConfigError(f"config.json: {where}.kind {kind!r} is not a feed-forward of this architecture")
        _only(mlp, ("kind", "expert", "router"), where)
        expert = _get(mlp, "expert", where)
        _only(expert, ("ff",), where + ".expert")
        _pint(expert, "ff", where + ".expert")
        router = _get(mlp, "router", where)
        _only(router, ("experts", "top"), where + ".router")
        if _pint(router, "top", where + ".router") > _pint(router, "experts", where + ".router"):
            raise ConfigError(f"config.json: {where}.router chooses more experts than it has")

    # ---- sizes that only the checkpoint gives
    def needs_tensor_shapes(self) -> bool:
        return any(l.type == "wkv" and l.mixer.get("decay_rank") is None for l in self.layers)

    def with_tensor_shapes(self, shapes: Mapping[str, Tuple[int, ...]]) -> "RetuvikConfig":
        """A copy in which every recurrent layer knows the inner width of its decay's two products, taken from the
        first axis of `l<i>.mix.w1` where config.json does not give it."""
        layers = []
        for i, l in enumerate(self.layers):
            if l.type == "wkv" and l.mixer.get("decay_rank") is None:
                shape = shapes.get(f"l{i}.mix.w1")
                if shape is None or len(shape) != 2 or shape[0] <= 0:
                    raise ConfigError(f"the checkpoint has no matrix l{i}.mix.w1 to take layer {i}'s decay width from")
                l = RetuvikLayer(l.type, {**l.mixer, "decay_rank": int(shape[0])}, l.mlp)
            layers.append(l)
        return replace(self, layers=tuple(layers))

    def to_dict(self) -> dict:
        """The config.json this configuration is read back from."""
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "embedding": {"scale": self.embedding_scale},
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
        w, eps, groups = self.width, self.norm_eps, self.norm_groups

        def norm(name: str) -> PartSpec:
            return PartSpec("rmsnorm", dict(size=w, eps=eps, groups=groups, names=dict(weight=name)))

        layers = []
        for i, l in enumerate(self.layers):
            p, m = f"l{i}", l.mixer
            if l.type == "wkv":
                if m.get("decay_rank") is None:
                    raise ConfigError(f"layers[{i}].mixer: the decay's inner width is not known; it is the first axis of "
                                      f"{p}.mix.w1 (read the configuration from the model's folder, or give decay_rank)")
                mixer = PartSpec("matrix_state_recurrence", dict(
                    hidden_size=w, heads=m["heads"], head_dim=m["dim"], decay_rank=m["decay_rank"], eps=eps,
                    names=dict(mu=f"{p}.mix.mu.{{s}}", r=f"{p}.mix.r", k=f"{p}.mix.k", v=f"{p}.mix.v", g=f"{p}.mix.g",
                               w1=f"{p}.mix.w1", w2=f"{p}.mix.w2", w0=f"{p}.mix.w0", u=f"{p}.mix.u", norm=f"{p}.mix.norm",
                               o=f"{p}.mix.o")))
            else:
                qt = m.get("q_temp") or {}
                mixer = PartSpec("distance_bias_attention", dict(
                    hidden_size=w, q_heads=m["heads"], kv_heads=m.get("kv_heads") or m["heads"], head_dim=m["dim"],
                    v_dim=m.get("vdim") or m["dim"], scale=float(m["scale"]), window=(m.get("mask") or {}).get("size"),
                    qk_norm_eps=eps, temp_coef=qt.get("coef"), temp_every=qt.get("every"), v_unit=True, slope_span=SLOPE_SPAN,
                    gate=True,
                    names=dict(q=f"{p}.mix.q", k=f"{p}.mix.k", v=f"{p}.mix.v", g=f"{p}.mix.g", o=f"{p}.mix.o",
                               q_norm=f"{p}.mix.q.norm", k_norm=f"{p}.mix.k.norm")))
            parts = dict(mixer_norm=norm(f"{p}.norm1"), mixer=mixer)
            if l.mlp is not None:
                parts["ffn_norm"] = norm(f"{p}.norm2")
                if l.mlp["kind"] == "dense":
                    parts["ffn"] = PartSpec("biased_mlp", dict(
                        hidden_size=w, intermediate_size=l.mlp["ff"], activation="quad_exp",
                        names=dict(up=f"{p}.mlp.up", up_bias=f"{p}.mlp.up.b", down=f"{p}.mlp.down",
                                   down_bias=f"{p}.mlp.down.b", act=f"{p}.mlp.act")))
                else:
                    r = l.mlp["router"]
                    parts["ffn"] = PartSpec("routed_experts", dict(
                        hidden_size=w, experts=r["experts"], identity=0, top=r["top"], groups=1, keep_groups=1,
                        expert_size=l.mlp["expert"]["ff"], activation="swiglu", choice="logits",
                        names=dict(router=f"{p}.mlp.router", correction=f"{p}.mlp.router.b", gate=f"{p}.mlp.e{{e}}.gate",
                                   up=f"{p}.mlp.e{{e}}.up", down=f"{p}.mlp.e{{e}}.down")))
            layers.append(LayerSpec(block="prenorm" if l.mlp is not None else "prenorm_mixer", parts=parts))
        order = []
        for i, t in self.run_layers():
            before = None
            if t is not None:
                before = PartSpec("pass_opener", dict(
                    hidden_size=w, vocab_size=self.vocab, scale=self.embedding_scale, add_embedding=t > 0, step_row=t,
                    step_rows=self.loop.times, names=dict(table="embed", step="loop.step")))
            order.append(RunEntry(i, before=before))
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=w,
            max_position_embeddings=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", dict(vocab_size=self.vocab, hidden_size=w, scale=self.embedding_scale,
                                                       names=dict(weight="embed"))),
            positions={}, layers=tuple(layers), run_order=tuple(order),
            final_norm=norm("final.norm"),
            head=PartSpec("lm_head", dict(vocab_size=self.vocab, hidden_size=w, tied=False, names=dict(weight="head"))),
            stop_token_ids=tuple(self.eos_token_ids), checkpoint_dtype=self.dtype)
        spec.validate()
        return spec
