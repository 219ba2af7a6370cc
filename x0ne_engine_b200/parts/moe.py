"""Routed feed-forward: a router picks a few small experts per row; a shared expert may run beside them."""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorNeed
from .base import FEED_FORWARDS, FeedForward
from .linear import Linear
from .mlp import SwiGLU


class RoutedExperts(FeedForward):
    """out = sum over the row's chosen experts of weight_e expert_e(x)  (+ sigmoid(w_g . x) shared(x)).

    Router: float32 logits z = x W_r^T over `experts` + `identity` outputs; scores s = softmax(z); the
    choice is made on s + correction: the outputs form `groups` equal groups of neighbours, a group
    is worth its largest such value, only the `keep_groups` best groups can give experts, and of
    those the `top` largest values are chosen; the weights are the chosen outputs' scores s, not
    renormalized.  With `choice` "logits" there is no softmax over all outputs: the `top` largest z + correction (the
    correction is then the router's bias) are chosen and the weights are the softmax over the chosen values alone.
    With `choice` "sigmoid" the scores are s = sigmoid(z), each output by itself; the choice is made on s (+ correction,
    if the model has one) and the weights are the chosen scores.  For every kind of choice a group may be worth the sum
    of its `group_top` largest values instead of the largest one, and with `normalize` the chosen weights are divided
    by their sum (+ 1e-20) and multiplied by `weight_scale`.
    An expert is down(act(up x)) with act the squared ReLU, or, with `activation` "swiglu",
    down(silu(gate x) * up x) (gate and up packed per expert, gate rows first); no biases.  The last
    `identity` router outputs are identity experts: they return x itself and have no tensors.  The
    shared expert has the same form with a width of its own, runs for every row, and is multiplied
    by the sigmoid of one more projection of x (`shared_gate`; without it the shared expert is added as it is).  Beside
    gated experts the shared expert is gated too (names.shared_gate_proj is its gate matrix).

    One product gives the router logits and the shared gate's logit (float32); a kernel makes the
    choice; the (row, choice) pairs are listed expert by expert on the device and both products of the
    experts run over tiles of one expert's pairs (`ops.moe_product`), so the host never learns who
    chose what and the launches replay from a graph.  The sum is taken in float32 in the order of
    the choices.

    Parameters: hidden_size, experts, identity, top, groups, keep_groups, expert_size, activation
    ("relu2" | "swiglu"), choice ("scores" | "logits" | "sigmoid"), group_top (default 1), normalize, weight_scale,
    shared_size (None: no shared expert), shared_gate, names.{router, correction (may be absent with "sigmoid"), gate,
    up, down (patterns with {e}), shared_up, shared_down, shared_gate, shared_gate_proj}.
    """
    replayable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        g = spec.get
        self.hidden = int(spec["hidden_size"])
        self.experts = int(spec["experts"])
        self.identity = int(g("identity") or 0)
        self.n_out = self.experts + self.identity
        self.top = int(spec["top"])
        self.groups = int(g("groups") or 1)
        self.keep_groups = int(g("keep_groups") or self.groups)
        self.inter = int(spec["expert_size"])
        self.shared_size = int(g("shared_size") or 0)
        self.shared_gate = bool(g("shared_gate")) and self.shared_size > 0
        self.activation = g("activation", "relu2") or "relu2"
        if self.activation not in ("relu2", "swiglu"):
            raise ValueError(f"expert activation {self.activation!r} is not served; served: 'relu2', 'swiglu'")
        self.gated = self.activation == "swiglu"
        self.pair_block = 0
        self.choice = g("choice", "scores") or "scores"
        if self.choice not in ("scores", "logits", "sigmoid"):
            raise ValueError(f"router choice {self.choice!r} is not served; served: 'scores', 'logits', 'sigmoid'")
        self.group_top = int(g("group_top") or 1)
        self.normalize = bool(g("normalize"))
        self.weight_scale = float(g("weight_scale", 1.0) if g("weight_scale") is not None else 1.0)
        self.has_correction = spec["names"].get("correction") is not None
        if not self.has_correction and self.choice != "sigmoid":
            raise ValueError("only a router that scores with the sigmoid goes without a correction")
        if self.group_top < 1:
            raise ValueError("a group is worth the sum of at least one of its values")
        self.shared_glu = None
        if self.gated and self.shared_size:
            if self.shared_gate:
                raise ValueError("a gate on the shared expert beside gated experts is not served")
            n = spec["names"]
            self.shared_glu = SwiGLU(PartSpec("swiglu", dict(hidden_size=self.hidden, intermediate_size=self.shared_size,
                                                            names=dict(gate=n["shared_gate_proj"], up=n["shared_up"], down=n["shared_down"]))), env)
            self.shared_glu.out_buffer = "moe.shared_out"
        if self.n_out % self.groups or not 1 <= self.keep_groups <= self.groups or \
                not 1 <= self.top <= self.keep_groups * (self.n_out // self.groups):
            raise ValueError(f"{self.n_out} router outputs in {self.groups} groups of which {self.keep_groups} stay cannot "
                             f"give {self.top} choices")
        self.router = self.correction = self.up = self.down = self.shared_up = self.shared_down = None

    @staticmethod
    def tensor_needs(spec: PartSpec) -> List[TensorNeed]:
        h, n = int(spec["hidden_size"]), spec["names"]
        E, I, ff = int(spec["experts"]), int(spec.get("identity") or 0), int(spec["expert_size"])
        needs = []
        gated = (spec.get("activation") or "relu2") == "swiglu"
        for e in range(E):
            if gated:
                needs.append(TensorNeed(n["gate"].format(e=e), (ff, h)))
            needs += [TensorNeed(n["up"].format(e=e), (ff, h)), TensorNeed(n["down"].format(e=e), (h, ff))]
        needs.append(TensorNeed(n["router"], (E + I, h)))
        if n.get("correction") is not None:
            needs.append(TensorNeed(n["correction"], (E + I,), role="vector", init="linear"))
        sf = int(spec.get("shared_size") or 0)
        if sf and gated:
            needs += [TensorNeed(n["shared_gate_proj"], (sf, h)), TensorNeed(n["shared_up"], (sf, h)), TensorNeed(n["shared_down"], (h, sf))]
        elif sf:
            needs += [TensorNeed(n["shared_up"], (sf, h)), TensorNeed(n["shared_down"], (h, sf))]
            if spec.get("shared_gate"):
                needs.append(TensorNeed(n["shared_gate"], (1, h)))
        return needs

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.spec["names"]
        rows = [tensors[n["router"]]] + ([tensors[n["shared_gate"]]] if self.shared_gate else [])
        self.router = Linear(torch.cat(rows, dim=0).contiguous())
        self.correction = tensors[n["correction"]] if self.has_correction else None
        if self.gated:
            # [E, 2 ff, hidden]: an expert's gate rows, then its up rows; where ff is a multiple of MOE_PAIR_BLOCK, in blocks of that
            # many gate rows followed by the up rows of the same outputs, so that a tile of the tensor-core product holds both
            b = self.pair_block = ops.MOE_PAIR_BLOCK if self.inter % ops.MOE_PAIR_BLOCK == 0 else 0

            def packed(gate, up):
                if not b:
                    return torch.cat([gate, up], dim=0)
                return torch.cat([gate.reshape(-1, b, self.hidden), up.reshape(-1, b, self.hidden)], dim=1).reshape(2 * self.inter, self.hidden)
            self.up = torch.stack([packed(tensors[n["gate"].format(e=e)], tensors[n["up"].format(e=e)])
                                   for e in range(self.experts)]).contiguous()
        else:
            self.up = torch.stack([tensors[n["up"].format(e=e)] for e in range(self.experts)]).contiguous()   # [E, ff, hidden]
        self.down = torch.stack([tensors[n["down"].format(e=e)] for e in range(self.experts)]).contiguous()   # [E, hidden, ff]
        if self.shared_glu is not None:
            self.shared_glu.bind(tensors)
        elif self.shared_size:
            self.shared_up = Linear(tensors[n["shared_up"]])
            self.shared_down = Linear(tensors[n["shared_down"]])

    def weight_bytes(self) -> int:
        """The router, the shared expert and every expert: what a step of a batch large enough to reach all experts
        reads (a small batch reads at most rows x top of them)."""
        total = self.router.weight_bytes() + (self.up.numel() + self.down.numel()) * self.up.element_size()
        if self.shared_glu is not None:
            total += self.shared_glu.weight_bytes()
        elif self.shared_size:
            total += self.shared_up.weight_bytes() + self.shared_down.weight_bytes()
        return total

    def forward(self, ctx, x, n_rows):
        dt, rows, top = self.env.dtype, ctx.ws.max_rows, self.top
        ws = ctx.ws
        z = ws.buffer("moe.logits", (rows, self.router.out_features), torch.float32)
        chosen = ws.buffer("moe.chosen", (rows, top), torch.int32)
        weights = ws.buffer("moe.weights", (rows, top), torch.float32)
        sgate = ws.buffer("moe.shared_gate", (rows,), torch.float32) if self.shared_gate else None
        offsets = ws.buffer("moe.offsets", (self.experts + 1,), torch.int32)
        listed = ws.buffer("moe.listed", (rows * top,), torch.int32)
        tiles = ws.buffer("moe.tiles", (ops.moe_max_tiles(rows * top, self.experts), 3), torch.int32)
        n_real = ws.buffer("moe.n_tiles", (1,), torch.int32)
        act = ws.buffer("moe.act", (rows * top, self.inter), dt)
        y = ws.buffer("moe.y", (rows * top, self.hidden), torch.float32)
        out = ws.buffer(self.out_buffer, (rows, self.hidden), dt)
        self.router(x, z, n_rows)
        ops.moe_route(z, self.correction, self.n_out, self.groups, self.keep_groups, top, n_rows, chosen, weights, sgate, self.n_out,
                      on_logits=self.choice == "logits", sigmoid=self.choice == "sigmoid", group_top=self.group_top,
                      normalize=self.normalize, weight_scale=self.weight_scale)
        pairs = n_rows * top
        up_kind = 2 if self.gated else 0
        if (not self.gated or self.pair_block) and ops.moe_tc_takes(dt, pairs, self.hidden, self.inter):
            # many pairs: tiles of 128 listed pairs on the tensor cores; the rows are gathered into the listed order first,
            # the activations stay in that order, the down product writes by pair
            n_tiles = ops.moe_max_tiles(pairs, self.experts, ops.MOE_TC_TILE_ROWS)
            xs = ws.buffer("moe.gathered", (rows * top, self.hidden), dt)
            ops.moe_group(chosen, pairs, self.experts, offsets, listed, tiles[:n_tiles], ops.MOE_TC_TILE_ROWS, n_real)
            ops.moe_gather_rows(x, listed, offsets, self.experts, top, xs, pairs)
            ops.moe_product_tc(up_kind, xs, self.up, listed, tiles, n_real, n_tiles, act)
            ops.moe_product_tc(1, act, self.down, listed, tiles, n_real, n_tiles, y)
        else:
            n_tiles = ops.moe_max_tiles(pairs, self.experts)
            ops.moe_group(chosen, pairs, self.experts, offsets, listed, tiles[:n_tiles])
            ops.moe_product(up_kind, x, self.up, listed, tiles, n_tiles, top, act, self.pair_block)
            ops.moe_product(1, act, self.down, listed, tiles, n_tiles, top, y)
        shared = None
        if self.shared_glu is not None:
            shared = self.shared_glu.forward(ctx, x, n_rows)
        elif self.shared_size:
            su = ws.buffer("moe.shared_up", (rows, self.shared_size), dt)
            shared = ws.buffer("moe.shared_out", (rows, self.hidden), dt)
            self.shared_up(x, su, n_rows)
            ops.relu2(su, su, n_rows)
            self.shared_down(su, shared, n_rows)
        ops.moe_combine(y, x, chosen, weights, top, self.experts, shared, sgate, out, n_rows)
        return out


FEED_FORWARDS.register("routed_experts", RoutedExperts)
