"""Dense feed-forwards: SiLU-gated units, and a two-product unit with biases."""
from __future__ import annotations

import math
from typing import List, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorNeed
from .base import FEED_FORWARDS, FeedForward
from .linear import Linear


class SwiGLU(FeedForward):
    """down( silu(gate x) * up x ): one product on the packed [gate; up] weight (gate rows, then
    up rows: x0ne-core/runtime/src/weights.rs:218-219), the activation
    g / (1 + expf(-g)) * u (x0ne-core/kernels/cuda/swiglu.cu:5-11), one product with down.
    Parameters: hidden_size, intermediate_size, names.{gate, up, down}."""
    replayable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        self.gate_up = None
        self.down = None

    @staticmethod
    def tensor_needs(spec: PartSpec) -> List[TensorNeed]:
        h, i, n = int(spec["hidden_size"]), int(spec["intermediate_size"]), spec["names"]
        return [TensorNeed(n["gate"], (i, h)), TensorNeed(n["up"], (i, h)), TensorNeed(n["down"], (h, i))]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.spec["names"]
        self.gate_up = Linear(torch.cat([tensors[n["gate"]], tensors[n["up"]]], dim=0).contiguous())
        self.down = Linear(tensors[n["down"]])

    def weight_bytes(self) -> int:
        return self.gate_up.weight_bytes() + self.down.weight_bytes()

    def forward(self, ctx, x, n_rows):
        gu = ctx.ws.buffer("ffn.gate_up", (ctx.ws.max_rows, 2 * self.inter), self.env.dtype)
        act = ctx.ws.buffer("ffn.act", (ctx.ws.max_rows, self.inter), self.env.dtype)
        out = ctx.ws.buffer(self.out_buffer, (ctx.ws.max_rows, self.hidden), self.env.dtype)
        kernel = ops.product_kernel(self.gate_up.weight, n_rows, fused=True)       # the routing table (csrc/routes.py)
        if kernel == "skinny":
            ops.gemm_bf16_skinny_tcgen05(x, self.gate_up.weight, act, n_rows, swiglu=True)   # 9 to 64 rows, tcgen05
        elif kernel == "smallm":
            ops.gemm_bf16_smallm(x, self.gate_up.weight, act, n_rows, swiglu=True)     # activation in the epilogue
        elif kernel == "tc_pair":
            ops.gemm_bf16_tcgen05(x, self.gate_up.weight, act, n_rows, swiglu=True)    # tcgen05, activation in the epilogue
        else:
            self.gate_up(x, gu, n_rows)
            ops.swiglu(gu, act, n_rows)
        self.down(act, out, n_rows)
        return out


class ClippedGLU(SwiGLU):
    """down( g sigmoid(slope g) (u + shift) ) with g = min(gate x, limit) and u = clamp(up x, -limit,
    limit): a gated unit whose gate is bounded above and whose linear branch is bounded on both sides
    and shifted.  One product on the packed [gate; up] weight, the activation in float32 (in the
    product's epilogue wherever SwiGLU's is: the same routing table decides), one product with down.
    Parameters: hidden_size, intermediate_size, limit, slope, shift, names.{gate, up, down}."""
    replayable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.limit = float(spec["limit"])
        self.slope = float(spec.get("slope", 1.0))
        self.shift = float(spec.get("shift", 0.0))

    def forward(self, ctx, x, n_rows):
        gu = ctx.ws.buffer("ffn.gate_up", (ctx.ws.max_rows, 2 * self.inter), self.env.dtype)
        act = ctx.ws.buffer("ffn.act", (ctx.ws.max_rows, self.inter), self.env.dtype)
        out = ctx.ws.buffer(self.out_buffer, (ctx.ws.max_rows, self.hidden), self.env.dtype)
        glu = (self.limit, self.slope, self.shift)
        kernel = ops.product_kernel(self.gate_up.weight, n_rows, fused=True) if self.env.dtype == torch.bfloat16 else "library"
        if kernel == "skinny":
            ops.gemm_bf16_skinny_tcgen05(x, self.gate_up.weight, act, n_rows, swiglu=True, glu=glu)
        elif kernel == "smallm":
            ops.gemm_bf16_smallm(x, self.gate_up.weight, act, n_rows, swiglu=True, glu=glu)
        elif kernel == "tc_pair":
            ops.gemm_bf16_tcgen05(x, self.gate_up.weight, act, n_rows, swiglu=True, glu=glu)
        else:
            self.gate_up(x, gu, n_rows)
            ops.glu_clipped(gu, act, n_rows, self.limit, self.slope, self.shift)
        self.down(act, out, n_rows)
        return out


def _softplus(x: float) -> float:
    return x + math.log1p(math.exp(-x)) if x > 0 else math.log1p(math.exp(x))


class BiasedMLP(FeedForward):
    """down(act(up x + b_up)) + b_down: two products with biases and no gate.  Activation "quad_exp": with the two
    stored numbers p, q of `act`,  z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2
    (slope 1/2 at zero from both sides); the two coefficients are worked out once at bind, in double precision.  Bias
    and activation are float32 inside, in one kernel behind the product.
    Parameters: hidden_size, intermediate_size, activation ("quad_exp"), names.{up, up_bias, down, down_bias, act}."""
    replayable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        if spec.get("activation", "quad_exp") != "quad_exp":
            raise ValueError(f"activation {spec.get('activation')!r} is not served by this feed-forward; served: 'quad_exp'")
        self.up = self.down = self.up_bias = self.down_bias = None
        self.a = self.b = 0.0

    @staticmethod
    def tensor_needs(spec: PartSpec) -> List[TensorNeed]:
        h, i, n = int(spec["hidden_size"]), int(spec["intermediate_size"]), spec["names"]
        return [TensorNeed(n["up"], (i, h)), TensorNeed(n["up_bias"], (i,), role="vector", init="linear"),
                TensorNeed(n["down"], (h, i)), TensorNeed(n["down_bias"], (h,), role="vector", init="linear"),
                TensorNeed(n["act"], (2,), role="vector", init="linear")]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.spec["names"]
        self.up, self.down = Linear(tensors[n["up"]]), Linear(tensors[n["down"]])
        self.up_bias, self.down_bias = tensors[n["up_bias"]], tensors[n["down_bias"]]
        p, q = (float(v) for v in tensors[n["act"]].detach().to("cpu", torch.float64))
        self.a, self.b = _softplus(p), 0.5 + _softplus(q)

    def weight_bytes(self) -> int:
        return self.up.weight_bytes() + self.down.weight_bytes()

    def forward(self, ctx, x, n_rows):
        z = ctx.ws.buffer("ffn.act", (ctx.ws.max_rows, self.inter), self.env.dtype)
        out = ctx.ws.buffer(self.out_buffer, (ctx.ws.max_rows, self.hidden), self.env.dtype)
        self.up(x, z, n_rows)
        ops.bias_act(z, self.up_bias, z, n_rows, ops.ACT_QUAD_EXP, self.a, self.b)
        self.down(z, out, n_rows)
        ops.bias_act(out, self.down_bias, out, n_rows)
        return out


FEED_FORWARDS.register("swiglu", SwiGLU)
FEED_FORWARDS.register("biased_mlp", BiasedMLP)
FEED_FORWARDS.register("clipped_glu", ClippedGLU)
