"""RMSNorm with the residual add fused in front of it."""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorNeed
from .base import NORMS, Norm


class PostNormed:
    """A sublayer's result that is still to be normed by `norm` (an RMSNorm of its own) before it joins the
    residual: what a layer with norms after its sublayers hands to the next add.  The norm that takes it
    norms the delta in float32, adds it, and norms the sum, in one launch."""
    __slots__ = ("delta", "norm")

    def __init__(self, delta: torch.Tensor, norm: "RMSNorm"):
        self.delta = delta
        self.norm = norm


class RMSNorm(Norm):
    """out = r * rsqrt(mean(r^2) + eps) * w with r = resid + delta, in float32; eps inside the
    root, the weight multiplies directly (x0ne-core/kernels/cuda/rmsnorm.cu:11-20).
    With `groups` > 1 the row is that many equal consecutive parts and each is divided by its own root mean square;
    the weight still has one value per value of the row.
    Parameters: size, eps, groups (default 1), names.weight."""
    replayable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.groups = int(spec.get("groups") or 1)
        if self.groups < 1 or self.size % self.groups:
            raise ValueError(f"a norm over {self.size} values cannot have {self.groups} equal groups")
        self.weight = None

    @staticmethod
    def tensor_needs(spec: PartSpec) -> List[TensorNeed]:
        return [TensorNeed(spec["names"]["weight"], (int(spec["size"]),), role="vector", init="norm")]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.spec["names"]["weight"]]

    def add_norm(self, ctx, resid, delta, out, n_rows, rows=None):
        if isinstance(delta, PostNormed):
            if self.groups != 1 or delta.norm.groups != 1:
                raise ValueError("a norm in groups does not take a result that is still to be normed")
            ops.add_normed_rmsnorm(resid, delta.delta, delta.norm.weight, delta.norm.eps, self.weight, out, n_rows, self.eps, rows)
        else:
            ops.add_rmsnorm(resid, delta, self.weight, out, n_rows, self.eps, rows, groups=self.groups)


NORMS.register("rmsnorm", RMSNorm)
