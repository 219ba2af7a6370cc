"""The two ends of the model: token embedding and the output head."""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorNeed
from .base import EMBEDDINGS, HEADS, OPENERS, Embedding, Head, Opener
from .linear import Linear


class TokenEmbedding(Embedding):
    """resid[r] = float32(table[token[r]]); an id outside the table gives a zero row
    (x0ne-core/kernels/cuda/embedding.cu:5-17).  With `scale` the row is multiplied by it in float32
    on its way into the residual.  Parameters: vocab_size, hidden_size, scale (default 1), names.weight."""
    replayable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.table = None
        self.scale = float(spec.get("scale", 1.0) or 1.0)

    @staticmethod
    def tensor_needs(spec: PartSpec) -> List[TensorNeed]:
        return [TensorNeed(spec["names"]["weight"], (int(spec["vocab_size"]), int(spec["hidden_size"])),
                           init="embedding")]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = tensors[self.spec["names"]["weight"]]

    def forward(self, ctx, resid, n_rows):
        ops.embedding(self.table, ctx.tokens, resid, n_rows, self.scale)


class PassOpener(Opener):
    """The start of a pass over a stretch of layers that a model repeats:
    resid = ((resid + pending delta) + scale * table[token]) + step[step_row], one float32 add after the other.  The
    embedding term is the model's embedding output over again (`add_embedding`; a first pass leaves it out); `step` is a
    [step_rows, hidden_size] tensor of which every pass has a row of its own.
    Parameters: hidden_size, vocab_size, scale, add_embedding, step_row, step_rows, names.{table, step}."""
    replayable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.scale = float(spec.get("scale", 1.0) or 1.0)
        self.add_embedding = bool(spec.get("add_embedding"))
        self.row = int(spec["step_row"])
        if not 0 <= self.row < int(spec["step_rows"]):
            raise ValueError("a pass opener names a row of its step tensor that does not exist")
        self.table = self.step = None

    @staticmethod
    def tensor_needs(spec: PartSpec) -> List[TensorNeed]:
        h, n = int(spec["hidden_size"]), spec["names"]
        needs = [TensorNeed(n["step"], (int(spec["step_rows"]), h), role="vector", init="linear")]
        if spec.get("add_embedding"):
            needs.append(TensorNeed(n["table"], (int(spec["vocab_size"]), h), init="embedding"))
        return needs

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.spec["names"]
        self.step = tensors[n["step"]][self.row].contiguous()
        self.table = tensors[n["table"]] if self.add_embedding else None

    def forward(self, ctx, resid, delta, n_rows):
        if delta is not None and not isinstance(delta, torch.Tensor):
            raise ValueError("a pass opener takes the pending result of a layer as one tensor")
        ops.open_pass(resid, delta, self.table, ctx.tokens if self.add_embedding else None, self.scale, self.step, n_rows)
        return None


class LMHead(Head):
    """logits = normed W^T in float32 for the wanted rows only; W is the embedding table when the
    model is tied (x0ne-core/runtime/src/engine.rs:823-835).  Parameters: vocab_size,
    hidden_size, tied, names.weight."""
    replayable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.linear = None

    @staticmethod
    def tensor_needs(spec: PartSpec) -> List[TensorNeed]:
        return [TensorNeed(spec["names"]["weight"], (int(spec["vocab_size"]), int(spec["hidden_size"])),
                           init="embedding")]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.linear = Linear(tensors[self.spec["names"]["weight"]])

    @staticmethod
    def optional_duplicates(spec: PartSpec):
        # a tied checkpoint may also store lm_head.weight, equal to the table (x0ne-core/runtime/src/weights.rs:154-159)
        return {"lm_head.weight": spec["names"]["weight"]} if spec.get("tied") else {}

    def weight_bytes(self) -> int:
        return self.linear.weight_bytes()

    def forward(self, normed, logits, n_rows):
        return self.linear(normed, logits, n_rows)


EMBEDDINGS.register("token_embedding", TokenEmbedding)
HEADS.register("lm_head", LMHead)
OPENERS.register("pass_opener", PassOpener)
