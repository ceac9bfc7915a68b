"""Token embedding and the output layer.

`token_embedding`: rows of the table times a constant, sqrt(width) for Gemma 2
(simply/utils/module.py:450-481).  `tied_head`: logits = x . table^T with the
same table, no bias, then the final soft cap (simply/model_lib.py:3183-3188,
simply/utils/module.py:416-433); logits are produced in float32.  `logit_scale` multiplies them
(float32, before the cap).  `linear_head`
is the same with a table of its own.
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.parts.base import Embedding, Head
from simply_b200.registry import EMBEDDINGS, HEADS
from simply_b200.weights.loader import TensorSpec, WeightError


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Embedding):

  graph_safe = True

  def __init__(self, prefix: str, vocab_size: int, width: int, scale: float = 1.0, name: str | None = None,
               position_table: str | None = None, max_positions: int = 0, round_scale: bool = True):
    """`position_table`: name of a learned table [max_positions, width] whose row `position` is added
    (unscaled) to every token's row.  `round_scale`: the factor is rounded to the table's dtype first
    (the reference's way); False multiplies by the float32 factor."""
    self.name = name or f"{prefix}.weight"
    self.vocab_size = vocab_size
    self.width = width
    self.scale = float(scale)
    self.round_scale = bool(round_scale)
    self.position_name, self.max_positions = position_table, int(max_positions)
    if position_table is not None and self.max_positions <= 0:
      raise ValueError(f"{prefix}: a position table needs max_positions")
    self.table: torch.Tensor | None = None
    self.positions: torch.Tensor | None = None

  def tensor_specs(self) -> list[TensorSpec]:
    specs = [TensorSpec(self.name, (self.vocab_size, self.width), "matrix")]
    if self.position_name is not None:
      specs.append(TensorSpec(self.position_name, (self.max_positions, self.width), "matrix"))
    return specs

  def bind(self, tensors, ops) -> None:
    self.table = tensors[self.name]
    if self.position_name is not None:
      self.positions = tensors[self.position_name]

  def forward(self, ctx: Any) -> torch.Tensor:
    """float32 [T, width]: the start of the residual stream."""
    if self.positions is None and self.round_scale:
      return ctx.ops.embed(self.table, ctx.token_ids, self.scale)
    return ctx.ops.embed(self.table, ctx.token_ids, self.scale, positions=ctx.positions,
                         position_table=self.positions, round_scale=self.round_scale)

  def rides_exactly(self, dtype: torch.dtype) -> bool:
    """True if `forward`'s float32 rows are exact in `dtype` (rows of the table as they are)."""
    if self.positions is not None and dtype != torch.float32:
      return False
    return dtype == torch.float32 or (self.scale == 1.0 and self.table is not None and self.table.dtype == dtype)


@HEADS.register("tied_head")
class TiedHead(Head):

  graph_safe = True

  def __init__(self, prefix: str, embedding: Embedding, logit_softcap: float = 0.0, logit_scale: float = 1.0):
    self.embedding = embedding
    self.logit_softcap = float(logit_softcap or 0.0)
    self.logit_scale = float(logit_scale)

  def tensor_specs(self) -> list[TensorSpec]:
    # A folder may repeat the tied table under the output layer's name.
    return [TensorSpec("lm_head.weight", (self.embedding.vocab_size, self.embedding.width),
                       "matrix", optional=True)]

  def bind(self, tensors, ops) -> None:
    # The tied table may appear a second time under the output layer's name, but only as a copy.
    duplicate = tensors.get("lm_head.weight")
    if duplicate is not None:
      table = tensors[self.embedding.name]
      if duplicate.shape != table.shape or not torch.equal(duplicate.to(table.dtype), table):
        raise WeightError([], [], [], [], other=[
            f"lm_head.weight differs from {self.embedding.name}: this model ties its output layer to "
            "the embedding table, so the folder may repeat the table but not hold another one"])

  def forward(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
    if self.logit_scale != 1.0:
      return ctx.ops.lm_head(x, self.embedding.table, self.logit_softcap, scale=self.logit_scale)
    return ctx.ops.lm_head(x, self.embedding.table, self.logit_softcap)


@HEADS.register("linear_head")
class LinearHead(Head):
  """An output layer with a table of its own: logits = x . W^T, then the final soft cap."""

  graph_safe = True

  def __init__(self, prefix: str, embedding: Embedding, logit_softcap: float = 0.0, name: str | None = None):
    self.name = name or f"{prefix}.weight"
    self.vocab_size, self.width = embedding.vocab_size, embedding.width
    self.logit_softcap = float(logit_softcap or 0.0)
    self.table: torch.Tensor | None = None

  def tensor_specs(self) -> list[TensorSpec]:
    return [TensorSpec(self.name, (self.vocab_size, self.width), "matrix")]

  def bind(self, tensors, ops) -> None:
    self.table = tensors[self.name]

  def forward(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
    return ctx.ops.lm_head(x, self.table, self.logit_softcap)
