"""Steps that act on the residual stream between layer calls.

`projected_input` gives the stream the embedding's output again, through a matrix:

  x <- W [x; x0] + step[pass]

with W [width, 2 width] (the columns that read x first), x0 the stream as the embedding left it,
and `step` [passes, width] one learned row per pass of a run of layers that is walked several
times.  A run order names the step and the pass (`LayerCall.stream_input`); the step runs right
before that call.  The product takes both halves in the activation dtype and leaves float32
sums; the row is added in float32, and the result replaces the stream.
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.parts.base import Part
from simply_b200.registry import STREAM_INPUTS
from simply_b200.weights.loader import TensorSpec


class StreamInput(Part):

  def forward(self, stream: Any, first: torch.Tensor, index: int, ctx: Any) -> None:
    """Rewrites `stream` (a `ResidualStream`) in place; `first` is the embedding's output, float32."""
    raise NotImplementedError


@STREAM_INPUTS.register("projected_input")
class ProjectedInput(StreamInput):

  graph_safe = True

  def __init__(self, prefix: str, width: int, passes: int, matrix: str = "in", rows: str | None = "step"):
    self.prefix, self.width, self.passes = prefix, width, int(passes)
    self.matrix_name = f"{prefix}.{matrix}"
    self.rows_name = f"{prefix}.{rows}" if rows else None
    self.matrix = self.rows = None

  def tensor_specs(self) -> list[TensorSpec]:
    specs = [TensorSpec(self.matrix_name, (self.width, 2 * self.width), "matrix")]
    if self.rows_name:
      specs.append(TensorSpec(self.rows_name, (self.passes, self.width), "scale"))
    return specs

  def bind(self, tensors, ops) -> None:
    self.matrix = tensors[self.matrix_name]
    if self.rows_name:
      self.rows = tensors[self.rows_name].float().contiguous()

  def forward(self, stream: Any, first: torch.Tensor, index: int, ctx: Any) -> None:
    if not 0 <= index < self.passes:
      raise ValueError(f"{self.prefix}: pass {index} of {self.passes}")
    stream.flush(ctx)
    both = ctx.ops.pack_pair(stream.h, first)  # [T, 2 width] in the activation dtype
    stream.h = ctx.ops.linear_wide(both, self.matrix, self.rows[index] if self.rows is not None else None)
