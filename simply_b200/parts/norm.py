"""RMS normalisation with an optional (1 + w) scale.

simply/model_lib.py:154-178 with use_bias=False: `x * rsqrt(mean(x^2) + eps) * (1 + scale)`,
the mean of squares and the rsqrt in float32.  `plus_one` is the reference's
`scale_plus_one` (simply/config_lib.py:296).
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.parts.base import Norm
from simply_b200.registry import NORMS
from simply_b200.weights.loader import TensorSpec


@NORMS.register("rms_norm")
class RMSNorm(Norm):

  graph_safe = True

  def __init__(self, prefix: str, width: int, eps: float, plus_one: bool = True, name: str | None = None):
    self.name = name or f"{prefix}.weight"  # `name`: the scale's whole tensor name, where it is not "<prefix>.weight"
    self.width = width
    self.eps = float(eps)
    self.plus_one = bool(plus_one)
    self.weight: torch.Tensor | None = None

  def tensor_specs(self) -> list[TensorSpec]:
    return [TensorSpec(self.name, (self.width,), "scale" if self.plus_one else "gain")]

  def bind(self, tensors, ops) -> None:
    self.weight = tensors[self.name]

  def apply(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
    return ctx.ops.rms_norm(x, self.weight, self.eps, self.plus_one)


@NORMS.register("dynamic_tanh")
class DynamicTanh(Norm):
  """A norm that computes no statistics: y = tanh(alpha x) * w + b, with one learned number
  `alpha`, a scale `w` and an offset `b` per channel, in float32.  Tensor names: `name` (the scale),
  `name`.alpha, `name`.b."""

  graph_safe = True

  def __init__(self, prefix: str, width: int, name: str | None = None, eps: float = 0.0):
    self.name = name or f"{prefix}.weight"
    self.width = width
    self.weight = self.bias = self.alpha = None

  def tensor_specs(self) -> list[TensorSpec]:
    return [TensorSpec(self.name, (self.width,), "gain"), TensorSpec(f"{self.name}.b", (self.width,), "scale"),
            TensorSpec(f"{self.name}.alpha", (), "gain")]

  def bind(self, tensors, ops) -> None:
    self.weight = tensors[self.name].float().contiguous()
    self.bias = tensors[f"{self.name}.b"].float().contiguous()
    self.alpha = tensors[f"{self.name}.alpha"].float().reshape(1).contiguous()

  def apply(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
    return ctx.ops.scaled_residual_tanh(x, None, None, None, None, self, None)


@NORMS.register("channel_scale")
class ChannelScale(Norm):
  """y = x * w with one learned factor per channel (a branch's scale before it joins the stream)."""

  graph_safe = True

  def __init__(self, prefix: str, width: int, name: str | None = None):
    self.name = name or f"{prefix}.weight"
    self.width = width
    self.weight = None

  def tensor_specs(self) -> list[TensorSpec]:
    return [TensorSpec(self.name, (self.width,), "gain")]

  def bind(self, tensors, ops) -> None:
    self.weight = tensors[self.name].float().contiguous()

  def apply(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
    return ctx.ops.scale_channels(x, self.weight)
