"""Gated feed-forward: down(act(gate(x)) * up(x)), no biases.

simply/model_lib.py:714-730 with use_gated_activation_in_ffn: the activation
acts on the gate projection (`ffn_0_gate`), the product with `ffn_0` (up) feeds
`ffn_1` (down).  The activation is chosen by name; `gelu_tanh` is
simply/model_lib.py:93-96.  `clamped_swish` takes a `limit` L and acts on both halves:
g' = min(g, L), u' = clamp(u, -L, L), z = g' sigmoid(1.702 g') (u' + 1).
"""

from __future__ import annotations

import math
from typing import Any

import torch

from simply_b200.parts.base import FeedForward
from simply_b200.parts.linear import Linear, fuse_rows
from simply_b200.registry import ACTIVATIONS, FEED_FORWARDS
from simply_b200.weights.loader import TensorSpec

# Activation name -> code the gated-activation kernel takes.
ACTIVATIONS.register("gelu_tanh", 0)
ACTIVATIONS.register("silu", 1)
ACTIVATIONS.register("relu", 2)
ACTIVATIONS.register("clamped_swish", 3)
ACTIVATIONS.register("gelu_erf", 4)  # the exact gelu; experts without a gate only


@FEED_FORWARDS.register("gated")
class GatedFeedForward(FeedForward):

  graph_safe = True

  def __init__(self, prefix: str, width: int, hidden: int, activation: str,
               names: dict[str, str] | None = None, limit: float = 0.0):
    self.prefix = prefix
    self.width = width
    self.hidden = hidden
    self.activation = ACTIVATIONS.get(activation)
    if self.activation > 3:
      raise ValueError(f"{prefix}: the gated products take gelu_tanh, silu, relu and clamped_swish")
    self.limit = float(limit)
    if activation == "clamped_swish" and not self.limit > 0:
      raise ValueError(f"{prefix}: the clamped activation needs a positive limit")
    names = names or {}  # role -> the tensor's name after the prefix
    self.gate_proj = Linear(f"{prefix}.{names.get('gate', 'gate_proj.weight')}", hidden, width)
    self.up_proj = Linear(f"{prefix}.{names.get('up', 'up_proj.weight')}", hidden, width)
    self.down_proj = Linear(f"{prefix}.{names.get('down', 'down_proj.weight')}", width, hidden)
    self.gate_up_weight: torch.Tensor | None = None

  def tensor_specs(self) -> list[TensorSpec]:
    return [self.gate_proj.spec(), self.up_proj.spec(), self.down_proj.spec()]

  def bind(self, tensors, ops) -> None:
    # Gate rows first, up rows second: one product yields [T, 2 * hidden].
    self.gate_up_weight = fuse_rows([tensors[self.gate_proj.name], tensors[self.up_proj.name]])
    self.down_proj.bind(tensors)

  def forward(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
    ops = ctx.ops
    if self.limit:
      z = ops.gated_linear(x, self.gate_up_weight, self.activation, limit=self.limit)
    else:
      z = ops.gated_linear(x, self.gate_up_weight, self.activation)
    return self.down_proj(z, ctx)


@FEED_FORWARDS.register("learned_activation")
class LearnedActivationFeedForward(FeedForward):
  """down(act(up(x))) without a gate, no biases, with an activation that has learned numbers.

  `activation` "xielu": two numbers p, q (tensor `act`, [2]) give a_p = softplus(p) and
  a_n = 1/2 + softplus(q), both in float32;
    z > 0:   a_p z^2 + z / 2
    z <= 0:  a_n (e^z - 1 - z) + z / 2
  """

  graph_safe = True

  def __init__(self, prefix: str, width: int, hidden: int, activation: str = "xielu",
               names: dict[str, str] | None = None):
    if activation != "xielu":
      raise ValueError(f"{prefix}: known learned activations: xielu")
    names = names or {}
    self.prefix, self.width, self.hidden = prefix, width, hidden
    self.up_proj = Linear(f"{prefix}.{names.get('up', 'up')}", hidden, width)
    self.down_proj = Linear(f"{prefix}.{names.get('down', 'down')}", width, hidden)
    self.act_name = f"{prefix}.{names.get('act', 'act')}"
    self.act: torch.Tensor | None = None
    self.factors: tuple[float, float] | None = None

  def tensor_specs(self) -> list[TensorSpec]:
    return [self.up_proj.spec(), self.down_proj.spec(), TensorSpec(self.act_name, (2,), "scale", precision="stored")]

  def bind(self, tensors, ops) -> None:
    self.up_proj.bind(tensors)
    self.down_proj.bind(tensors)
    self.act = tensors[self.act_name].float().contiguous()
    # (weights: known to the host once, so that a kernel can take them as plain numbers)
    p, q = (float(v) for v in self.act.double().cpu())
    softplus = lambda z: math.log1p(math.exp(-abs(z))) + max(z, 0.0)
    self.factors = (softplus(p), 0.5 + softplus(q))

  def forward(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
    return self.down_proj(ctx.ops.linear_xielu(x, self.up_proj.weight, self.act, self.factors), ctx)


@FEED_FORWARDS.register("none")
class NoFeedForward(FeedForward):
  """A layer without a feed-forward: block arrangements skip it."""

  graph_safe = True

  def __init__(self, prefix: str = ""):
    pass

  def forward(self, x: torch.Tensor, ctx: Any) -> None:
    return None
