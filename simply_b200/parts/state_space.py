"""The state-space mixer of Mamba-2 (state-space duality), in its recurrent form.

One product of the mixer's input gives [z: inner | x: inner | B: G N | C: G N | dt: heads] with
inner = heads * value_dim, N the state size and G groups of heads that share B and C.  x, B and C
pass a causal convolution per channel (`conv` [channels, taps] with bias `conv.b`, the last column the
current token's) and silu.  Per head h of group g = h // (heads / G), with a matrix S [N, value_dim]
(float32, zero at a request's start):

  dt  = softplus(dt + dt_bias_h)                  no clamp
  S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T
  y_t = S_t^T C_t + D_h x_t

y (heads side by side) is multiplied by silu(z), RMS-normed in `norm_groups` equal parts, scaled per
channel and projected by W_o.  A request's state is S and the convolution's last taps - 1 inputs.
Everything between the product and the output projection is float32.
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.cache.needs import SlotStateNeed
from simply_b200.parts.base import Mixer
from simply_b200.parts.linear import Linear
from simply_b200.registry import MIXERS
from simply_b200.weights.loader import TensorSpec

_NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "step_bias": "dt_bias", "rate_log": "A_log",
          "skip": "D", "norm": "norm", "out": "o"}


@MIXERS.register("state_space_duality")
class StateSpaceDuality(Mixer):

  graph_safe = True  # reads the step's device tensors only; rows that repeat a slot do not write its state

  def __init__(self, prefix: str, width: int, num_heads: int, value_dim: int, state_dim: int, num_groups: int,
               norm_groups: int, conv_taps: int, eps: float, names: dict[str, str] | None = None):
    if num_heads % num_groups:
      raise ValueError(f"{prefix}: num_heads {num_heads} is no multiple of num_groups {num_groups}")
    inner = self.inner = num_heads * value_dim
    if inner % norm_groups:
      raise ValueError(f"{prefix}: norm_groups {norm_groups} does not divide {inner} channels")
    if conv_taps < 1:
      raise ValueError(f"{prefix}: a convolution needs at least one tap, got {conv_taps}")
    self.prefix, self.width = prefix, width
    self.num_heads, self.value_dim, self.state_dim, self.num_groups = num_heads, value_dim, state_dim, num_groups
    self.norm_groups, self.conv_taps, self.eps = norm_groups, conv_taps, float(eps)
    self.channels = inner + 2 * num_groups * state_dim  # what the convolution sees: x | B | C
    n = self.names = {**_NAMES, **(names or {})}
    self.in_proj = Linear(f"{prefix}.{n['in']}", inner + self.channels + num_heads, width)
    self.o_proj = Linear(f"{prefix}.{n['out']}", width, inner)

  def _name(self, role: str) -> str:
    return f"{self.prefix}.{self.names[role]}"

  def cache_need(self):
    need = {"state": SlotStateNeed((self.num_heads, self.state_dim, self.value_dim), "float32")}
    if self.conv_taps > 1:
      need["conv"] = SlotStateNeed((self.conv_taps - 1, self.channels), "float32")
    return need

  def tensor_specs(self) -> list[TensorSpec]:
    return [self.in_proj.spec(), self.o_proj.spec(),
            TensorSpec(self._name("conv"), (self.channels, self.conv_taps), "matrix"),
            TensorSpec(self._name("conv_bias"), (self.channels,), "scale", precision="stored"),
            TensorSpec(self._name("step_bias"), (self.num_heads,), "scale", precision="stored"),
            TensorSpec(self._name("rate_log"), (self.num_heads,), "scale", precision="stored"),
            TensorSpec(self._name("skip"), (self.num_heads,), "gain", precision="stored"),
            TensorSpec(self._name("norm"), (self.inner,), "gain")]

  def bind(self, tensors, ops) -> None:
    t = tensors
    w = t[self.in_proj.name]
    extra = -w.shape[0] % 8
    self.in_weight = torch.cat([w, w.new_zeros(extra, w.shape[1])]).contiguous() if extra else w.contiguous()
    self.o_proj.bind(t)
    self.conv_weight = t[self._name("conv")].float().contiguous()
    self.conv_bias = t[self._name("conv_bias")].float().contiguous()
    self.step_bias = t[self._name("step_bias")].float().contiguous()
    self.neg_rate = (-torch.exp(t[self._name("rate_log")].float())).contiguous()
    self.skip = t[self._name("skip")].float().contiguous()
    self.norm_weight = t[self._name("norm")].float().contiguous()

  def forward(self, x: torch.Tensor, ctx: Any, cache: Any, writes_cache: bool = True) -> torch.Tensor:
    ops = ctx.ops
    inner = self.inner
    pre = ops.linear(x, self.in_weight)  # z | x | B | C | dt, before the convolution
    conv_state = cache["conv"].storage if self.conv_taps > 1 else None
    xbc = ops.short_conv(pre, self.conv_weight, self.conv_bias, conv_state, ctx, activation=1, residual=False,
                         offset=inner, channels=self.channels, out_dtype=torch.float32)
    y = ops.state_space_scan(xbc, pre, inner + self.channels, self.step_bias, self.neg_rate, self.skip,
                             cache["state"].storage, ctx, num_heads=self.num_heads, value_dim=self.value_dim,
                             state_dim=self.state_dim, num_groups=self.num_groups)
    y = ops.group_norm_gate(y, self.norm_weight, self.eps, groups=self.norm_groups, gate=pre, gate_offset=0,
                            gate_kind="silu_before")
    return self.o_proj(y, ctx)
