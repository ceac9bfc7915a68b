"""The generalized delta rule: a recurrent mixer whose state forgets per channel and unlearns along
the key before it learns.

Per head a matrix S [head_dim, head_dim] (float32, zero at a request's start, one per request in
a state slot).  From the mixer's input y, all per head and key channel:

  r = W_r y,  k = W_k y,  v = W_v y
  w = exp(-e^(-1/2) * sigmoid(W_w2 tanh(W_w1 y) + w0))      decay, through a low rank
  a = sigmoid(W_a y + b_a)                                   removal rate
  u = k / sqrt(sum k^2 + 1e-6)                               the unit key
  S_t = diag(w) S_(t-1) - (a * u) (u^T S_(t-1)) + k v^T      both first terms read the old state
  o_t = S_t^T r

Each head's o is divided by its root mean square, scaled per channel (a scale over all heads'
channels), multiplied by sigmoid(W_g y), and the heads side by side go through W_o.  r, k, v, the
gate, a and the low rank's first half come out of one fused product; everything between the
products and the output projection is float32.
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.cache.needs import SlotStateNeed
from simply_b200.parts.base import Mixer
from simply_b200.parts.linear import Linear, fuse_rows
from simply_b200.registry import MIXERS
from simply_b200.weights.loader import TensorSpec

_NAMES = {"r": "r", "k": "k", "v": "v", "gate": "g", "removal": "a", "removal_bias": "a.b", "decay_in": "w1",
          "decay_out": "w2", "decay_bias": "w0", "norm": "norm", "out": "o"}


@MIXERS.register("generalized_delta_rule")
class GeneralizedDeltaRule(Mixer):

  graph_safe = True  # reads the step's device tensors only; rows that repeat a slot do not write its state

  def __init__(self, prefix: str, width: int, num_heads: int, head_dim: int, eps: float, decay_rank: int = -1,
               names: dict[str, str] | None = None):
    self.prefix, self.width, self.num_heads, self.head_dim = prefix, width, num_heads, head_dim
    self.eps = float(eps)
    n = self.names = {**_NAMES, **(names or {})}
    inner = self.inner = num_heads * head_dim
    self.projections = [Linear(f"{prefix}.{n[role]}", inner, width) for role in ("r", "k", "v", "gate", "removal")]
    self.decay_in = Linear(f"{prefix}.{n['decay_in']}", decay_rank, width)
    self.decay_out = Linear(f"{prefix}.{n['decay_out']}", inner, decay_rank)
    self.o_proj = Linear(f"{prefix}.{n['out']}", width, inner)

  def _name(self, role: str) -> str:
    return f"{self.prefix}.{self.names[role]}"

  def cache_need(self):
    return SlotStateNeed((self.num_heads, self.head_dim, self.head_dim), "float32")

  def tensor_specs(self) -> list[TensorSpec]:
    specs = [p.spec() for p in self.projections + [self.decay_in, self.decay_out, self.o_proj]]
    specs += [TensorSpec(self._name("removal_bias"), (self.inner,), "scale", precision="stored"),
              TensorSpec(self._name("decay_bias"), (self.inner,), "scale", precision="stored"),
              TensorSpec(self._name("norm"), (self.inner,), "gain")]
    return specs

  def bind(self, tensors, ops) -> None:
    t = tensors
    w = fuse_rows([t[p.name] for p in self.projections + [self.decay_in]])  # r | k | v | gate | a | low rank
    self.rank = t[self.decay_in.name].shape[0]
    if t[self.decay_out.name].shape[1] != self.rank:
      raise ValueError(f"{self.prefix}: the low-rank pair does not fit")
    extra = -w.shape[0] % 8
    self.in_weight = torch.cat([w, w.new_zeros(extra, w.shape[1])]).contiguous() if extra else w
    self.decay_out.bind(t)
    self.o_proj.bind(t)
    self.removal_bias = t[self._name("removal_bias")].float().contiguous()
    self.decay_bias = t[self._name("decay_bias")].float().contiguous()
    self.norm_weight = t[self._name("norm")].float().contiguous()

  def forward(self, x: torch.Tensor, ctx: Any, cache: Any, writes_cache: bool = True) -> torch.Tensor:
    ops = ctx.ops
    inner = self.inner
    pre = ops.linear(x, self.in_weight)
    low = ops.linear(ops.tanh_columns(pre, 5 * inner, self.rank), self.decay_out.weight)
    o = ops.general_delta_scan(pre, low, self.decay_bias, self.removal_bias, cache.storage, ctx,
                               num_heads=self.num_heads, head_dim=self.head_dim)
    y = ops.group_norm_gate(o, self.norm_weight, self.eps, groups=self.num_heads, gate=pre, gate_offset=3 * inner,
                            gate_kind="sigmoid_after")
    return self.o_proj(y, ctx)
