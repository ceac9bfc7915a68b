"""A feed-forward made of routed experts, identity experts and a shared expert.

Per token y:

  z = W_r y (+ b_r)                         router logits, float32, one per expert (identity ones too;
                                            `router_bias`: a learned offset per expert, tensor `router.b`)
  s = softmax(z)   (`score` "sigmoid": sigmoid(z))
  chosen = the `top` experts with the largest s + c   (`correction`: c is a learned number per
           expert that shifts the choice only)
  a_e = s_e * weight_scale                  (`renormalize`: divided by the chosen experts' sum of s)
  out = sum over chosen e of a_e * expert_e(y)  +  sigmoid(w_sg . y) * shared(y)

expert_e(y) = W_down (act(W_gate y) * (W_up y)) for e < num_experts; the last `num_identity`
router outputs are identity experts without tensors: expert_e(y) = y.  The shared expert has the
same form with a hidden size of its own, runs for every token, and is gated by one number per token
(`shared_gate`; without it it is added as it is).  With softmax scores and `renormalize` the
weights are the softmax over the chosen experts' logits alone.  The activation `clamped_swish`
acts on both halves (g' = min(g, L), u' = clamp(u, -L, L), g' sigmoid(1.702 g') (u' + 1)) with
`limit` L for the routed experts and `shared_limit` for the shared one.

The experts' matrices are stacked into [experts, 2 hidden, width] (gate rows, then up rows) and
[experts, width, hidden]; the tokens of a step are sorted by expert on the device and every expert
multiplies its own rows only.
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.parts.base import FeedForward
from simply_b200.parts.linear import Linear, fuse_rows
from simply_b200.registry import ACTIVATIONS, FEED_FORWARDS
from simply_b200.weights.loader import TensorSpec

_NAMES = {"gate": "gate", "up": "up", "down": "down", "router": "router", "correction": "correction",
          "shared": "shared", "shared_gate": "shared.sg", "expert": "e"}
_SCORES = {"softmax": 0, "sigmoid": 1}


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):

  graph_safe = True  # the tokens are dealt out on the device; the host never learns how

  def __init__(self, prefix: str, width: int, hidden: int, num_experts: int, top: int, activation: str = "silu",
               num_identity: int = 0, weight_scale: float = 1.0, score: str = "softmax", correction: bool = False,
               renormalize: bool = False, shared_hidden: int = 0, shared_gate: bool = False,
               names: dict[str, str] | None = None, router_bias: bool = False, limit: float = 0.0,
               shared_limit: float | None = None):
    if score not in _SCORES:
      raise ValueError(f"{prefix}: router score must be one of {sorted(_SCORES)}, got {score!r}")
    if not 1 <= top <= num_experts + num_identity:
      raise ValueError(f"{prefix}: the router chooses {top} of {num_experts + num_identity} experts")
    self.prefix, self.width, self.hidden = prefix, width, hidden
    self.num_experts, self.num_identity, self.top = num_experts, num_identity, top
    self.activation = ACTIVATIONS.get(activation)
    if self.activation > 3:
      raise ValueError(f"{prefix}: experts take the activations gelu_tanh, silu, relu and clamped_swish")
    self.limit = float(limit)
    self.shared_limit = self.limit if shared_limit is None else float(shared_limit)
    if self.activation == 3 and not (self.limit > 0 and self.shared_limit > 0):
      raise ValueError(f"{prefix}: the clamped activation needs positive limits")
    self.has_router_bias = bool(router_bias)
    self.weight_scale, self.score = float(weight_scale), _SCORES[score]
    self.has_correction, self.renormalize = bool(correction), bool(renormalize)
    self.shared_hidden, self.has_shared_gate = shared_hidden, bool(shared_gate and shared_hidden)
    n = self.names = {**_NAMES, **(names or {})}
    self.experts = [
        (Linear(f"{prefix}.{n['expert']}{e}.{n['gate']}", hidden, width),
         Linear(f"{prefix}.{n['expert']}{e}.{n['up']}", hidden, width),
         Linear(f"{prefix}.{n['expert']}{e}.{n['down']}", width, hidden)) for e in range(num_experts)]
    self.shared = None
    if shared_hidden:
      sp = f"{prefix}.{n['shared']}"
      self.shared = (Linear(f"{sp}.{n['gate']}", shared_hidden, width), Linear(f"{sp}.{n['up']}", shared_hidden, width),
                     Linear(f"{sp}.{n['down']}", width, shared_hidden))
    self.router_name = f"{prefix}.{n['router']}"
    self.correction_name = f"{prefix}.{n['correction']}"
    self.router_bias_name = f"{prefix}.{n['router']}.{n.get('bias', 'b')}"
    self.router_bias = None
    self.shared_gate_name = f"{prefix}.{n['shared_gate']}"
    self.gate_up = self.down = self.router = self.correction = self.shared_gate_w = None
    self.shared_gate_up = None

  def tensor_specs(self) -> list[TensorSpec]:
    total = self.num_experts + self.num_identity
    specs = [p.spec() for trio in self.experts for p in trio]
    specs.append(TensorSpec(self.router_name, (total, self.width), "matrix", precision="stored"))
    if self.has_router_bias:
      specs.append(TensorSpec(self.router_bias_name, (total,), "scale", precision="stored"))
    if self.has_correction:
      specs.append(TensorSpec(self.correction_name, (total,), "scale", precision="stored"))
    if self.shared is not None:
      specs += [p.spec() for p in self.shared]
      if self.has_shared_gate:
        specs.append(TensorSpec(self.shared_gate_name, (1, self.width), "matrix", precision="stored"))
    return specs

  def bind(self, tensors, ops) -> None:
    t = tensors
    if self.experts:
      self.gate_up = torch.stack([fuse_rows([t[g.name], t[u.name]]) for g, u, _ in self.experts]).contiguous()
      self.down = torch.stack([t[d.name] for _, _, d in self.experts]).contiguous()
    self.router = t[self.router_name].float().contiguous()
    self.correction = t[self.correction_name].float().contiguous() if self.has_correction else None
    self.router_bias = t[self.router_bias_name].float().contiguous() if self.has_router_bias else None
    if self.shared is not None:
      self.shared_gate_up = fuse_rows([t[self.shared[0].name], t[self.shared[1].name]])
      self.shared[2].bind(tensors)
      if self.has_shared_gate:
        self.shared_gate_w = t[self.shared_gate_name].float().reshape(-1).contiguous()

  def forward(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
    ops = ctx.ops
    # (only what differs from the plain case is passed on: see HeadNormAttention._store_options)
    more = {"bias": self.router_bias} if self.router_bias is not None else {}
    chosen, weight, gate = ops.route_tokens(
        x, self.router, self.correction, self.shared_gate_w, top=self.top, scale=self.weight_scale,
        score=self.score, renormalize=self.renormalize, **more)
    shared = None
    if self.shared is not None:
      if self.activation == 3:
        shared = self.shared[2](ops.gated_linear(x, self.shared_gate_up, self.activation, limit=self.shared_limit), ctx)
      else:
        shared = self.shared[2](ops.gated_linear(x, self.shared_gate_up, self.activation), ctx)
    more = {"limit": self.limit} if self.activation == 3 else {}
    return ops.mix_experts(x, chosen, weight, self.gate_up, self.down, self.num_experts, self.activation,
                           shared, gate, **more)


@FEED_FORWARDS.register("table_experts")
class TableExperts(FeedForward):
  """Experts without a router: a table `table` [vocab, top] of integers gives each token id its
  `top` experts (the entries of a row differ), each with weight 1 / top.  An expert is
  W_down act(W_up y), without biases and without a gate; `activation` "gelu_erf" is the exact gelu."""

  graph_safe = True  # the table is read on the device

  def __init__(self, prefix: str, width: int, hidden: int, num_experts: int, top: int, vocab_size: int,
               activation: str = "gelu_erf", names: dict[str, str] | None = None):
    if not 1 <= top <= num_experts:
      raise ValueError(f"{prefix}: each token uses {top} of {num_experts} experts")
    self.prefix, self.width, self.hidden = prefix, width, hidden
    self.num_experts, self.top, self.vocab_size = num_experts, top, vocab_size
    self.activation = ACTIVATIONS.get(activation)
    if self.activation == 3:
      raise ValueError(f"{prefix}: the clamped activation acts on a gate and an up half; these experts have no gate")
    n = self.names = {"up": "up", "down": "down", "expert": "e", "table": "table", **(names or {})}
    self.experts = [(Linear(f"{prefix}.{n['expert']}{e}.{n['up']}", hidden, width),
                     Linear(f"{prefix}.{n['expert']}{e}.{n['down']}", width, hidden)) for e in range(num_experts)]
    self.table_name = f"{prefix}.{n['table']}"
    self.up = self.down = self.table = None

  def tensor_specs(self) -> list[TensorSpec]:
    specs = [p.spec() for pair in self.experts for p in pair]
    return specs + [TensorSpec(self.table_name, (self.vocab_size, self.top), "table", choices=self.num_experts)]

  def bind(self, tensors, ops) -> None:
    self.up = torch.stack([tensors[u.name] for u, _ in self.experts]).contiguous()
    self.down = torch.stack([tensors[d.name] for _, d in self.experts]).contiguous()
    self.table = tensors[self.table_name].to(torch.int32).contiguous()

  def forward(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
    ops = ctx.ops
    chosen, weight = ops.route_by_table(ctx.token_ids, self.table, self.num_experts)
    return ops.mix_experts(x, chosen, weight, self.up, self.down, self.num_experts, self.activation, None, None,
                           gated=False)
