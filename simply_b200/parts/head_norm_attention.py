"""Grouped-query attention whose heads are normed one by one, with tied values and an output gate.

Beside `paged_attention` and `qk_norm_attention` for designs whose attention differs from them in
any of these, each switched by a parameter:

* rotary positions on the first `rotary["dims"]` dims of every q and k head, pairing neighbours
  (2i, 2i + 1) (`layout` "neighbours") or halves (i, i + dims/2) (`layout` "halves"), angle
  p * base^(-2i/dims);
* `head_norm`: after the rotation every q and k head is divided by its own root mean square
  (over head_dim, eps inside the root, no scale);
* `tie_values`: there is no value projection: a key head as projected (before rotation and
  norm) is also the value head;
* score = q.k * score_scale, then `score_softcap` * tanh(score / score_softcap) before the softmax;
* causal, optionally over a window of `window` keys;
* `output_gate`: the heads side by side are multiplied by sigmoid(W_g y) before the output
  projection; the gate reads the mixer's input, like q and k.  `gate_per_head`: W_g has one row
  per head, and a head's whole result is multiplied by its one number;
* `value_dim`: value heads of another size than key heads (not with tied values);
* `projection_bias`: q, k and v each have a bias (tensor `<name>.b`), added in float32 to the
  projection before the rotation;
* `distance_bias`: the score of query i and key j loses r1_h * log(1 + r2_h * (i - j)), with two
  learned numbers per query head (tensors `r1`, `r2`), in float32.

q, k, (v) and the gate come out of one fused product.
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.cache.needs import PagedKVNeed
from simply_b200.parts.base import Mixer
from simply_b200.parts.linear import Linear, fuse_rows
from simply_b200.parts.normed_attention import rotation_frequencies
from simply_b200.registry import MIXERS
from simply_b200.weights.loader import TensorSpec

_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "r1": "r1", "r2": "r2", "bias": "b"}


@MIXERS.register("head_norm_attention")
class HeadNormAttention(Mixer):

  graph_safe = True

  def __init__(self, prefix: str, width: int, num_heads: int, num_kv_heads: int, head_dim: int,
               score_scale: float, eps: float, score_softcap: float = 0.0, window: int | None = None,
               rotary: dict | None = None, head_norm: bool = True, tie_values: bool = True,
               output_gate: bool = True, names: dict[str, str] | None = None, value_dim: int | None = None,
               gate_per_head: bool = False, projection_bias: bool = False, distance_bias: bool = False):
    if num_heads % num_kv_heads:
      raise ValueError(f"{prefix}: num_heads {num_heads} is no multiple of num_kv_heads {num_kv_heads}")
    self.prefix, self.width = prefix, width
    self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
    self.score_scale, self.eps = float(score_scale), float(eps)
    self.score_softcap = float(score_softcap or 0.0)
    self.window = window
    self.rotary = dict(rotary) if rotary else None
    if self.rotary:
      if self.rotary["dims"] % 2 or self.rotary["dims"] > head_dim:
        raise ValueError(f"{prefix}: {self.rotary['dims']} rotated dims do not fit a head of {head_dim}")
      if self.rotary.get("layout", "neighbours") not in ("neighbours", "halves"):
        raise ValueError(f"{prefix}: rotary layout must be 'neighbours' or 'halves'")
    self.head_norm, self.tie_values, self.output_gate = bool(head_norm), bool(tie_values), bool(output_gate)
    self.value_dim = head_dim if value_dim is None else int(value_dim)
    if self.tie_values and self.value_dim != head_dim:
      raise ValueError(f"{prefix}: tied values have the keys' size")
    self.gate_per_head, self.projection_bias = bool(gate_per_head), bool(projection_bias)
    self.distance_bias = bool(distance_bias)
    n = self.names = {**_NAMES, **(names or {})}
    self.q_proj = Linear(f"{prefix}.{n['q']}", num_heads * head_dim, width)
    self.k_proj = Linear(f"{prefix}.{n['k']}", num_kv_heads * head_dim, width)
    self.v_proj = None if self.tie_values else Linear(f"{prefix}.{n['v']}", num_kv_heads * self.value_dim, width)
    gate_rows = num_heads if self.gate_per_head else num_heads * self.value_dim
    self.g_proj = Linear(f"{prefix}.{n['g']}", gate_rows, width) if self.output_gate else None
    self.o_proj = Linear(f"{prefix}.{n['o']}", width, num_heads * self.value_dim)
    self.in_weight = self.rot_freq = self.in_bias = self.distance = None
    self.gate_offset = 0

  def _inputs(self) -> list[Linear]:
    return [p for p in (self.q_proj, self.k_proj, self.v_proj, self.g_proj) if p is not None]

  def cache_need(self):
    return PagedKVNeed(self.num_kv_heads, self.head_dim, self.window,
                       value_dim=None if self.value_dim == self.head_dim else self.value_dim)

  def graph_plans(self, ops, batch: int, bucket: int, max_burst: int, page_size: int) -> list:
    if self.value_dim != self.head_dim:
      return []  # (the general kernel needs no list)
    plan = ops.attention_graph_plan(
        window=self.window, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
        batch=batch, bucket=bucket, max_burst=max_burst, page_size=page_size)
    return [plan] if plan is not None else []

  def tensor_specs(self) -> list[TensorSpec]:
    specs = [p.spec() for p in self._inputs()] + [self.o_proj.spec()]
    if self.projection_bias:
      specs += [TensorSpec(f"{p.name}.{self.names['bias']}", (p.out_features,), "scale", precision="stored")
                for p in self._biased()]
    if self.distance_bias:
      specs += [TensorSpec(f"{self.prefix}.{self.names[r]}", (self.num_heads,), "gain", precision="stored")
                for r in ("r1", "r2")]
    return specs

  def _biased(self) -> list[Linear]:
    return [p for p in (self.q_proj, self.k_proj, self.v_proj) if p is not None]

  def bind(self, tensors, ops) -> None:
    if self.head_dim % 2 == 0 and self.value_dim == self.head_dim:  # (the general kernel takes the rest)
      ops.check_attention(self.head_dim, self.num_heads, self.num_kv_heads)
    w = fuse_rows([tensors[p.name] for p in self._inputs()])
    extra = -w.shape[0] % 8  # whole 16-byte groups of output features for the products' stores
    self.in_weight = torch.cat([w, w.new_zeros(extra, w.shape[1])]).contiguous() if extra else w
    self.gate_offset = sum(p.out_features for p in self._inputs()[:-1]) if self.output_gate else 0
    self.o_proj.bind(tensors)
    if self.projection_bias:
      self.in_bias = torch.cat([tensors[f"{p.name}.{self.names['bias']}"].float() for p in self._biased()]).contiguous()
    if self.distance_bias:  # [2, heads]: r1, then r2
      self.distance = torch.stack([tensors[f"{self.prefix}.{self.names[r]}"].float() for r in ("r1", "r2")]).contiguous()
    if self.rotary:
      freq = rotation_frequencies(self.rotary["dims"], self.rotary["base"])
      self.rot_freq = torch.from_numpy(freq).to(self.in_weight.device)

  def _store_options(self) -> dict:
    """(only what differs from the plain case is passed on, so that a kernel table that predates
    an option still serves the models that do not use it)"""
    opts: dict[str, Any] = {}
    if self.value_dim != self.head_dim:
      opts["value_dim"] = self.value_dim
    if self.in_bias is not None:
      opts["bias"] = self.in_bias
    return opts

  def _attention_options(self) -> dict:
    opts: dict[str, Any] = {}
    if self.value_dim != self.head_dim:
      opts["value_dim"] = self.value_dim
    if self.distance is not None:
      opts["distance_bias"] = self.distance
    return opts

  def forward(self, x: torch.Tensor, ctx: Any, cache: Any, writes_cache: bool = True) -> torch.Tensor:
    ops = ctx.ops
    block_table = ctx.block_tables[cache.group]
    proj = ops.linear(x, self.in_weight)  # q | k | (v) | (gate)
    q = ops.rotate_headnorm_store(
        proj, self.eps, self.score_scale, self.rot_freq,
        interleaved=bool(self.rotary) and self.rotary.get("layout", "neighbours") == "neighbours",
        head_norm=self.head_norm, tie_values=self.tie_values, num_heads=self.num_heads,
        num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
        storage=cache.storage if writes_cache else None, block_table=block_table, ctx=ctx,
        **self._store_options())
    o = ops.paged_attention(
        q, cache.storage, block_table, ctx, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads,
        head_dim=self.head_dim, logit_softcap=self.score_softcap, window=self.window, **self._attention_options())
    if self.output_gate:
      o = ops.sigmoid_gate(o, proj, self.gate_offset, self.value_dim if self.gate_per_head else 1)
    return self.o_proj(o, ctx)
