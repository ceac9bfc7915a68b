"""Attention whose keys and values are read out of one small latent per token.

Per token, from the mixer's input y:

  c_q = rms(W_dq y) * n_q                          the queries' latent         [query_rank]
  q   = W_uq c_q                                   per head [head_dim plain | rotated_dim rotated]
  c   = rms((W_dkv y)[:kv_rank]) * n_kv            the keys' and values' latent [kv_rank]
  k_r = turn((W_dkv y)[kv_rank:], position)        one rotated key part for all heads [rotated_dim]
  k_h = W_uk,h c,  v_h = W_uv,h c                  per head
  s   = scale * (q_plain . k_h + turn(q_rot) . k_r)

over the keys that the window admits (`window` W: the token itself and the W - 1 before it), with
a softmax whose denominator also holds exp(sink_h), a learned number per head that has no key and
no value.  Head h's result is multiplied by sigmoid(W_g y)_h and the heads side by side go through
W_o.  The rotation pairs dimension i of the rotated part with dimension i + dims/2 and turns them
by position * base^(-2 i / dims).

The cache holds c and k_r only: one row of kv_rank + rotated_dim numbers per token.  Since
q_plain . (W_uk,h c) = (W_uk,h^T q_plain) . c and sum_j p_j W_uv,h c_j = W_uv,h sum_j p_j c_j, every head
asks the cache with the vector [W_uk,h^T q_plain | turn(q_rot)] and reads a weighted sum of latents,
which W_uv,h expands afterwards: attention over one shared key/value head whose keys are the rows
themselves and whose values are their first kv_rank numbers.
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.cache.needs import PagedKVNeed
from simply_b200.parts.base import Mixer
from simply_b200.parts.linear import Linear, fuse_rows
from simply_b200.registry import MIXERS
from simply_b200.weights.loader import TensorSpec

_NAMES = {"query_down": "dq", "query_norm": "dq.norm", "query_up": "uq", "kv_down": "dkv", "kv_norm": "dkv.norm",
          "key_up": "uk", "value_up": "uv", "sink": "sink", "gate": "g", "out": "o"}


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):

  graph_safe = True

  def __init__(self, prefix: str, width: int, num_heads: int, head_dim: int, rotated_dim: int, value_dim: int,
               query_rank: int, kv_rank: int, score_scale: float, eps: float, rotary: dict | None = None,
               window: int | None = None, sink: bool = True, output_gate: bool = True,
               names: dict[str, str] | None = None):
    self.prefix, self.width = prefix, width
    self.num_heads, self.head_dim, self.rotated_dim, self.value_dim = num_heads, head_dim, rotated_dim, value_dim
    self.query_rank, self.kv_rank = query_rank, kv_rank
    self.score_scale, self.eps = float(score_scale), float(eps)
    self.window = window
    self.rot_dims = int(rotary["dims"]) if rotary else 0
    self.rot_base = float(rotary["base"]) if rotary else 1.0
    if self.rot_dims % 2 or self.rot_dims > rotated_dim:
      raise ValueError(f"{prefix}: the rotation takes an even number of dims, at most rotated_dim")
    self.has_sink, self.has_gate = bool(sink), bool(output_gate)
    n = self.names = {**_NAMES, **(names or {})}
    p = prefix
    self.query_down = Linear(f"{p}.{n['query_down']}", query_rank, width)
    self.query_up = Linear(f"{p}.{n['query_up']}", num_heads * (head_dim + rotated_dim), query_rank)
    self.kv_down = Linear(f"{p}.{n['kv_down']}", kv_rank + rotated_dim, width)
    self.key_up = Linear(f"{p}.{n['key_up']}", num_heads * head_dim, kv_rank)
    self.value_up = Linear(f"{p}.{n['value_up']}", num_heads * value_dim, kv_rank)
    self.gate_proj = Linear(f"{p}.{n['gate']}", num_heads, width) if self.has_gate else None
    self.o_proj = Linear(f"{p}.{n['out']}", width, num_heads * value_dim)
    self.row_dim = kv_rank + rotated_dim  # what the cache holds per token

  def _name(self, role: str) -> str:
    return f"{self.prefix}.{self.names[role]}"

  def cache_need(self):
    return PagedKVNeed(1, self.row_dim, self.window, value_dim=self.kv_rank, values_in_keys=True)

  def tensor_specs(self) -> list[TensorSpec]:
    specs = [p.spec() for p in (self.query_down, self.query_up, self.kv_down, self.key_up, self.value_up,
                                self.gate_proj, self.o_proj) if p is not None]
    specs += [TensorSpec(self._name("query_norm"), (self.query_rank,), "gain"),
              TensorSpec(self._name("kv_norm"), (self.kv_rank,), "gain")]
    if self.has_sink:
      specs.append(TensorSpec(self._name("sink"), (self.num_heads,), "scale", precision="stored"))
    return specs

  def bind(self, tensors, ops) -> None:
    t = tensors
    down = [t[self.query_down.name], t[self.kv_down.name]] + ([t[self.gate_proj.name]] if self.has_gate else [])
    w = fuse_rows(down)  # c_q | c, k_r | gate, before norms and rotation
    extra = -w.shape[0] % 8
    self.down_weight = torch.cat([w, w.new_zeros(extra, w.shape[1])]).contiguous() if extra else w
    self.query_up.bind(t)
    self.o_proj.bind(t)
    # Per head: [head_dim, kv_rank] as stored turns q_plain into a vector over the latent (x . W, no
    # transpose), and [value_dim, kv_rank] expands a sum of latents (x . W^T).
    self.key_up_t = t[self.key_up.name].reshape(self.num_heads, self.head_dim, self.kv_rank).transpose(1, 2).contiguous()
    self.value_up_w = t[self.value_up.name].reshape(self.num_heads, self.value_dim, self.kv_rank).contiguous()
    self.query_norm = t[self._name("query_norm")].float().contiguous()
    self.kv_norm = t[self._name("kv_norm")].float().contiguous()
    self.sink = t[self._name("sink")].float().contiguous() if self.has_sink else None
    half = self.rot_dims // 2
    self.freq = None
    if half:
      i = torch.arange(half, dtype=torch.float64)
      self.freq = (self.rot_base ** (-2.0 * i / self.rot_dims)).to(torch.float32).to(self.query_norm.device)

  def forward(self, x: torch.Tensor, ctx: Any, cache: Any, writes_cache: bool = True) -> torch.Tensor:
    ops = ctx.ops
    table = ctx.block_tables[cache.group]
    down = ops.linear(x, self.down_weight)
    # norms of both latents, the shared key part turned, the token's row into its page
    cq = ops.latent_prepare(down, self.query_norm, self.kv_norm, self.eps, self.freq, query_rank=self.query_rank,
                            kv_rank=self.kv_rank, rotated_dim=self.rotated_dim,
                            storage=cache.storage if writes_cache else None, block_table=table, ctx=ctx)
    q = ops.linear(cq, self.query_up.weight)
    asked = ops.latent_queries(q, self.key_up_t, self.freq, self.score_scale, ctx, num_heads=self.num_heads,
                               head_dim=self.head_dim, rotated_dim=self.rotated_dim)
    mixed = ops.paged_attention(asked, cache.storage, table, ctx, num_heads=self.num_heads, num_kv_heads=1,
                                head_dim=self.row_dim, logit_softcap=0.0, window=self.window,
                                value_dim=self.kv_rank, values_in_keys=True, sink=self.sink)
    out = ops.head_linear(mixed, self.value_up_w)  # [T, heads * value_dim]
    if self.has_gate:
      out = ops.sigmoid_gate(out, down, self.query_rank + self.row_dim, per=self.value_dim)
    return self.o_proj(out, ctx)
