"""A pre-norm block whose residual stream is kept several times, with a short convolution on what
the mixer reads.

With `streams` = s > 0 the stream is s copies x_1 .. x_s (all equal to the embedding's output when
the first such block meets it).  Sublayer q (1: the mixer, 2: the feed-forward) has three learned
tensors `hc<q>.in` [s], `hc<q>.out` [s] and `hc<q>.mix` [s, s] (indexed [from, to]):

  u    = sum_s in[s] x_s
  y    = sublayer(norm_q(u))
  x_t <- sum_s mix[s, t] x_s + out[t] y        every copy from the old ones

and whoever reads the stream as one vector (the final norm) reads the sum of the copies.  With
`streams` = 0 there is one stream and x <- x + y.  All of this is float32; the write of one sublayer
and the read and norm of the next are one kernel.

With `input_conv_taps` = K > 0 the mixer reads h + conv(h) in place of h = norm_1(u), conv a causal
convolution over time per channel (`canon1` [width, K], the last column the current token's, zeros
before a sequence's start).  The last K - 1 rows of h are part of a request's state.
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.cache.needs import SlotStateNeed
from simply_b200.config.model_spec import PartSpec
from simply_b200.parts.base import Block, FeedForward, Mixer, Norm, build_part
from simply_b200.parts.block import ResidualStream
from simply_b200.parts.feedforward import NoFeedForward
from simply_b200.registry import BLOCKS, NORMS
from simply_b200.weights.loader import TensorSpec

_NAMES = {"pre_mixer": "norm1", "pre_feed_forward": "norm2", "conv": "canon1", "mixer_streams": "hc1",
          "feed_forward_streams": "hc2"}


@BLOCKS.register("hyper_connection")
class HyperConnectionBlock(Block):

  def __init__(self, prefix: str, width: int, norm: PartSpec, mixer: Mixer, feed_forward: FeedForward,
               streams: int = 0, input_conv_taps: int = 0, names: dict[str, str] | None = None):
    self.prefix, self.width = prefix, width
    self.mixer = mixer
    self.feed_forward = None if isinstance(feed_forward, NoFeedForward) else feed_forward
    self.streams, self.taps = int(streams), int(input_conv_taps)
    n = self.names = {**_NAMES, **(names or {})}

    def make(role: str) -> Norm:
      return build_part(NORMS, PartSpec(norm.kind, f"{prefix}.{n[role]}",
                                        {"width": width, **norm.params, "name": f"{prefix}.{n[role]}"}))
    self.pre_mixer = make("pre_mixer")
    self.pre_feed_forward = make("pre_feed_forward") if self.feed_forward is not None else None
    self.conv_weight: torch.Tensor | None = None
    self.lane_weights: dict[str, tuple] = {}

  def _sublayers(self) -> list[str]:
    return ["mixer_streams"] + (["feed_forward_streams"] if self.feed_forward is not None else [])

  def _parts(self) -> list:
    return [p for p in (self.mixer, self.feed_forward, self.pre_mixer, self.pre_feed_forward) if p is not None]

  def cache_need(self):
    needs = {}
    if self.mixer.cache_need() is not None:
      needs["mixer"] = self.mixer.cache_need()
    if self.taps > 1:
      needs["input_conv"] = SlotStateNeed((self.taps - 1, self.width), "float32")
    return needs

  @property
  def graph_safe(self) -> bool:
    return all(p.graph_safe for p in self._parts())

  def graph_plans(self, *args, **kwargs) -> list:
    return self.mixer.graph_plans(*args, **kwargs)

  def tensor_specs(self) -> list[TensorSpec]:
    specs = [s for p in self._parts() for s in p.tensor_specs()]
    if self.taps:
      specs.append(TensorSpec(f"{self.prefix}.{self.names['conv']}", (self.width, self.taps), "matrix"))
    if self.streams:
      s = self.streams
      for role in self._sublayers():
        p = f"{self.prefix}.{self.names[role]}"
        specs += [TensorSpec(f"{p}.in", (s,), "gain", precision="stored"),
                  TensorSpec(f"{p}.out", (s,), "gain", precision="stored"),
                  TensorSpec(f"{p}.mix", (s, s), "gain", precision="stored")]
    return specs

  def bind(self, tensors, ops) -> None:
    for p in self._parts():
      p.bind(tensors, ops)
    if self.taps:
      self.conv_weight = tensors[f"{self.prefix}.{self.names['conv']}"].float().contiguous()
    if self.streams:
      for role in self._sublayers():
        p = f"{self.prefix}.{self.names[role]}"
        self.lane_weights[role] = tuple(tensors[f"{p}.{k}"].float().contiguous() for k in ("in", "mix", "out"))

  def _read(self, stream: ResidualStream, role: str, norm: Norm, ctx: Any) -> torch.Tensor:
    if not self.streams:
      return stream.normed(norm, ctx)
    stream.spread(self.streams, ctx)
    return stream.read_lanes(self.lane_weights[role][0], norm, ctx)

  def _write(self, stream: ResidualStream, role: str, y: torch.Tensor, ctx: Any) -> None:
    if not self.streams:
      stream.add(y, None, ctx)
    else:
      _, mix, out = self.lane_weights[role]
      stream.write_lanes(y, mix, out, ctx)

  def forward(self, stream: ResidualStream, ctx: Any, cache: Any, writes_cache: bool = True) -> None:
    cache = cache or {}
    h = self._read(stream, "mixer_streams", self.pre_mixer, ctx)
    if self.taps > 1:
      h = ctx.ops.short_conv(h, self.conv_weight, None, cache["input_conv"].storage, ctx, activation=0, residual=True)
    elif self.taps == 1:
      h = ctx.ops.short_conv(h, self.conv_weight, None, None, ctx, activation=0, residual=True)
    self._write(stream, "mixer_streams", self.mixer.forward(h, ctx, cache.get("mixer"), writes_cache), ctx)
    if self.feed_forward is None:
      return
    h = self._read(stream, "feed_forward_streams", self.pre_feed_forward, ctx)
    self._write(stream, "feed_forward_streams", self.feed_forward.forward(h, ctx), ctx)
