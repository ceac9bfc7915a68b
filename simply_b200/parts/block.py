"""Block arrangements and the residual stream they act on.

The residual stream is kept in float32 whatever the activation dtype.  A branch
is not added at once: it stays *pending* together with its post-norm until the
next reader of the stream asks for a normed view.  Then one fused kernel adds
norm_post(branch) to the stream and norms the sum for the reader, so the stream
is read and written once per branch.

`sandwich_norm` is the reference's block with use_pre_ln and use_post_ln
(simply/model_lib.py:2659-2708; simply/config_lib.py:868-870):
  h += post_mixer_norm(mixer(pre_mixer_norm(h)))
  h += post_ff_norm(feed_forward(pre_ff_norm(h)))
With `residual_scale` = m both branches are added times m (folded into the post norms' scales),
and a layer without a feed-forward has only the first line.
`pre_norm` is the same without post norms (use_post_ln=False).
`parallel_residual` has one norm whose output both sublayers read:
  h += mixer(norm(h)) + feed_forward(norm(h))
With `branch_scales` each result is first multiplied by a learned factor per channel:
  h += s_mixer * mixer(norm(h)) + s_ff * feed_forward(norm(h))
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.config.model_spec import PartSpec
from simply_b200.parts.base import Block, FeedForward, Mixer, Norm, build_part
from simply_b200.parts.feedforward import NoFeedForward
from simply_b200.parts.norm import ChannelScale, DynamicTanh, RMSNorm
from simply_b200.registry import BLOCKS, NORMS
from simply_b200.weights.loader import TensorSpec


class ResidualStream:
  """float32 [T, width] plus what is still to be added: a branch with its post-norm, and beside it a
  second branch that is added as it is (the two sublayers of a block whose norm they share)."""

  def __init__(self, h: torch.Tensor):
    self.h = h
    self._branch: torch.Tensor | None = None
    self._post: Norm | None = None
    self._second: torch.Tensor | None = None
    self._second_post: Norm | None = None
    # A stream that is kept several times (`hyper_connection` blocks): float32 [T, copies, width]
    # in place of `h`, and the write that is still to be done (branch, mix [from, to], out [to]).
    self.lanes: torch.Tensor | None = None
    self._lane_write: tuple | None = None

  # ---- a stream kept several times ------------------------------------------------------------
  def spread(self, copies: int, ctx: Any) -> None:
    """From here on the stream is `copies` equal copies of what it holds now."""
    if self.lanes is None:
      self.flush(ctx)
      self.lanes = ctx.ops.spread_streams(self.h, copies)
      self.h = None
    elif self.lanes.shape[1] != copies:
      raise ValueError(f"the stream is kept {self.lanes.shape[1]} times, a block wants {copies}")

  def write_lanes(self, branch: torch.Tensor, mix: torch.Tensor, out: torch.Tensor, ctx: Any) -> None:
    """copy_t <- sum_s mix[s, t] copy_s + out[t] * branch, done when the stream is next read."""
    self.flush(ctx)
    self._lane_write = (branch, mix, out)

  def read_lanes(self, weights: torch.Tensor | None, norm: Norm | None, ctx: Any,
                 rows: torch.Tensor | None = None) -> torch.Tensor | None:
    """norm(sum_s weights[s] copy_s) in the activation dtype after the pending write, in one kernel."""
    branch, mix, out = self._lane_write or (None, None, None)
    if norm is not None and not isinstance(norm, RMSNorm):
      raise TypeError("a stream kept several times is read through an RMS norm")
    y = ctx.ops.streams_step(self.lanes, branch, mix, out, weights, norm.weight if norm is not None else None,
                             norm.eps if norm is not None else 0.0, bool(norm.plus_one) if norm is not None else False,
                             rows)
    if rows is None:
      self._lane_write = None
    return y

  def total(self, ctx: Any) -> torch.Tensor:
    """The stream as one float32 [T, width] (the sum of its copies); a new tensor."""
    self.flush(ctx)
    return self.h.clone() if self.lanes is None else self.lanes.sum(dim=1)

  def add(self, branch: torch.Tensor, post_norm: Norm | None, ctx: Any) -> None:
    if self._branch is not None and self._second is None and (
        post_norm is None or (isinstance(post_norm, ChannelScale) and isinstance(self._post, (ChannelScale, type(None))))):
      self._second, self._second_post = branch, post_norm  # rides along: h + first + second in one kernel
      return
    self.flush(ctx)
    self._branch, self._post = branch, post_norm

  def add_input(self, x: torch.Tensor, ctx: Any) -> None:
    """Adds `x` as it is: in the activation dtype it rides along with what is pending, in float32
    (when the activation dtype would round it) it is added at once."""
    if x.dtype == self.h.dtype and x.dtype != ctx.ops.dtype:
      self.flush(ctx)
      ctx.ops.add_to_residual(self.h, x)
    else:
      self.add(x, None, ctx)

  def flush(self, ctx: Any) -> None:
    if self._lane_write is not None:
      self.read_lanes(None, None, ctx)
    if self._branch is not None:
      self._combine(None, ctx, None)

  def normed(self, norm: Norm, ctx: Any, rows: torch.Tensor | None = None) -> torch.Tensor:
    """norm(h + pending) in the activation dtype.  With `rows`, only those rows are
    computed and returned (the stream is then left as it is: use this last)."""
    if self.lanes is not None:
      return self.read_lanes(self._ones(ctx), norm, ctx, rows)
    return self._combine(norm, ctx, rows)

  def _ones(self, ctx: Any) -> torch.Tensor:
    key = ("stream_ones", self.lanes.shape[1])
    if key not in ctx.memo:
      ctx.memo[key] = torch.ones(self.lanes.shape[1], dtype=torch.float32, device=self.lanes.device)
    return ctx.memo[key]

  def _combine(self, pre: Norm | None, ctx: Any, rows: torch.Tensor | None):
    ops = ctx.ops
    branch, post, second, second_post = self._branch, self._post, self._second, self._second_post
    fusable = ((post is None or isinstance(post, RMSNorm)) and (pre is None or isinstance(pre, RMSNorm))
               and second_post is None)
    scaled = (isinstance(post, (ChannelScale, type(None))) and isinstance(second_post, (ChannelScale, type(None)))
              and isinstance(pre, (DynamicTanh, type(None)))
              and (isinstance(pre, DynamicTanh) or post is not None or second_post is not None))
    if scaled:
      # Branches times a factor per channel, then tanh(alpha h) w + b for the reader: one kernel.
      out = ops.scaled_residual_tanh(self.h, branch, post.weight if post is not None else None, second,
                                     second_post.weight if second_post is not None else None, pre, rows)
    elif fusable and second is None:
      out = ops.residual_norm(self.h, branch, post, pre, rows)
    elif fusable:
      out = ops.residual_norm(self.h, branch, post, pre, rows, branch2=second)
    else:
      # Norms the fused kernel does not know: compose from their own `apply`.
      if rows is not None:
        h = ops.gather_rows(self.h, rows)
        branch = ops.gather_rows(branch, rows) if branch is not None else None
        second = ops.gather_rows(second, rows) if second is not None else None
      else:
        h = self.h
      if branch is not None:
        ops.add_to_residual(h, post.apply(branch, ctx) if post is not None else branch)
      if second is not None:
        ops.add_to_residual(h, second_post.apply(second, ctx) if second_post is not None else second)
      out = pre.apply(h, ctx) if pre is not None else None
    if rows is None:
      self._branch = self._post = self._second = self._second_post = None
    return out


@BLOCKS.register("sandwich_norm")
class SandwichNormBlock(Block):

  uses_post_norms = True

  def __init__(self, prefix: str, width: int, norm: PartSpec, mixer: Mixer, feed_forward: FeedForward,
               names: dict[str, str] | None = None, residual_scale: float = 1.0, full_names: bool = False):
    self.prefix = prefix
    self.mixer = mixer
    self.feed_forward = None if isinstance(feed_forward, NoFeedForward) else feed_forward
    self.residual_scale = float(residual_scale)
    if self.residual_scale != 1.0 and not self.uses_post_norms:
      raise ValueError(f"{prefix}: a residual scale needs post norms to carry it")
    names = names or {}
    def make(role: str) -> Norm:
      params = {"width": width, **norm.params}
      if full_names:  # `names` gives the scale's whole name after the layer's prefix
        params["name"] = f"{prefix}.{names.get(role, role)}"
      return build_part(NORMS, PartSpec(norm.kind, f"{prefix}.{names.get(role, role)}", params))
    has_ff = self.feed_forward is not None
    self.pre_mixer = make("pre_mixer")
    self.pre_feed_forward = make("pre_feed_forward") if has_ff else None
    self.post_mixer = make("post_mixer") if self.uses_post_norms else None
    self.post_feed_forward = make("post_feed_forward") if self.uses_post_norms and has_ff else None

  def _norms(self) -> list[Norm]:
    return [n for n in (self.pre_mixer, self.post_mixer, self.pre_feed_forward,
                        self.post_feed_forward) if n is not None]

  def cache_need(self):
    return self.mixer.cache_need()

  @property
  def graph_safe(self) -> bool:
    return (self.mixer.graph_safe and (self.feed_forward is None or self.feed_forward.graph_safe)
            and all(n.graph_safe for n in self._norms()))

  def tensor_specs(self) -> list[TensorSpec]:
    specs = self.mixer.tensor_specs() + (self.feed_forward.tensor_specs() if self.feed_forward is not None else [])
    for n in self._norms():
      specs += n.tensor_specs()
    return specs

  def bind(self, tensors, ops) -> None:
    self.mixer.bind(tensors, ops)
    if self.feed_forward is not None:
      self.feed_forward.bind(tensors, ops)
    for n in self._norms():
      n.bind(tensors, ops)
    if self.residual_scale != 1.0:
      # m * (x / rms(x) * w) = x / rms(x) * (m w): the branch's factor lives in the post norm's
      # scale, in float32 (with a scale applied as 1 + w: 1 + w' = m (1 + w)).
      for n in (self.post_mixer, self.post_feed_forward):
        if n is not None:
          w = n.weight.float()
          n.weight = ((w + 1.0) * self.residual_scale - 1.0 if n.plus_one else w * self.residual_scale).contiguous()

  def forward(self, stream: ResidualStream, ctx: Any, cache: Any, writes_cache: bool = True) -> None:
    y = stream.normed(self.pre_mixer, ctx)
    stream.add(self.mixer.forward(y, ctx, cache, writes_cache), self.post_mixer, ctx)
    if self.feed_forward is None:
      return
    y = stream.normed(self.pre_feed_forward, ctx)
    stream.add(self.feed_forward.forward(y, ctx), self.post_feed_forward, ctx)


@BLOCKS.register("pre_norm")
class PreNormBlock(SandwichNormBlock):

  uses_post_norms = False


@BLOCKS.register("parallel_residual")
class ParallelResidualBlock(Block):
  """One norm; the mixer and the feed-forward (if the layer has one) both read its output, and both
  results are added to the stream."""

  def __init__(self, prefix: str, width: int, norm: PartSpec, mixer: Mixer, feed_forward: FeedForward,
               names: dict[str, str] | None = None, branch_scales: dict[str, str] | None = None):
    """`branch_scales`: {"mixer": name, "feed_forward": name}, tensors [width] after the layer's
    prefix by which the sublayers' results are multiplied before they join the stream."""
    self.prefix = prefix
    self.mixer = mixer
    self.feed_forward = None if isinstance(feed_forward, NoFeedForward) else feed_forward
    params = {"width": width, **norm.params}
    role = (names or {}).get("norm")
    if role is not None:
      params["name"] = f"{prefix}.{role}"  # the scale's whole tensor name
    self.norm = build_part(NORMS, PartSpec(norm.kind, f"{prefix}.norm", params))
    scales = branch_scales or {}
    def scale(role: str):
      if role not in scales:
        return None
      return ChannelScale(f"{prefix}.{scales[role]}", width, name=f"{prefix}.{scales[role]}")
    self.mixer_scale = scale("mixer")
    self.feed_forward_scale = scale("feed_forward") if self.feed_forward is not None else None

  def _parts(self) -> list:
    return [p for p in (self.mixer, self.feed_forward, self.norm, self.mixer_scale, self.feed_forward_scale)
            if p is not None]

  def cache_need(self):
    return self.mixer.cache_need()

  @property
  def graph_safe(self) -> bool:
    return all(p.graph_safe for p in self._parts())

  def tensor_specs(self) -> list[TensorSpec]:
    return [s for p in self._parts() for s in p.tensor_specs()]

  def bind(self, tensors, ops) -> None:
    for p in self._parts():
      p.bind(tensors, ops)

  def forward(self, stream: ResidualStream, ctx: Any, cache: Any, writes_cache: bool = True) -> None:
    y = stream.normed(self.norm, ctx)
    stream.add(self.mixer.forward(y, ctx, cache, writes_cache), self.mixer_scale, ctx)
    if self.feed_forward is not None:
      stream.add(self.feed_forward.forward(y, ctx), self.feed_forward_scale, ctx)
