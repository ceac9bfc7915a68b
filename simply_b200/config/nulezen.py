"""Configuration of the Nulezen decoder, read from config.json.

config.json of this design:

  architecture      "Nulezen"
  vocab, width      sizes of the embedding table and of the residual stream
  embedding.scale   the factor on a token's row of the table
  logit_scale       the factor on the logits; the output layer is the embedding table itself
  norm.eps          kept for the folder's sake: the design's norm (y = tanh(alpha x) w + b) has no eps
  layers            one entry per layer: `type` ("attention" or "attention_2"), `mixer` (its sizes)
                    and `mlp` (a feed-forward, or null)
  loop              (optional) {start, stop, times}: layers start .. stop - 1 run `times` times in a
                    row with the same weights and a cache of its own per pass.  Before every pass,
                    the first too, x <- W_in [x; x0] + step[pass] with x0 the embedding's output
                    (tensors `loop.in` [width, 2 width] and `loop.step` [times, width])
  max_context       (optional) the longest sequence the engine will serve; the design has no limit

A layer is `x += ls1 * mixer(y) + ls2 * mlp(y)` with y = norm1(x) (block `parallel_residual` with
branch scales, norm `dynamic_tanh`).  Tensor names: `embed`, `l<i>.norm1` (`.alpha`, `.b` beside
it), `l<i>.ls1|ls2`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`.

Both mixer types are the mixer `head_norm_attention` without its norm: heads, kv_heads, dim, vdim,
scale, mask.size (the window: a query sees itself and the mask.size - 1 tokens before it).
"attention": no rotation, the score loses r1_h log(1 + r2_h distance) (tensors r1, r2), a gate per
element of the heads' results (tensor g [heads * vdim, width]).  "attention_2": biases on q, k, v
(`q.b`, ...), rot.{dims, base} (halves pair up), a gate per head (g [heads, width]).

mlp: {"kind": "dense", "ff"} (feed-forward `learned_activation`: up, down, act) or {"kind": "moe",
"expert": {"ff", "limit"}, "router": {"experts", "top"}, "shared": {"ff", "limit"} or absent}
(feed-forward `routed_experts`: e<j>.{gate,up,down}, router, router.b, shared.{gate,up,down}).
"""

from __future__ import annotations

import copy
import dataclasses
from typing import Any

from simply_b200.config.gemma2 import ConfigError
from simply_b200.config.model_spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from simply_b200.registry import ARCHITECTURES

_DEFAULT_MAX_CONTEXT = 1 << 17
_MIXERS = ("attention", "attention_2")


def _need(d: dict, key: str, where: str):
  if not isinstance(d, dict) or key not in d or d[key] is None:
    raise ConfigError(f"config.json: {where} lacks {key!r}")
  return d[key]


@dataclasses.dataclass(frozen=True)
class NulezenConfig:
  vocab: int
  width: int
  embedding_scale: float
  logit_scale: float
  eps: float
  layers: tuple[dict, ...]
  loop: tuple[int, int, int] | None = None  # start, stop, times
  max_context: int = _DEFAULT_MAX_CONTEXT
  bos_token_id: int | None = None
  eos_token_id: int | tuple[int, ...] | None = None

  architecture = "Nulezen"

  # ---- reading and writing ------------------------------------------------------
  @classmethod
  def from_dict(cls, d: dict[str, Any]) -> "NulezenConfig":
    eos = d.get("eos_token_id")
    if isinstance(eos, list):
      eos = tuple(int(e) for e in eos)
    loop = d.get("loop")
    if loop:
      loop = (int(_need(loop, "start", "loop")), int(_need(loop, "stop", "loop")), int(_need(loop, "times", "loop")))
    cfg = cls(
        vocab=int(_need(d, "vocab", "the model")), width=int(_need(d, "width", "the model")),
        embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
        logit_scale=float(d["logit_scale"]) if d.get("logit_scale") is not None else 1.0,
        eps=float((d.get("norm") or {}).get("eps", 0.0)),
        layers=tuple(copy.deepcopy(l) for l in _need(d, "layers", "the model")),
        loop=loop or None,
        max_context=int(d.get("max_context") or _DEFAULT_MAX_CONTEXT),
        bos_token_id=d.get("bos_token_id"), eos_token_id=eos)
    cfg.validate()
    return cfg

  def to_dict(self) -> dict[str, Any]:
    d: dict[str, Any] = {
        "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
        "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale,
        "norm": {"eps": self.eps}, "layers": [copy.deepcopy(l) for l in self.layers],
        "max_context": self.max_context}
    if self.loop is not None:
      d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
    if self.bos_token_id is not None:
      d["bos_token_id"] = self.bos_token_id
    if self.eos_token_id is not None:
      d["eos_token_id"] = list(self.eos_token_id) if isinstance(self.eos_token_id, tuple) else self.eos_token_id
    return d

  def replace(self, **changes: Any) -> "NulezenConfig":
    cfg = dataclasses.replace(self, **changes)
    cfg.validate()
    return cfg

  # ---- checks -------------------------------------------------------------------
  def validate(self) -> None:
    if self.vocab <= 0 or self.width <= 0 or self.max_context <= 0:
      raise ConfigError("vocab, width and max_context must be positive")
    if not self.layers:
      raise ConfigError("the model has no layers")
    if self.loop is not None:
      start, stop, times = self.loop
      if not (0 <= start <= stop <= len(self.layers)) or times < 1:
        raise ConfigError(f"loop {self.loop} does not fit {len(self.layers)} layers (0 <= start <= stop, times >= 1)")
    for i, layer in enumerate(self.layers):
      where = f"layer {i}"
      kind = _need(layer, "type", where)
      if kind not in _MIXERS:
        raise ConfigError(f"{where}: unknown type {kind!r} (known: {', '.join(_MIXERS)})")
      m = _need(layer, "mixer", where)
      for key in ("heads", "kv_heads", "dim", "vdim"):
        if int(_need(m, key, where)) <= 0:
          raise ConfigError(f"{where}: {key} must be positive")
      _need(m, "scale", where)
      if int(_need(_need(m, "mask", where), "size", f"{where} (mask)")) <= 0:
        raise ConfigError(f"{where}: mask.size must be positive")
      if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{where}: heads must be a multiple of kv_heads")
      rot = m.get("rot")
      if rot and kind == "attention_2":
        dims = int(_need(rot, "dims", f"{where} (rot)"))
        _need(rot, "base", f"{where} (rot)")
        if dims % 2 or dims < 0 or dims > m["dim"]:
          raise ConfigError(f"{where}: rot.dims must be even and at most dim")
      mlp = layer.get("mlp")
      if mlp is None:
        continue
      if mlp.get("kind") == "dense":
        if int(_need(mlp, "ff", f"{where} (mlp)")) <= 0:
          raise ConfigError(f"{where}: ff must be positive")
      elif mlp.get("kind") == "moe":
        r = _need(mlp, "router", f"{where} (mlp)")
        experts, top = int(_need(r, "experts", f"{where} (router)")), int(_need(r, "top", f"{where} (router)"))
        if not 1 <= top <= experts:
          raise ConfigError(f"{where}: the router must choose between 1 and `experts` experts")
        e = _need(mlp, "expert", f"{where} (mlp)")
        if int(_need(e, "ff", f"{where} (expert)")) <= 0 or not float(_need(e, "limit", f"{where} (expert)")) > 0:
          raise ConfigError(f"{where}: the experts' ff and limit must be positive")
        s = mlp.get("shared")
        if s and (int(_need(s, "ff", f"{where} (shared)")) <= 0 or not float(_need(s, "limit", f"{where} (shared)")) > 0):
          raise ConfigError(f"{where}: the shared expert's ff and limit must be positive")
      else:
        raise ConfigError(f"{where}: unknown mlp kind {mlp.get('kind')!r} (known: dense, moe)")

  # ---- derived --------------------------------------------------------------------
  def _mixer_spec(self, p: str, kind: str, m: dict) -> PartSpec:
    params: dict[str, Any] = {
        "width": self.width, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
        "head_dim": int(m["dim"]), "value_dim": int(m["vdim"]), "score_scale": float(m["scale"]), "eps": 0.0,
        "window": int(m["mask"]["size"]), "head_norm": False, "tie_values": False, "output_gate": True}
    if kind == "attention":
      params.update(distance_bias=True, gate_per_head=False, rotary=None)
    else:
      rot = m.get("rot")
      rotary = None
      if rot and int(rot["dims"]) > 0:
        rotary = {"dims": int(rot["dims"]), "base": float(rot["base"]), "layout": "halves"}
      params.update(projection_bias=True, gate_per_head=True, rotary=rotary)
    return PartSpec("head_norm_attention", f"{p}.mix", params)

  def _mlp_spec(self, p: str, mlp: dict | None) -> PartSpec:
    if mlp is None:
      return PartSpec("none", f"{p}.mlp")
    if mlp["kind"] == "dense":
      return PartSpec("learned_activation", f"{p}.mlp", {
          "width": self.width, "hidden": int(mlp["ff"]), "activation": "xielu"})
    r, shared = mlp["router"], mlp.get("shared")
    return PartSpec("routed_experts", f"{p}.mlp", {
        "width": self.width, "hidden": int(mlp["expert"]["ff"]), "num_experts": int(r["experts"]),
        "top": int(r["top"]), "activation": "clamped_swish", "limit": float(mlp["expert"]["limit"]),
        "score": "softmax", "renormalize": True, "router_bias": True,
        "shared_hidden": int(shared["ff"]) if shared else 0,
        "shared_limit": float(shared["limit"]) if shared else None})

  def model_spec(self) -> ModelSpec:
    norm = PartSpec("dynamic_tanh")
    layers = []
    for i, layer in enumerate(self.layers):
      p = f"l{i}"
      block = PartSpec("parallel_residual", p, {
          "width": self.width, "norm": norm, "names": {"norm": "norm1"},
          "branch_scales": {"mixer": "ls1", "feed_forward": "ls2"}})
      layers.append(LayerSpec(p, block, self._mixer_spec(p, layer["type"], layer["mixer"]),
                              self._mlp_spec(p, layer.get("mlp"))))
    n = len(self.layers)
    inputs = {}
    if self.loop is None:
      order = [LayerCall(f"l{i}") for i in range(n)]
    else:
      start, stop, times = self.loop
      inputs["loop"] = PartSpec("projected_input", "loop", {"width": self.width, "passes": times})
      order = [LayerCall(f"l{i}") for i in range(start)]
      for rep in range(times):
        order += [LayerCall(f"l{i}", stream_input=("loop", rep) if i == start else None) for i in range(start, stop)]
      order += [LayerCall(f"l{i}") for i in range(stop, n)]
    spec = ModelSpec(
        architecture=self.architecture, vocab_size=self.vocab, width=self.width, max_context=self.max_context,
        embedding=PartSpec("token_embedding", "embed", {
            "vocab_size": self.vocab, "width": self.width, "scale": self.embedding_scale, "name": "embed",
            "round_scale": False}),
        layers=tuple(layers), run_order=tuple(order), stream_inputs=inputs,
        final_norm=PartSpec("dynamic_tanh", "final", {"width": self.width, "name": "final.norm"}),
        head=PartSpec("tied_head", "head", {"logit_scale": self.logit_scale}))
    spec.validate()
    return spec


ARCHITECTURES.register(NulezenConfig.architecture, NulezenConfig)
