"""Configuration of the Zesapel decoder, read from config.json.

config.json of this design:

  architecture     "Zesapel"
  vocab, width     sizes of the embedding table and of the residual stream
  embedding.scale  factor on the embedding rows (absent: 1)
  max_positions    rows of the learned position table `pos`, one of which is added per token; also
                   the longest sequence the engine serves
  decay_rank       (optional, this engine's own key) rank of the delta rule's w1 / w2 where no
                   folder of tensors gives it (random-weights mode)
  norm.eps         eps of every RMS norm
  streams          (optional) s: the residual stream is kept s times; every sublayer reads a learned
                   mix of the copies and writes back through learned matrices (block
                   `hyper_connection`); absent: one stream and plain residual sums
  canon.taps       (optional) a causal convolution over time on what each mixer reads,
                   h <- h + conv(h), with `taps` taps per channel
  layers           one entry per layer: `type` ("latent_attention", "general_delta" or "mamba2"),
                   `mixer` (its sizes) and `mlp` (a feed-forward, or null)

A layer is x <- x + mixer(norm1(x)), then x <- x + mlp(norm2(x)) (with streams: through the mix).
Tensor names: `embed`, `pos`, `l<i>.norm1|norm2`, `l<i>.canon1`, `l<i>.hc1|hc2.{in,out,mix}`,
`l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.

"latent_attention" (mixer `latent_attention`): heads, dim, rot_dim, vdim, q_rank, kv_rank, scale,
rot.{dims, base}, mask.size (absent: every earlier token is seen).  Tensors dq, dq.norm, uq, dkv,
dkv.norm, uk, uv, sink, g, o.
"general_delta" (mixer `generalized_delta_rule`): heads, dim.  Tensors r, k, v, g, a, a.b, w1, w2, w0,
norm, o (the rank of w1/w2 is the tensors' own).
"mamba2" (mixer `state_space_duality`): heads, vdim, state, groups, norm_groups, conv.  Tensors in,
conv, conv.b, dt_bias, A_log, D, norm, o.
mlp {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}} (feed-forward `table_experts`):
tensors e<j>.{up,down} and `table` [vocab, top] (integers).
"""

from __future__ import annotations

import copy
import dataclasses
from typing import Any

from simply_b200.config.gemma2 import ConfigError
from simply_b200.config.model_spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from simply_b200.registry import ARCHITECTURES

_MIXER_KEYS = {
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"),
    "general_delta": ("heads", "dim"),
    "mamba2": ("heads", "vdim", "state", "groups", "norm_groups", "conv"),
}


def _need(d: dict, key: str, where: str):
  if not isinstance(d, dict) or key not in d or d[key] is None:
    raise ConfigError(f"config.json: {where} lacks {key!r}")
  return d[key]


@dataclasses.dataclass(frozen=True)
class ZesapelConfig:
  vocab: int
  width: int
  eps: float
  max_positions: int
  layers: tuple[dict, ...]
  embedding_scale: float = 1.0
  streams: int = 0  # 0: one stream, plain residual sums
  canon_taps: int = 0  # 0: no convolution on the mixers' input
  decay_rank: int = -1  # rank of w1 / w2; -1: the folder's tensors give it (random-weights mode needs it named)
  bos_token_id: int | None = None
  eos_token_id: int | tuple[int, ...] | None = None

  architecture = "Zesapel"

  # ---- reading and writing ------------------------------------------------------
  @classmethod
  def from_dict(cls, d: dict[str, Any]) -> "ZesapelConfig":
    eos = d.get("eos_token_id")
    if isinstance(eos, list):
      eos = tuple(int(e) for e in eos)
    cfg = cls(
        vocab=int(_need(d, "vocab", "the model")), width=int(_need(d, "width", "the model")),
        eps=float(_need(_need(d, "norm", "the model"), "eps", "norm")),
        max_positions=int(_need(d, "max_positions", "the model")),
        layers=tuple(copy.deepcopy(l) for l in _need(d, "layers", "the model")),
        embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
        streams=int(d.get("streams") or 0), canon_taps=int((d.get("canon") or {}).get("taps") or 0),
        decay_rank=int(d.get("decay_rank") or -1),
        bos_token_id=d.get("bos_token_id"), eos_token_id=eos)
    cfg.validate()
    return cfg

  def to_dict(self) -> dict[str, Any]:
    d: dict[str, Any] = {
        "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
        "embedding": {"scale": self.embedding_scale}, "max_positions": self.max_positions,
        "norm": {"eps": self.eps}, "layers": [copy.deepcopy(l) for l in self.layers]}
    if self.decay_rank > 0:
      d["decay_rank"] = self.decay_rank
    if self.streams:
      d["streams"] = self.streams
    if self.canon_taps:
      d["canon"] = {"taps": self.canon_taps}
    if self.bos_token_id is not None:
      d["bos_token_id"] = self.bos_token_id
    if self.eos_token_id is not None:
      d["eos_token_id"] = list(self.eos_token_id) if isinstance(self.eos_token_id, tuple) else self.eos_token_id
    return d

  def replace(self, **changes: Any) -> "ZesapelConfig":
    cfg = dataclasses.replace(self, **changes)
    cfg.validate()
    return cfg

  # ---- checks -------------------------------------------------------------------
  def validate(self) -> None:
    if self.vocab <= 0 or self.width <= 0 or self.max_positions <= 0:
      raise ConfigError("vocab, width and max_positions must be positive")
    if not self.eps > 0:
      raise ConfigError("norm.eps must be positive")
    if self.streams < 0 or self.canon_taps < 0:
      raise ConfigError("streams and canon.taps must not be negative")
    if not self.layers:
      raise ConfigError("the model has no layers")
    for i, layer in enumerate(self.layers):
      where = f"layer {i}"
      kind = _need(layer, "type", where)
      if kind not in _MIXER_KEYS:
        raise ConfigError(f"{where}: unknown type {kind!r} (known: {', '.join(sorted(_MIXER_KEYS))})")
      m = _need(layer, "mixer", where)
      for key in _MIXER_KEYS[kind]:
        if int(_need(m, key, where)) <= 0:
          raise ConfigError(f"{where}: {key} must be positive")
      if kind == "latent_attention":
        _need(m, "scale", where)
        rot = m.get("rot")
        if rot:
          dims = int(_need(rot, "dims", f"{where} (rot)"))
          _need(rot, "base", f"{where} (rot)")
          if dims % 2 or dims < 0 or dims > m["rot_dim"]:
            raise ConfigError(f"{where}: rot.dims must be even and at most rot_dim")
        if m.get("mask") and int(_need(m["mask"], "size", f"{where} (mask)")) <= 0:
          raise ConfigError(f"{where}: mask.size must be positive")
      if kind == "mamba2":
        if m["heads"] % m["groups"]:
          raise ConfigError(f"{where}: heads must be a multiple of groups")
        if (m["heads"] * m["vdim"]) % m["norm_groups"]:
          raise ConfigError(f"{where}: norm_groups must divide heads * vdim")
      mlp = layer.get("mlp")
      if mlp is None:
        continue
      if mlp.get("kind") != "moe":
        raise ConfigError(f"{where}: unknown mlp kind {mlp.get('kind')!r} (known: moe)")
      r = _need(mlp, "router", f"{where} (mlp)")
      experts, top = int(_need(r, "experts", f"{where} (router)")), int(_need(r, "top", f"{where} (router)"))
      if not 1 <= top <= experts:
        raise ConfigError(f"{where}: each token uses between 1 and `experts` experts")
      if int(_need(_need(mlp, "expert", f"{where} (mlp)"), "ff", f"{where} (expert)")) <= 0:
        raise ConfigError(f"{where}: the experts' ff must be positive")

  # ---- derived --------------------------------------------------------------------
  def _mixer_spec(self, p: str, kind: str, m: dict) -> PartSpec:
    if kind == "latent_attention":
      rot = m.get("rot")
      rotary = None
      if rot and int(rot["dims"]) > 0:
        rotary = {"dims": int(rot["dims"]), "base": float(rot["base"])}
      mask = m.get("mask")
      return PartSpec("latent_attention", f"{p}.mix", {
          "width": self.width, "num_heads": int(m["heads"]), "head_dim": int(m["dim"]),
          "rotated_dim": int(m["rot_dim"]), "value_dim": int(m["vdim"]), "query_rank": int(m["q_rank"]),
          "kv_rank": int(m["kv_rank"]), "score_scale": float(m["scale"]), "rotary": rotary,
          "window": int(mask["size"]) if mask else None, "eps": self.eps, "sink": True, "output_gate": True})
    if kind == "general_delta":
      return PartSpec("generalized_delta_rule", f"{p}.mix", {
          "width": self.width, "num_heads": int(m["heads"]), "head_dim": int(m["dim"]), "eps": self.eps,
          "decay_rank": self.decay_rank})
    return PartSpec("state_space_duality", f"{p}.mix", {
        "width": self.width, "num_heads": int(m["heads"]), "value_dim": int(m["vdim"]),
        "state_dim": int(m["state"]), "num_groups": int(m["groups"]), "norm_groups": int(m["norm_groups"]),
        "conv_taps": int(m["conv"]), "eps": self.eps})

  def _mlp_spec(self, p: str, mlp: dict | None) -> PartSpec:
    if mlp is None:
      return PartSpec("none", f"{p}.mlp")
    r = mlp["router"]
    return PartSpec("table_experts", f"{p}.mlp", {
        "width": self.width, "hidden": int(mlp["expert"]["ff"]), "num_experts": int(r["experts"]),
        "top": int(r["top"]), "vocab_size": self.vocab, "activation": "gelu_erf"})

  def model_spec(self) -> ModelSpec:
    norm = PartSpec("rms_norm", params={"eps": self.eps, "plus_one": False})
    layers = []
    for i, layer in enumerate(self.layers):
      p = f"l{i}"
      block = PartSpec("hyper_connection", p, {
          "width": self.width, "norm": norm, "streams": self.streams, "input_conv_taps": self.canon_taps})
      layers.append(LayerSpec(p, block, self._mixer_spec(p, layer["type"], layer["mixer"]),
                              self._mlp_spec(p, layer.get("mlp"))))
    spec = ModelSpec(
        architecture=self.architecture, vocab_size=self.vocab, width=self.width, max_context=self.max_positions,
        embedding=PartSpec("token_embedding", "embed", {
            "vocab_size": self.vocab, "width": self.width, "scale": self.embedding_scale, "name": "embed",
            "position_table": "pos", "max_positions": self.max_positions, "round_scale": False}),
        layers=tuple(layers), run_order=tuple(LayerCall(f"l{i}") for i in range(len(self.layers))),
        final_norm=PartSpec("rms_norm", "final", {"width": self.width, "eps": self.eps, "plus_one": False,
                                                  "name": "final.norm"}),
        head=PartSpec("linear_head", "head", {"logit_softcap": 0.0, "name": "head"}))
    spec.validate()
    return spec


ARCHITECTURES.register(ZesapelConfig.architecture, ZesapelConfig)
