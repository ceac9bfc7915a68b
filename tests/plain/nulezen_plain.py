"""The Nulezen decoder in plain NumPy, float64, whole sequences, one function per mechanism.

A yardstick for the tests: it shares no code with the engine, keeps no cache (every call runs a
whole sequence from its first token) and takes its weights as a dictionary name -> array.

The design in short.  x = table[token] * s.  Layers run in the order of the configuration; a run
of layers may be walked several times with the same weights, and before every walk (the first
too) the stream is mixed with the embedding's output again, x <- W_in [x; x0] + step[walk].  A
layer reads y = dyt(x) once and adds both sublayers: x <- x + ls1 * mixer(y) + ls2 * ff(y).
dyt(x) = tanh(alpha x) * w + b.  Mixers: windowed attention whose scores lose
r1_h * log(1 + r2_h * distance) and whose heads side by side pass a sigmoid gate per element;
and windowed attention with biases on q, k, v, partly rotated heads (halves pair up) and one
sigmoid gate per head.  Feed-forwards: W_down xielu(W_up y), or routed experts (logits with a bias,
the `top` largest, softmax over those alone) with a clamped activation beside a shared expert.
"""

from __future__ import annotations

import numpy as np


def dyt(x, alpha, w, b):
  return np.tanh(float(alpha) * x) * w + b


def softplus(z):
  return np.log1p(np.exp(-abs(z))) + max(z, 0.0)


def sigmoid(z):
  return 1.0 / (1.0 + np.exp(-z))


def xielu(z, p, q):
  """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z/2."""
  ap, an = softplus(float(p)), 0.5 + softplus(float(q))
  zn = np.minimum(z, 0.0)
  return np.where(z > 0, ap * z * z + 0.5 * z, an * (np.expm1(zn) - zn) + 0.5 * z)


def clamped_expert(y, gate, up, down, limit):
  g = np.minimum(y @ gate.T, limit)
  u = np.clip(y @ up.T, -limit, limit)
  return (g * sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def rotate_halves(x, positions, dims, base):
  """x [T, heads, d]: dim i pairs with i + dims/2 for i < dims/2, angle p * base^(-2i/dims)."""
  if not dims:
    return x
  half = dims // 2
  freq = base ** (-2.0 * np.arange(half) / dims)
  ang = positions[:, None, None] * freq[None, None, :]
  c, s = np.cos(ang), np.sin(ang)
  out = x.copy()
  a, b = x[..., :half], x[..., half:dims]
  out[..., :half] = a * c - b * s
  out[..., half:dims] = b * c + a * s
  return out


def windowed_attention(q, k, v, scale, window, distance_bias=None):
  """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]; i sees j with 0 <= i - j < window.
  distance_bias = (r1 [H], r2 [H]): the score loses r1 log(1 + r2 (i - j))."""
  t, heads, _ = q.shape
  group = heads // k.shape[1]
  i = np.arange(t)[:, None]
  j = np.arange(t)[None, :]
  dist = (i - j).astype(np.float64)
  seen = (dist >= 0) & (dist < window)
  out = np.zeros((t, heads, v.shape[2]))
  for h in range(heads):
    s = (q[:, h] @ k[:, h // group].T) * scale
    if distance_bias is not None:
      s = s - distance_bias[0][h] * np.log1p(distance_bias[1][h] * np.maximum(dist, 0.0))
    s = np.where(seen, s, -np.inf)
    s = s - s.max(axis=1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(axis=1, keepdims=True)
    out[:, h] = p @ v[:, h // group]
  return out


def attention_mixer(y, w, p, m, kind):
  """`kind` "attention": distance bias, a gate per element.  "attention_2": biases, rotation, a gate per head."""
  t = y.shape[0]
  heads, kv, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
  q, k, v = y @ w[f"{p}.q"].T, y @ w[f"{p}.k"].T, y @ w[f"{p}.v"].T
  positions = np.arange(t, dtype=np.float64)
  bias = None
  if kind == "attention_2":
    q, k, v = q + w[f"{p}.q.b"], k + w[f"{p}.k.b"], v + w[f"{p}.v.b"]
  else:
    bias = (w[f"{p}.r1"], w[f"{p}.r2"])
  q, k, v = q.reshape(t, heads, d), k.reshape(t, kv, d), v.reshape(t, kv, dv)
  if kind == "attention_2":
    rot = m.get("rot") or {}
    q = rotate_halves(q, positions, int(rot.get("dims", 0)), float(rot.get("base", 1.0)))
    k = rotate_halves(k, positions, int(rot.get("dims", 0)), float(rot.get("base", 1.0)))
  o = windowed_attention(q, k, v, float(m["scale"]), int(m["mask"]["size"]), bias)
  gate = sigmoid(y @ w[f"{p}.g"].T)
  if kind == "attention_2":
    o = o * gate[:, :, None]
  else:
    o = o * gate.reshape(t, heads, dv)
  return o.reshape(t, heads * dv) @ w[f"{p}.o"].T


def dense_ff(y, w, p):
  act = w[f"{p}.act"]
  return xielu(y @ w[f"{p}.up"].T, act[0], act[1]) @ w[f"{p}.down"].T


def route(y, router, bias, top):
  """The `top` experts with the largest logits, and the softmax over their logits alone."""
  z = y @ router.T + bias
  chosen = np.argsort(-z, axis=1, kind="stable")[:, :top]
  zc = np.take_along_axis(z, chosen, axis=1)
  e = np.exp(zc - zc.max(axis=1, keepdims=True))
  return chosen, e / e.sum(axis=1, keepdims=True)


def moe_ff(y, w, p, mlp):
  top, limit = int(mlp["router"]["top"]), float(mlp["expert"]["limit"])
  chosen, weight = route(y, w[f"{p}.router"], w[f"{p}.router.b"], top)
  out = np.zeros((y.shape[0], w[f"{p}.e0.down"].shape[0]))
  for t in range(y.shape[0]):
    for j in range(top):
      e = int(chosen[t, j])
      out[t] += weight[t, j] * clamped_expert(y[t:t + 1], w[f"{p}.e{e}.gate"], w[f"{p}.e{e}.up"],
                                              w[f"{p}.e{e}.down"], limit)[0]
  shared = mlp.get("shared")
  if shared:
    out += clamped_expert(y, w[f"{p}.shared.gate"], w[f"{p}.shared.up"], w[f"{p}.shared.down"],
                          float(shared["limit"]))
  return out


def layer(x, w, i, spec):
  p = f"l{i}"
  y = dyt(x, w[f"{p}.norm1.alpha"], w[f"{p}.norm1"], w[f"{p}.norm1.b"])
  add = w[f"{p}.ls1"] * attention_mixer(y, w, f"{p}.mix", spec["mixer"], spec["type"])
  mlp = spec.get("mlp")
  if mlp is not None:
    ff = dense_ff(y, w, f"{p}.mlp") if mlp["kind"] == "dense" else moe_ff(y, w, f"{p}.mlp", mlp)
    add = add + w[f"{p}.ls2"] * ff
  return x + add


def run_order(config):
  """[(layer index, walk number or None for a layer outside the loop, first of its walk)]."""
  n = len(config["layers"])
  loop = config.get("loop") or {"start": 0, "stop": 0, "times": 1}
  start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
  order = [(i, None, False) for i in range(start)]
  if stop > start:
    for walk in range(times):
      order += [(i, walk, i == start) for i in range(start, stop)]
  order += [(i, None, False) for i in range(stop, n)]
  return order


def forward(config, weights, tokens, layer_outputs=None):
  """float64 logits [T, vocab] of one sequence."""
  w = {k: np.asarray(v, dtype=np.float64) if np.asarray(v).dtype.kind == "f" else np.asarray(v)
       for k, v in weights.items()}
  x0 = w["embed"][np.asarray(tokens)] * float(config["embedding"]["scale"])
  x = x0.copy()
  for i, walk, first in run_order(config):
    if first:
      x = np.concatenate([x, x0], axis=1) @ w["loop.in"].T + w["loop.step"][walk]
    x = layer(x, w, i, config["layers"][i])
    if layer_outputs is not None:
      layer_outputs.append(x.copy())
  y = dyt(x, w["final.norm.alpha"], w["final.norm"], w["final.norm.b"])
  return (y @ w["embed"].T) * float(config["logit_scale"])
