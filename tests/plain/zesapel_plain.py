"""The Zesapel decoder, stated plainly in NumPy float64: whole sequences, one function per
mechanism, no code shared with the engine.  The yardstick of tests/test_zesapel*.py.

`cfg` is config.json as a dictionary, `w` maps tensor names to float64 arrays (integer tables stay
integers).  Linear weights are [out, in].
"""

from __future__ import annotations

import math

import numpy as np


def rms(x, eps):
  return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(x):
  return 1.0 / (1.0 + np.exp(-x))


def silu(x):
  return x * sigmoid(x)


def softplus(x):
  return np.logaddexp(0.0, x)


def gelu_erf(x):
  return 0.5 * x * (1.0 + np.vectorize(math.erf)(x / math.sqrt(2.0)))


def causal_conv(x, taps_w, bias=None):
  """x [T, C], taps_w [C, K]: y_t = sum_j taps_w[:, j] * x_(t - K + 1 + j), zeros before the start."""
  t, c = x.shape
  k = taps_w.shape[1]
  padded = np.concatenate([np.zeros((k - 1, c)), x], axis=0)
  y = sum(padded[j:j + t] * taps_w[:, j][None, :] for j in range(k))
  return y if bias is None else y + bias[None, :]


# ---- the streams ----------------------------------------------------------------------------------
def streams_read(lanes, w_in):
  """lanes [S, T, W] -> sum_s w_in[s] lanes[s]."""
  return np.einsum("s,stw->tw", w_in, lanes)


def streams_write(lanes, y, mix, w_out):
  """new[t] = sum_s mix[s, t] old[s] + w_out[t] * y, all from the old lanes."""
  return np.einsum("sr,stw->rtw", mix, lanes) + w_out[:, None, None] * y[None, :, :]


# ---- mixers ---------------------------------------------------------------------------------------
def state_space_mixer(h, m, w, p, eps):
  """Mamba-2's recurrence, token by token."""
  heads, vdim, n, groups = m["heads"], m["vdim"], m["state"], m["groups"]
  inner = heads * vdim
  proj = h @ w[p + ".in"].T
  z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * groups * n], proj[:, 2 * inner + 2 * groups * n:]
  xbc = silu(causal_conv(xbc, w[p + ".conv"], w[p + ".conv.b"]))
  x = xbc[:, :inner].reshape(-1, heads, vdim)
  bmat = xbc[:, inner:inner + groups * n].reshape(-1, groups, n)
  cmat = xbc[:, inner + groups * n:].reshape(-1, groups, n)
  dt = softplus(dt + w[p + ".dt_bias"][None, :])
  rate = np.exp(w[p + ".A_log"])
  per_group = heads // groups
  state = np.zeros((heads, n, vdim))
  y = np.zeros((h.shape[0], heads, vdim))
  for t in range(h.shape[0]):
    for a in range(heads):
      g = a // per_group
      state[a] = math.exp(-rate[a] * dt[t, a]) * state[a] + dt[t, a] * np.outer(bmat[t, g], x[t, a])
      y[t, a] = state[a].T @ cmat[t, g] + w[p + ".D"][a] * x[t, a]
  y = y.reshape(-1, inner) * silu(z)
  parts = m["norm_groups"]
  y = rms(y.reshape(-1, parts, inner // parts), eps).reshape(-1, inner) * w[p + ".norm"][None, :]
  return y @ w[p + ".o"].T


def turn_halves(x, positions, dims, base):
  """x [T, ..., D]: dims i and i + dims/2 of the first `dims` turn by positions * base^(-2i/dims)."""
  half = dims // 2
  freq = base ** (-2.0 * np.arange(half) / dims)
  angle = positions[:, None] * freq[None, :]
  while angle.ndim < x.ndim:
    angle = angle[:, None]
  c, s = np.cos(angle), np.sin(angle)
  out = x.copy()
  a, b = x[..., :half], x[..., half:dims]
  out[..., :half] = a * c - b * s
  out[..., half:dims] = b * c + a * s
  return out


def latent_attention_mixer(h, m, w, p, eps):
  heads, dim, rdim, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
  t = h.shape[0]
  positions = np.arange(t, dtype=np.float64)
  cq = rms(h @ w[p + ".dq"].T, eps) * w[p + ".dq.norm"][None, :]
  q = (cq @ w[p + ".uq"].T).reshape(t, heads, dim + rdim)
  down = h @ w[p + ".dkv"].T
  c = rms(down[:, :rank], eps) * w[p + ".dkv.norm"][None, :]
  k_turned = down[:, rank:]
  rot = m.get("rot")
  if rot:
    q[..., dim:] = turn_halves(q[..., dim:], positions, rot["dims"], rot["base"])
    k_turned = turn_halves(k_turned, positions, rot["dims"], rot["base"])
  k_plain = (c @ w[p + ".uk"].T).reshape(t, heads, dim)
  v = (c @ w[p + ".uv"].T).reshape(t, heads, vdim)
  span = (m.get("mask") or {}).get("size")
  gate = sigmoid(h @ w[p + ".g"].T)
  out = np.zeros((t, heads, vdim))
  for i in range(t):
    lo = 0 if span is None else max(i - span + 1, 0)
    for a in range(heads):
      s = (k_plain[lo:i + 1, a] @ q[i, a, :dim] + k_turned[lo:i + 1] @ q[i, a, dim:]) * m["scale"]
      sink = w[p + ".sink"][a]
      top = max(s.max(), sink)
      e = np.exp(s - top)
      out[i, a] = (e @ v[lo:i + 1, a]) / (e.sum() + math.exp(sink - top)) * gate[i, a]
  return out.reshape(t, heads * vdim) @ w[p + ".o"].T


def delta_mixer(h, m, w, p, eps):
  """The generalized delta rule, token by token."""
  heads, dim = m["heads"], m["dim"]
  t = h.shape[0]
  r = (h @ w[p + ".r"].T).reshape(t, heads, dim)
  k = (h @ w[p + ".k"].T).reshape(t, heads, dim)
  v = (h @ w[p + ".v"].T).reshape(t, heads, dim)
  low = np.tanh(h @ w[p + ".w1"].T) @ w[p + ".w2"].T + w[p + ".w0"][None, :]
  decay = np.exp(-math.exp(-0.5) * sigmoid(low)).reshape(t, heads, dim)
  take = sigmoid(h @ w[p + ".a"].T + w[p + ".a.b"][None, :]).reshape(t, heads, dim)
  unit = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
  state = np.zeros((heads, dim, dim))
  o = np.zeros((t, heads, dim))
  for i in range(t):
    for a in range(heads):
      old = state[a]
      state[a] = (decay[i, a][:, None] * old - np.outer(take[i, a] * unit[i, a], unit[i, a] @ old)
                  + np.outer(k[i, a], v[i, a]))
      o[i, a] = state[a].T @ r[i, a]
  o = rms(o, eps).reshape(t, heads * dim) * w[p + ".norm"][None, :] * sigmoid(h @ w[p + ".g"].T)
  return o @ w[p + ".o"].T


MIXERS = {"mamba2": state_space_mixer, "latent_attention": latent_attention_mixer, "general_delta": delta_mixer}


# ---- feed-forward -----------------------------------------------------------------------------------
def table_experts(h, tokens, mlp, w, p):
  top = mlp["router"]["top"]
  out = np.zeros_like(h)
  for t, tok in enumerate(tokens):
    for j in range(top):
      e = int(w[p + ".table"][tok, j])
      hidden = gelu_erf(w[f"{p}.e{e}.up"] @ h[t])
      out[t] += (w[f"{p}.e{e}.down"] @ hidden) / top
  return out


# ---- the model --------------------------------------------------------------------------------------
def forward(cfg, w, tokens, layer_outputs=None):
  """Logits [T, vocab] of one sequence from its first token on."""
  tokens = np.asarray(tokens)
  t = len(tokens)
  eps = cfg["norm"]["eps"]
  x = w["embed"][tokens] * (cfg.get("embedding") or {}).get("scale", 1.0)
  if "pos" in w:
    x = x + w["pos"][np.arange(t)]
  streams = cfg.get("streams")
  lanes = np.stack([x] * streams) if streams else None
  taps = (cfg.get("canon") or {}).get("taps")
  for i, layer in enumerate(cfg["layers"]):
    p = f"l{i}"
    for q, sub in ((1, "mix"), (2, "mlp")):
      if sub == "mlp" and layer.get("mlp") is None:
        continue
      u = streams_read(lanes, w[f"{p}.hc{q}.in"]) if streams else x
      h = rms(u, eps) * w[f"{p}.norm{q}"][None, :]
      if sub == "mix":
        if taps:
          h = h + causal_conv(h, w[f"{p}.canon1"])
        y = MIXERS[layer["type"]](h, layer["mixer"], w, f"{p}.mix", eps)
      else:
        y = table_experts(h, tokens, layer["mlp"], w, f"{p}.mlp")
      if streams:
        lanes = streams_write(lanes, y, w[f"{p}.hc{q}.mix"], w[f"{p}.hc{q}.out"])
      else:
        x = x + y
    if layer_outputs is not None:
      layer_outputs.append(lanes.sum(0) if streams else x.copy())
  x = lanes.sum(0) if streams else x
  return (rms(x, eps) * w["final.norm"][None, :]) @ w["head"].T
