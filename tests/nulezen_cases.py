"""Small Nulezen configurations with random (and crafted) weights for the tests.

Every comparison is between the engine (with a kernel table: the CUDA one on a GPU, the plain
PyTorch statements on the CPU) and the plain NumPy model of `tests/plain/nulezen_plain.py`, which
sees whole sequences and has no cache.  The ways of running an engine (one request cut into
portions, several side by side) are those of `tests/generax_cases.py`.
"""

from __future__ import annotations

import copy

import numpy as np
import torch

from simply_b200.config import config_from_dict
from simply_b200.parts.model import DecoderModel
from simply_b200.weights import random_tensors
from tests.generax_cases import as_numpy, build_engine, cuts_of, run_cuts, run_mixed  # noqa: F401
from tests.sapivik_cases import check_close  # noqa: F401  (a router's choice may hang on a rounding in bfloat16)
from tests.plain import nulezen_plain as plain


def biased(heads=4, kv_heads=2, dim=16, vdim=16, window=12, scale=0.3):
  """Attention whose scores lose r1 log(1 + r2 distance); a gate per element."""
  return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                         "scale": scale, "mask": {"size": window}}}


def rotated(heads=4, kv_heads=2, dim=16, vdim=16, window=12, scale=0.3, dims=8, base=300.0):
  """Attention with biases on q, k, v, partly rotated heads and a gate per head."""
  m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window}}
  if dims is not None:
    m["rot"] = {"dims": dims, "base": base}
  return {"type": "attention_2", "mixer": m}


def dense(ff=64):
  return {"kind": "dense", "ff": ff}


def moe(experts=6, top=3, ff=24, limit=1.2, shared=40, shared_limit=2.0):
  m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
  if shared:
    m["shared"] = {"ff": shared, "limit": shared_limit}
  return m


def config(layers, mlps, width=48, vocab=97, embed_scale=3.0, logit_scale=0.7, loop=None):
  out = []
  for layer, mlp in zip(layers, mlps):
    layer = copy.deepcopy(layer)
    layer["mlp"] = copy.deepcopy(mlp)
    out.append(layer)
  d = {"architecture": "Nulezen", "vocab": vocab, "width": width, "embedding": {"scale": embed_scale},
       "logit_scale": logit_scale, "norm": {"eps": 1e-6}, "layers": out, "max_context": 512}
  if loop is not None:
    d["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
  return d


# A: a loop over the first three layers, both mixers, both feed-forwards, windows that differ from
# layer to layer, value heads smaller than key heads.
CONFIG_A = config(
    [biased(), rotated(window=9), biased(heads=2, kv_heads=1, dim=32, vdim=8, window=17), rotated(heads=2, kv_heads=2, dim=32, vdim=32, dims=32, window=5)],
    [dense(), moe(), moe(experts=4, top=1, ff=16, shared=0), dense(ff=40)],
    loop=(0, 3, 2))
# B: a loop of one layer run three times in the middle, as many kv heads as heads, value heads larger
# than key heads, heads that are not rotated at all, a router that takes every expert, a layer
# without a feed-forward, a window of one (a token sees itself alone), factors of 1.
CONFIG_B = config(
    [rotated(heads=3, kv_heads=3, dim=8, vdim=24, dims=None, window=7), biased(heads=6, kv_heads=2, dim=12, vdim=20, window=30, scale=0.5),
     biased(heads=1, kv_heads=1, dim=40, vdim=40, window=1), rotated(heads=6, kv_heads=3, dim=12, vdim=12, dims=4, window=64)],
    [moe(experts=3, top=3, ff=8, shared=56), None, dense(ff=72), moe(experts=5, top=2, ff=20, shared=0)],
    width=40, vocab=131, embed_scale=1.0, logit_scale=1.0, loop=(1, 2, 3))
# C: no loop entry at all; sizes without whole 16-byte groups anywhere.
CONFIG_C = config([biased(heads=2, kv_heads=1, dim=6, vdim=10, window=11), rotated(heads=3, kv_heads=1, dim=10, vdim=6, dims=6, window=4)],
                  [moe(experts=3, top=2, ff=10, shared=6), dense(ff=14)], width=36, vocab=50)
# D: the loop covers every layer.
CONFIG_D = config([rotated(heads=2, kv_heads=1, dim=16, vdim=16, dims=16, window=20), biased(heads=2, kv_heads=2, dim=16, vdim=16, window=6)],
                  [dense(ff=32), moe(experts=4, top=2, ff=12)], width=32, vocab=60, loop=(0, 2, 3))


def weights(cfg_dict, seed=0, matrix_std=0.18, scale_std=0.2):
  """bfloat16-representable random weights by tensor name (CPU, bfloat16)."""
  cfg = config_from_dict(cfg_dict)
  specs = DecoderModel(cfg.model_spec()).tensor_specs()
  t = random_tensors(specs, seed, matrix_std=matrix_std, scale_std=scale_std, dtype=torch.bfloat16)
  gen = torch.Generator().manual_seed(seed + 1)
  width = cfg_dict["width"]
  for name in t:
    shape = t[name].shape
    if name == "embed":
      t[name] = torch.randn(shape, generator=gen).to(torch.bfloat16)
    elif name.endswith(".router"):
      t[name] = (torch.randn(shape, generator=gen) * 0.6).to(torch.bfloat16)
    elif name.endswith(".router.b") or name.endswith(".act") or name == "loop.step":
      t[name] = (torch.randn(shape, generator=gen) * 0.5).to(torch.bfloat16)
    elif name.endswith(".alpha"):
      t[name] = (0.4 + 0.4 * torch.rand(shape, generator=gen)).to(torch.bfloat16)
    elif name.endswith(".r1") or name.endswith(".r2"):
      t[name] = (0.2 + torch.rand(shape, generator=gen)).to(torch.bfloat16)
    elif name.endswith(".q.b") or name.endswith(".k.b") or name.endswith(".v.b"):
      t[name] = (torch.randn(shape, generator=gen) * 0.3).to(torch.bfloat16)
    elif name == "loop.in":  # near [I, I] / 2 so that the stream keeps its size from pass to pass
      eye = torch.cat([torch.eye(width), torch.eye(width)], dim=1) * 0.5
      t[name] = (eye + 0.1 * torch.randn(shape, generator=gen)).to(torch.bfloat16)
  return cfg, t


def plant_needle(cfg_dict, t, layer, needle, asker, strength=7.0):
  """In a model whose layer `layer` reads the embedding's output (no loop, layer 0): makes the key
  of token `needle` and the query of token `asker` point the same way in the last dim of every
  head (outside a rotated range smaller than the head), far longer than their other dims, so
  that the score strength^2 * scale stands out however many other keys there are, and gives the
  needle a value of its own."""
  m = cfg_dict["layers"][layer]["mixer"]
  p = f"l{layer}.mix"
  width, d = cfg_dict["width"], m["dim"]
  gen = torch.Generator().manual_seed(4321 + layer)
  for tok, sign in ((needle, 1.0), (asker, -1.0)):
    row = torch.zeros(width)
    row[(7 * tok + 3) % width] = 1.5 * sign
    row[(5 * tok + 1) % width] = 1.5
    t["embed"][tok] = row.to(torch.bfloat16)
  n1 = f"l{layer}.norm1"
  # (the norm's offset is common to every token's y and would give every key a share of the needle's)
  t[f"{n1}.b"] = torch.zeros_like(t[f"{n1}.b"])
  ys = {}
  for tok in (needle, asker):
    x = t["embed"][tok].float().numpy()[None] * cfg_dict["embedding"]["scale"]
    ys[tok] = torch.from_numpy(plain.dyt(x, t[f"{n1}.alpha"].float().item(), t[n1].float().numpy(),
                                         t[f"{n1}.b"].float().numpy())[0]).float()
  for name, tok, heads in ((f"{p}.k", needle, m["kv_heads"]), (f"{p}.q", asker, m["heads"])):
    w = t[name].float()
    y = ys[tok]
    for h in range(heads):
      w[h * d + d - 1] += strength * y / (y @ y)
    t[name] = w.to(torch.bfloat16)
  v = t[f"{p}.v"].float()
  v += 2.0 * torch.randn(v.shape[0], generator=gen)[:, None] * ys[needle][None, :] / float(ys[needle] @ ys[needle])
  t[f"{p}.v"] = v.to(torch.bfloat16)
  return t
