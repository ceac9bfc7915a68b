"""Small Zesapel configurations with random (and crafted) weights for the tests.

Every comparison is between the engine (with a kernel table: the CUDA one on a GPU, the plain
PyTorch statements on the CPU) and the plain NumPy model of `tests/plain/zesapel_plain.py`, which
sees whole sequences and has no cache.  The ways of running an engine are those of
`tests/generax_cases.py`.
"""

from __future__ import annotations

import copy

import numpy as np
import torch

from simply_b200.config import config_from_dict
from simply_b200.parts.model import DecoderModel
from simply_b200.weights import random_tensors
from tests.generax_cases import as_numpy as _as_numpy, build_engine, cuts_of, run_cuts, run_mixed  # noqa: F401
from tests.tolerances import assert_logits_close
from tests.plain import zesapel_plain as plain


def latent(heads=3, dim=12, rot_dim=8, vdim=10, q_rank=20, kv_rank=14, dims=4, base=300.0, scale=0.3, window=11):
  m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
       "scale": scale}
  if dims:
    m["rot"] = {"dims": dims, "base": base}
  if window:
    m["mask"] = {"size": window}
  return {"type": "latent_attention", "mixer": m}


def delta(heads=2, dim=12):
  return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim}}


def mamba(heads=4, vdim=6, state=10, groups=2, norm_groups=3, conv=3):
  return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups,
                                      "norm_groups": norm_groups, "conv": conv}}


def moe(experts=5, top=2, ff=16):
  return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(layers, mlps, width=40, vocab=83, eps=1e-5, streams=3, taps=2, scale=3.0, max_positions=512, rank=5):
  out = []
  for layer, mlp in zip(layers, mlps):
    layer = copy.deepcopy(layer)
    layer["mlp"] = copy.deepcopy(mlp)
    out.append(layer)
  d = {"architecture": "Zesapel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
       "max_positions": max_positions, "layers": out, "decay_rank": rank}
  if streams:
    d["streams"] = streams
  if taps:
    d["canon"] = {"taps": taps}
  return d


# Models that differ in every size and switch.  A: three streams, two taps, every mixer, experts of
# which a token uses two and three.  B: four taps, two streams, heads rotated over all of their rotated
# part, no window in one attention layer, a layer without feed-forward, one group and one norm
# group, a token with a single expert.  C: one stream (plain residual sums), no convolution on the
# mixers' input, one tap in the state-space convolution.  D: sizes without whole 16-byte groups.
CONFIG_A = config(
    [latent(), delta(), mamba(), latent(heads=2, dim=16, rot_dim=4, vdim=16, q_rank=12, kv_rank=20, dims=2, window=5)],
    [moe(), moe(experts=4, top=3, ff=12), None, moe(experts=3, top=1, ff=24)])
CONFIG_B = config(
    [mamba(heads=2, vdim=16, state=8, groups=1, norm_groups=1, conv=4), latent(heads=4, dim=8, rot_dim=8, vdim=4, dims=8, window=None),
     delta(heads=3, dim=8), latent(heads=1, dim=20, rot_dim=6, vdim=24, q_rank=9, kv_rank=11, dims=6, base=50.0, window=17)],
    [moe(experts=2, top=2, ff=8), None, moe(experts=6, top=1, ff=20), moe(experts=7, top=4, ff=8)],
    width=48, vocab=131, eps=1e-6, streams=2, taps=4, scale=1.0, rank=3)
CONFIG_C = config([delta(heads=1, dim=16), mamba(heads=3, vdim=8, state=4, groups=3, norm_groups=2, conv=1), latent(window=3)],
                  [moe(experts=3, top=2, ff=10), moe(), None], width=32, vocab=60, streams=0, taps=0)
CONFIG_D = config([latent(heads=3, dim=5, rot_dim=6, vdim=7, q_rank=9, kv_rank=7, dims=2, window=9), delta(heads=3, dim=5),
                   mamba(heads=3, vdim=5, state=7, groups=1, norm_groups=5, conv=2)],
                  [moe(experts=3, top=2, ff=9), moe(experts=4, top=2, ff=7), moe(experts=2, top=1, ff=11)],
                  width=36, vocab=50, streams=1, taps=3, rank=2)


def as_numpy(t):
  return {k: (v.float().numpy().astype(np.float64) if v.is_floating_point() else v.numpy()) for k, v in t.items()}


def weights(cfg_dict, seed=0, matrix_std=0.1, scale_std=0.2):
  """bfloat16-representable random weights by tensor name (CPU; integer tables stay integers)."""
  cfg = config_from_dict(cfg_dict)
  specs = DecoderModel(cfg.model_spec()).tensor_specs()
  t = random_tensors(specs, seed, matrix_std=matrix_std, scale_std=scale_std, dtype=torch.bfloat16)
  gen = torch.Generator().manual_seed(seed + 1)

  def draw(name, std, mean=0.0):
    t[name] = (torch.randn(t[name].shape, generator=gen) * std + mean).to(torch.bfloat16)

  for name in list(t):
    if name == "embed":
      draw(name, 1.0)
    elif name == "pos":
      draw(name, 0.5)
    elif name.endswith(".sink") or name.endswith(".a.b") or name.endswith(".w0") or name.endswith(".dt_bias"):
      draw(name, 1.0)
    elif name.endswith(".A_log"):
      draw(name, 0.5, -1.0)  # slow decays, so that the state still holds tokens from far back
    elif name.endswith(".conv.b"):
      draw(name, 0.3)
    elif name.endswith((".in", ".out")) and ".hc" in name:
      draw(name, 0.3, 0.8)
    elif name.endswith(".mix") and ".hc" in name:
      s = t[name].shape[0]
      t[name] = (0.7 * torch.eye(s) + 0.3 * torch.randn(s, s, generator=gen)).to(torch.bfloat16)
    elif name.endswith((".w2", ".canon1")) or (name.endswith(".conv") and ".mix." in name):
      draw(name, 0.5)
  return cfg, t


def plant_needle(cfg_dict, t, layer, needle, asker, strength=9.0):
  """Makes the key of token `needle` and the query of token `asker` large in the last dim of the
  rotated part, which lies outside the rotated range (rot.dims < rot_dim) and which all heads share on
  the key's side: that one score stands out however many other keys there are.  Needs a model
  without a convolution on the mixer's input, and is approximate (positions add to the embedding)."""
  m = cfg_dict["layers"][layer]["mixer"]
  p = f"l{layer}.mix"
  width = cfg_dict["width"]
  eps = cfg_dict["norm"]["eps"]
  for tok, sign in ((needle, 1.0), (asker, -1.0)):
    row = torch.zeros(width)
    row[(7 * tok + 3) % width] = 6.0 * sign
    row[(5 * tok + 1) % width] = 6.0
    t["embed"][tok] = row.to(torch.bfloat16)
  w = as_numpy(t)
  read = w[f"l{layer}.hc1.in"].sum() if cfg_dict.get("streams") else 1.0
  y = {tok: plain.rms(w["embed"][tok][None] * cfg_dict["embedding"]["scale"] * read, eps)[0] * w[f"l{layer}.norm1"]
       for tok in (needle, asker)}
  dkv = t[f"{p}.dkv"].float()
  dkv[m["kv_rank"] + m["rot_dim"] - 1] += strength * torch.from_numpy(y[needle] / (y[needle] @ y[needle])).float()
  t[f"{p}.dkv"] = dkv.to(torch.bfloat16)
  cq = plain.rms(y[asker][None] @ w[f"{p}.dq"].T, eps)[0] * w[f"{p}.dq.norm"]
  uq = t[f"{p}.uq"].float()
  per = m["dim"] + m["rot_dim"]
  for h in range(m["heads"]):
    uq[h * per + per - 1] += strength * torch.from_numpy(cq / (cq @ cq)).float()
  t[f"{p}.uq"] = uq.to(torch.bfloat16)
  return t


def check_close(got, want, dtype, what):
  assert_logits_close(got, want, dtype, what)
