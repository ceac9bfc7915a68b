"""Prefill and decode throughput of a design beside the engine's closest other model at equal size
(Generax beside Gemma 2, Sapivik beside Generax, Zesapel beside Sapivik, Nulezen beside Sapivik), and the time of every kernel
call of one step of each with its share of the measured peaks.

Used by `bench.py --design generax|sapivik|zesapel|nulezen` (the default benchmark does not import this file).  Layer
shapes resemble a real model's; weights are random.  Per size and design:

* prefill: one 2,048-token prompt in one step, median of 5 after 3 warm-up steps, CUDA events;
* decode: batch 8 whose requests end at 2,048 cached tokens, the engine's own decode runner
  (CUDA-graph replays), median of 5 bursts;
* kernels: one eager prefill step and one eager decode step with every call of the kernel table
  timed on its own (CUDA events around the call, L2 flushed before it by writing 256 MB),
  grouped by kernel, with the algorithmic bytes and FLOPs of the call.
"""

from __future__ import annotations

import time
from typing import Any

import numpy as np
import torch

SIZES = {
    # name: width, heads, kv heads, head size, feed-forward, vocabulary, layers
    "2b-like": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=8192, vocab=32768, layers=6),
    "8b-like": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=14336, vocab=32768, layers=3),
}
WINDOW, LEFT_WINDOW, POOL, RANK, TAPS = 1024, 512, 64, 64, 4


def generax_dict(s: dict) -> dict:
  att = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"],
         "scale": s["dim"] ** -0.5, "mask": {"size": WINDOW},
         "rot": {"dims": s["dim"], "base": 10000.0, "scaling": {"factor": 1.0}}}
  par = {"left": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"],
                  "scale": s["dim"] ** -0.5, "mask": {"size": LEFT_WINDOW, "pool": POOL}},
         "right": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "conv": TAPS,
                   "decay_rank": RANK, "gate_rank": RANK}}
  layers = []
  for i in range(s["layers"]):
    kind = i % 3
    if kind == 0:
      layers.append({"type": "parallel", "mixer": par})
    elif kind == 1:
      layers.append({"type": "attention", "mixer": dict(att)})
    else:
      layers.append({"type": "attention", "mixer": dict(att, kv_from=i - 1)})
    layers[-1]["mlp"] = {"kind": "dense", "ff": s["ff"]}
  return {"architecture": "Generax", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
          "logit_softcap": 30.0, "layers": layers, "max_context": 8192}


def sapivik_dict(s: dict) -> dict:
  """Attention layers with a dense feed-forward and recurrent layers with routed experts in turn (one
  in three is attention, as one in three Generax layers has keys of its own); the experts' hidden
  size is a quarter of the dense one, four of sixteen chosen, so a token's products are those of a
  dense layer; the first three layers run twice."""
  att = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"],
         "scale": s["dim"] ** -0.5, "softcap": 30.0, "rot": {"dims": s["dim"] // 2, "base": 10000.0}}
  rec = {"heads": s["heads"], "dim": s["dim"], "vdim": s["dim"]}
  dense = {"kind": "dense", "ff": s["ff"], "limit": 7.0}
  experts = {"kind": "moe", "expert": {"ff": s["ff"] // 4}, "shared": {"ff": s["ff"] // 4},
             "router": {"experts": 16, "identity": 2, "top": 4, "scale": 1.0}}
  layers = []
  for i in range(s["layers"]):
    if i % 3 == 0:
      layers.append({"type": "attention", "mixer": dict(att), "mlp": dict(dense)})
    else:
      layers.append({"type": "hgrn2", "mixer": dict(rec), "mlp": dict(experts)})
  times = 2
  stop = min(3, s["layers"])
  return {"architecture": "Sapivik", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
          "residual_mult": 0.5, "layers": layers[:s["layers"] - stop * (times - 1)] if s["layers"] > stop else layers,
          "loop": {"start": 0, "stop": stop, "times": times if s["layers"] > stop else 1}, "max_context": 8192}


def zesapel_dict(s: dict) -> dict:
  """Latent attention, the generalized delta rule and the state-space mixer in turn (one layer in
  three is attention, as in the Sapivik arm), each with table experts: sixteen of the hidden size of
  a quarter of the dense one, four per token.  The latent of keys and values has four heads' size,
  the rotated part half a head's; the recurrent states have heads of 64 channels; two streams and a
  convolution of three taps on what every mixer reads."""
  att = {"heads": s["heads"], "dim": s["dim"], "rot_dim": s["dim"] // 2, "vdim": s["dim"], "q_rank": s["width"] // 2,
         "kv_rank": 4 * s["dim"], "scale": (s["dim"] + s["dim"] // 2) ** -0.5, "mask": {"size": WINDOW},
         "rot": {"dims": s["dim"] // 2, "base": 10000.0}}
  delta = {"heads": s["width"] // 64, "dim": 64}
  ssm = {"heads": 2 * s["width"] // 64, "vdim": 64, "state": 128, "groups": 1, "norm_groups": 1, "conv": TAPS}
  experts = {"kind": "moe", "expert": {"ff": s["ff"] // 4}, "router": {"experts": 16, "top": 4}}
  kinds = (("latent_attention", att), ("general_delta", delta), ("mamba2", ssm))
  layers = [{"type": kinds[i % 3][0], "mixer": dict(kinds[i % 3][1]), "mlp": dict(experts)} for i in range(s["layers"])]
  return {"architecture": "Zesapel", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
          "embedding": {"scale": 1.0}, "max_positions": 8192, "streams": 2, "canon": {"taps": 3}, "decay_rank": RANK,
          "layers": layers}


def nulezen_dict(s: dict) -> dict:
  """Windowed attention everywhere: one layer in three rotates its heads, has biases and a gate per
  head and a dense feed-forward with the learned activation; the others take the distance bias off
  their scores, gate every element and have routed experts of the Sapivik arm's shape (sixteen of a
  quarter of the dense hidden size, four per token, a shared one).  The first three layers run
  twice, as in the Sapivik arm."""
  att = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"],
         "scale": s["dim"] ** -0.5, "mask": {"size": WINDOW}}
  experts = {"kind": "moe", "expert": {"ff": s["ff"] // 4, "limit": 7.0}, "shared": {"ff": s["ff"] // 4, "limit": 7.0},
             "router": {"experts": 16, "top": 4}}
  layers = []
  for i in range(s["layers"]):
    if i % 3 == 0:
      layers.append({"type": "attention_2", "mixer": dict(att, rot={"dims": s["dim"] // 2, "base": 10000.0}),
                     "mlp": {"kind": "dense", "ff": s["ff"]}})
    else:
      layers.append({"type": "attention", "mixer": dict(att), "mlp": dict(experts)})
  times = 2
  stop = min(3, s["layers"])
  d = {"architecture": "Nulezen", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
       "embedding": {"scale": 1.0}, "logit_scale": 1.0,
       "layers": layers[:s["layers"] - stop * (times - 1)] if s["layers"] > stop else layers, "max_context": 8192}
  d["loop"] = {"start": 0, "stop": stop, "times": times if s["layers"] > stop else 1}
  return d


def gemma2_dict(s: dict) -> dict:
  return {"architectures": ["Gemma2ForCausalLM"], "hidden_size": s["width"], "num_hidden_layers": s["layers"],
          "num_attention_heads": s["heads"], "num_key_value_heads": s["kv_heads"], "head_dim": s["dim"],
          "intermediate_size": s["ff"], "vocab_size": s["vocab"], "rms_norm_eps": 1e-6, "rope_theta": 10000.0,
          "sliding_window": WINDOW, "attn_logit_softcapping": 50.0, "final_logit_softcapping": 30.0,
          "query_pre_attn_scalar": s["dim"], "hidden_activation": "gelu_pytorch_tanh",
          "max_position_embeddings": 8192, "layer_types": ["sliding_attention"] * s["layers"]}


# ---- per-call timing ---------------------------------------------------------------------------

def _nbytes(x) -> int:
  if isinstance(x, torch.Tensor):
    return x.numel() * x.element_size()
  if isinstance(x, (tuple, list)):
    return sum(_nbytes(y) for y in x)
  return 0


class TimedOps:
  """Stands in front of the kernel table for one step: every call is timed alone, after a write of
  256 MB has pushed its inputs out of L2.  Bytes of a call: its tensor arguments (weights and
  activations) and results; calls that read a cache count what they can see of it instead."""

  def __init__(self, ops: Any, flush: torch.Tensor):
    self._ops, self._flush, self.rows = ops, flush, []

  def __getattr__(self, name):
    fn = getattr(self._ops, name)
    if not callable(fn) or name.startswith("_") or name in ("check_errors", "hold_stream", "attention_graph_plan",
                                                          "check_attention", "pack_sample_params", "cast"):
      return fn

    def timed(*args, **kw):
      self._flush.fill_(1.0)
      torch.cuda.synchronize()
      e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
      e0.record()
      out = fn(*args, **kw)
      e1.record()
      torch.cuda.synchronize()
      tensors = [a for a in args if isinstance(a, torch.Tensor)] + [v for v in kw.values() if isinstance(v, torch.Tensor)]
      big = max((t.numel() * t.element_size() for t in tensors), default=0)
      moved = sum(_nbytes(t) for t in tensors) + _nbytes(out)
      flops = 0.0
      ctx = next((a for a in list(args) + list(kw.values()) if hasattr(a, "num_tokens") and hasattr(a, "cu_q")), None)
      if name in ("linear", "gated_linear", "lm_head", "linear_xielu", "linear_wide"):
        x, w = args[0], args[1]
        flops = 2.0 * x.shape[0] * w.shape[0] * w.shape[1]
      if name == "mix_experts":
        t_, top_ = args[1].shape
        if args[3] is not None:
          flops = 2.0 * t_ * top_ * (args[3].shape[1] + args[4].shape[1]) * args[3].shape[2]
      if name in ("paged_attention", "project_rotate_store", "rope_and_cache_write", "qk_norm_rotate_store", "pool_blocks",
                  "delta_rule_inputs", "gated_delta_scan", "rotate_headnorm_store", "forget_gate_scan", "latent_prepare"):
        moved -= big if name != "delta_rule_inputs" else 0  # the cache (or state) storage is not read whole
      if name == "paged_attention" and ctx is not None:
        q = args[0]
        heads, kv_heads, dim = kw["num_heads"], kw["num_kv_heads"], kw["head_dim"]
        vdim = kw.get("value_dim") or dim
        window = kw.get("window") or (1 << 30)
        starts, lens = ctx.host["q_start"], np.diff(ctx.host["cu_q"])
        pairs = seen = 0
        for s0, n in zip(starts, lens):
          pos = np.arange(s0, s0 + n)
          keys = np.minimum(pos + 1, window)
          if kw.get("pooled") is not None:
            keys = keys + np.maximum(pos - window + 1, 0) // kw["pooled"][2]
          pairs += int(keys.sum())
          seen += int(min(s0 + n, window + n)) + (int((s0 + n) // kw["pooled"][2]) if kw.get("pooled") is not None else 0)
        flops = 2.0 * pairs * heads * (dim + vdim)
        moved += seen * kv_heads * (dim + (0 if kw.get("values_in_keys") else vdim)) * args[1].element_size()
      if name == "gated_delta_scan" and ctx is not None:
        state = args[5]
        per_slot = state[0].numel() * 4
        moved += 2 * per_slot * ctx.num_seqs  # the state is read and written once per sequence
        flops = 6.0 * args[0].shape[0] * kw["num_heads"] * kw["head_dim"] * kw["value_dim"]
      if name == "forget_gate_scan" and ctx is not None:
        moved += 2 * args[3][0].numel() * 4 * ctx.num_seqs
        flops = 5.0 * args[0].shape[0] * kw["num_heads"] * kw["head_dim"] * kw["value_dim"]
      if name in ("general_delta_scan", "state_space_scan") and ctx is not None:
        state = args[4] if name == "general_delta_scan" else args[6]
        moved += 2 * state[0].numel() * 4 * ctx.num_seqs - _nbytes(state)
        per_token = (8.0 * kw["num_heads"] * kw["head_dim"] ** 2 if name == "general_delta_scan" else
                     5.0 * kw["num_heads"] * kw["state_dim"] * kw["value_dim"])
        flops = per_token * out.shape[0]
      self.rows.append((name, out.shape[0] if isinstance(out, torch.Tensor) else 0, e0.elapsed_time(e1), moved, flops))
      return out

    return timed


def time_calls(engine, entries, peaks) -> list[dict]:
  """One eager step with every kernel-table call timed alone; rows grouped by call name."""
  flush = torch.empty(64 << 20, dtype=torch.float32, device=engine.device)
  proxy = TimedOps(engine.ops, flush)
  ctx = engine._prepare(entries)
  ctx.ops = proxy
  engine.model.forward(ctx, engine.caches)
  torch.cuda.synchronize()
  groups: dict[str, list] = {}
  for name, rows, ms, moved, flops in proxy.rows:
    g = groups.setdefault(name, [0, 0.0, 0.0, 0.0])
    g[0] += 1
    g[1] += ms
    g[2] += moved
    g[3] += flops
  out = []
  for name, (calls, ms, moved, flops) in sorted(groups.items(), key=lambda kv: -kv[1][1]):
    gbs, tfl = moved / (ms * 1e-3) / 1e9, flops / (ms * 1e-3) / 1e12
    out.append({"call": name, "calls": calls, "ms": round(ms, 4), "gb_s": round(gbs, 1),
                "hbm_frac": round(gbs / peaks["hbm_gbs"], 4), "tflops": round(tfl, 2),
                "bf16_frac": round(tfl / peaks["bf16_tflops"], 4)})
  return out


# ---- whole steps ---------------------------------------------------------------------------------

def _prefill_ms(engine, tokens: int, vocab: int) -> float:
  from simply_b200 import StepEntry
  rng = np.random.default_rng(5)
  prompt = rng.integers(0, vocab, tokens).astype(np.int32)
  times = []
  for i in range(3 + 5):
    slot = engine.open_request(f"prefill{i}")
    if i >= 3:
      torch.cuda.synchronize()
      time.sleep(0.25)  # each timed step starts from settled clocks
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    engine.step_raw([StepEntry(slot, prompt, (tokens - 1,))])
    e1.record()
    torch.cuda.synchronize()
    if i >= 3:
      times.append(e0.elapsed_time(e1))
    engine.close_request(slot)
  return float(np.median(times))


PAIRS = {"generax": ("generax", "gemma2"), "sapivik": ("sapivik", "generax"), "zesapel": ("zesapel", "sapivik"),
         "nulezen": ("nulezen", "sapivik")}
DICTS = {"generax": generax_dict, "gemma2": gemma2_dict, "sapivik": sapivik_dict, "zesapel": zesapel_dict,
         "nulezen": nulezen_dict}


def run(args, peaks: dict, time_decode, design: str = "generax") -> dict:
  """The design and its neighbour at every size; `time_decode` is bench.py's burst timer."""
  from simply_b200 import Engine, EngineConfig, StepEntry
  from simply_b200.config import config_from_dict

  batch, context, tokens = 8, 2048, 2048
  results = {}
  launches = 0
  for size_name, s in SIZES.items():
    results[size_name] = {"shape": s}
    for which, d in ((name, DICTS[name](s)) for name in PAIRS[design]):
      cfg = config_from_dict(d)
      ec = EngineConfig(activation_dtype="bfloat16", page_size=64, batch_size=batch, max_seq_len=context + 64,
                        max_cache_tokens=batch * (context + 64), max_num_issue_tokens=2048, intermediate_steps=1)
      engine = Engine.from_config(cfg, seed=0, engine_config=ec, matrix_std=0.02, scale_std=0.0)
      vocab = s["vocab"]
      r: dict[str, Any] = {"graphs": engine._decode_runner is not None}
      ms = _prefill_ms(engine, tokens, vocab)
      r["prefill_ms"] = round(ms, 3)
      r["prefill_tok_s"] = round(tokens / (ms * 1e-3), 1)
      if engine._decode_runner is not None:
        ms_step, per_step, _ = time_decode(engine, torch, batch, context, args.steps, args.warmup, seed=1)
        launches += int(per_step * args.steps)
      else:
        ms_step = float("nan")
      r["decode_ms_per_step"] = round(ms_step, 4)
      r["decode_tok_s"] = round(batch / (ms_step * 1e-3), 1)
      # every kernel-table call of one prompt step and one decode step, each timed alone
      rng = np.random.default_rng(7)
      slot = engine.open_request("calls")
      r["prefill_calls"] = time_calls(engine, [StepEntry(slot, rng.integers(0, vocab, tokens).tolist(), (tokens - 1,))], peaks)
      engine.close_request(slot)
      slots = [engine.open_request(f"calls{i}") for i in range(batch)]
      for sl in slots:
        engine.step_raw([StepEntry(sl, rng.integers(0, vocab, context - 1).tolist(), ())])
      r["decode_calls"] = time_calls(engine, [StepEntry(sl, [int(rng.integers(0, vocab))], (0,)) for sl in slots], peaks)
      for sl in slots:
        engine.close_request(sl)
      engine.ops.check_errors()
      results[size_name][which] = r
      del engine
      torch.cuda.empty_cache()
  return {"sizes": results, "launches": launches}
