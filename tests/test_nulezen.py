"""The Nulezen decoder through the engine against the plain NumPy model.

Each scenario runs on the CPU with the plain PyTorch kernel statements (this checks the parts,
the configuration, the cache manager and the step function) and, marked `gpu`, with the CUDA
kernels in float32 and bfloat16."""

import copy
import json
import os

import numpy as np
import pytest
import torch

from simply_b200 import Engine, EngineConfig, SamplingParams, StepEntry
from simply_b200.config import ConfigError, config_from_dict, load_config
from simply_b200.weights import write_model_folder
from tests import nulezen_cases as nx
from tests.plain import nulezen_plain as plain
from tests.reference_ops import ReferenceOps

CPU = pytest.param(("float32", "cpu"), id="cpu")
GPU32 = pytest.param(("float32", "cuda"), id="gpu-f32", marks=pytest.mark.gpu)
GPU16 = pytest.param(("bfloat16", "cuda"), id="gpu-bf16", marks=pytest.mark.gpu)
WHERE = [CPU, GPU32, GPU16]
CONFIGS = {"a": nx.CONFIG_A, "b": nx.CONFIG_B, "c": nx.CONFIG_C, "d": nx.CONFIG_D}


def engine_for(cfg_dict, where, seed=0, tensors=None, **kw):
  dtype, device = where
  cfg, t = nx.weights(cfg_dict, seed)
  if tensors is not None:
    t = tensors
  ops = ReferenceOps(torch.float32) if device == "cpu" else None
  return nx.build_engine(cfg, t, dtype, device, ops, **kw), t


def tokens_for(cfg_dict, n, seed):
  return np.random.default_rng(seed).integers(0, cfg_dict["vocab"], n).tolist()


# ---- whole prompts, portions, decoding, batches -------------------------------------------------

@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("which", ["a", "b", "c", "d"])
def test_whole_portions_and_decoding(which, where):
  cfg_dict = CONFIGS[which]
  engine, t = engine_for(cfg_dict, where, seed=3)
  toks = tokens_for(cfg_dict, 61, 1)
  want = plain.forward(cfg_dict, nx.as_numpy(t), toks)
  n = len(toks)
  for what, cuts in [
      ("whole", [n]),
      ("token by token", [1] * n),
      ("prompt then decoding", [n - 40] + [1] * 40),
      ("portions down to two tokens", nx.cuts_of(n, [7, 2, 5, 3, 11, 2, 13, 4, 2, 9])),
      ("portions that end at the pages' borders", nx.cuts_of(n, [8, 8, 1, 7, 16, 2])),
      ("portions of two", [2] * (n // 2) + [1]),
      ("one token, then the rest", [1, n - 1]),
  ]:
    nx.check_close(nx.run_cuts(engine, toks, cuts), want, where[0], f"{which}: {what}")
  engine.cache.check_invariants()
  assert engine.cache.all_pages_free()
  engine.ops.check_errors()


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("which", ["a", "b"])
def test_unequal_requests_side_by_side_with_pages_and_slots_used_again(which, where):
  cfg_dict = CONFIGS[which]
  # room for three live requests of these lengths, not for all six: pages and slots come back
  engine, t = engine_for(cfg_dict, where, seed=5, slots=3, max_cache_tokens=3 * 80, poison=True)
  lengths = [70, 9, 33, 1, 58, 21]
  requests = [tokens_for(cfg_dict, n, 10 + i) for i, n in enumerate(lengths)]
  w = nx.as_numpy(t)
  want = [plain.forward(cfg_dict, w, r) for r in requests]
  got = nx.run_mixed(engine, requests, seed=2)
  for i, (g, x) in enumerate(zip(got, want)):
    nx.check_close(g, x, where[0], f"request {i} in a mixed batch")
  # the same requests once more through the used slots and pages, each alone
  for i in (0, 4):
    nx.check_close(nx.run_cuts(engine, requests[i], [len(requests[i])]), want[i], where[0], f"request {i} again")
  engine.cache.check_invariants()
  assert engine.cache.all_pages_free()
  engine.ops.check_errors()


@pytest.mark.parametrize("where", WHERE)
def test_long_decoding_past_many_pages_and_windows(where):
  """150 tokens over pages of 4: every window (5 to 17 keys) passes over decoded tokens many times
  and the pages behind it are given back on the way."""
  cfg_dict = nx.CONFIG_A
  engine, t = engine_for(cfg_dict, where, seed=7, page_size=4)
  toks = tokens_for(cfg_dict, 150, 4)
  want = plain.forward(cfg_dict, nx.as_numpy(t), toks)
  nx.check_close(nx.run_cuts(engine, toks, [3] + [1] * 147), want, where[0], "long decoding")
  engine.cache.check_invariants()
  engine.ops.check_errors()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompts_pages_of_64_and_head_sizes_of_the_tensor_core_kernels(dtype):
  """500 tokens over pages of 64: head sizes 64, 96 and 128 with several heads per kv head (the
  tensor-core attention kernels in bfloat16 where they take the layer), windows that end inside
  a page and that span several, more routed rows per expert than one tile holds."""
  cfg_dict = nx.config(
      [nx.biased(heads=8, kv_heads=2, dim=64, vdim=64, window=150, scale=0.1),
       nx.rotated(heads=12, kv_heads=2, dim=96, vdim=96, dims=96, base=5000.0, window=80, scale=0.09),
       nx.rotated(heads=4, kv_heads=2, dim=128, vdim=128, dims=64, window=300, scale=0.07),
       nx.biased(heads=4, kv_heads=4, dim=32, vdim=48, window=65, scale=0.15)],
      [nx.moe(experts=3, top=2, ff=96, shared=128), nx.dense(ff=256), nx.moe(experts=8, top=4, ff=32, shared=0), None],
      width=128, vocab=300, loop=(1, 3, 2))
  cfg, t = nx.weights(cfg_dict, seed=3, matrix_std=0.1)
  engine = nx.build_engine(cfg, t, dtype, "cuda", None, page_size=64, slots=2, max_seq_len=512)
  toks = tokens_for(cfg_dict, 500, 1)
  want = plain.forward(cfg_dict, nx.as_numpy(t), toks)
  for what, cuts in [("whole", [500]), ("portions", nx.cuts_of(500, [100, 2, 37, 64, 3, 129, 200])),
                     ("decoding", [440] + [1] * 60)]:
    nx.check_close(nx.run_cuts(engine, toks, cuts), want, dtype, what)
  engine.ops.check_errors()


@pytest.mark.parametrize("where", WHERE)
def test_many_query_heads_per_kv_head(where):
  """32 and 12 query heads per kv head: a single token's rows no longer fit the split-key kernel's
  16, so decoded tokens take the tile kernels too."""
  cfg_dict = nx.config(
      [nx.biased(heads=32, kv_heads=1, dim=64, vdim=64, window=50, scale=0.12),
       nx.rotated(heads=24, kv_heads=2, dim=32, vdim=32, dims=16, window=31, scale=0.2),
       nx.biased(heads=20, kv_heads=1, dim=16, vdim=16, window=40, scale=0.25)],
      [nx.dense(ff=64), None, nx.moe(experts=4, top=2, ff=32, shared=0)], width=64, vocab=90, loop=(0, 2, 2))
  engine, t = engine_for(cfg_dict, where, seed=8, page_size=16, max_seq_len=128)
  toks = tokens_for(cfg_dict, 90, 2)
  want = plain.forward(cfg_dict, nx.as_numpy(t), toks)
  for what, cuts in [("whole", [90]), ("decoding", [60] + [1] * 30), ("portions", nx.cuts_of(90, [17, 2, 40, 3]))]:
    nx.check_close(nx.run_cuts(engine, toks, cuts), want, where[0], what)
  engine.ops.check_errors()


# ---- a key that stands out: far back, at a page's border, either side of the window's edge -----------

@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("kind", ["biased", "rotated"])
def test_a_key_that_stands_out_inside_and_outside_the_window(kind, where):
  """One attention layer whose query of token 1 is answered by the key of token 2 alone while the
  window holds it: the needle among hundreds of keys, at the first tokens, either side of a page's
  border, as the oldest key the window keeps and as the newest one it has lost, in prompts'
  portions and asked for by a token decoded alone."""
  window = 200
  layer = (nx.biased(heads=4, kv_heads=2, dim=16, vdim=16, window=window, scale=0.5) if kind == "biased"
           else nx.rotated(heads=4, kv_heads=2, dim=16, vdim=16, dims=8, window=window, scale=0.5))
  cfg_dict = nx.config([layer], [nx.dense(ff=32)], width=32, vocab=50, embed_scale=2.0)
  cfg, t = nx.weights(cfg_dict, seed=11)
  nx.plant_needle(cfg_dict, t, 0, needle=2, asker=1)
  w = nx.as_numpy(t)
  engine, _ = engine_for(cfg_dict, where, tensors=t, page_size=8, max_seq_len=512)
  rng = np.random.default_rng(0)
  decides = {}
  cases = [(40, 0, 1), (40, 0, 39), (75, 7, 8), (75, 8, 71), (75, 3, 16), (330, 131, 329), (330, 15, 200),
           (330, 100, 100 + window - 1), (330, 100, 100 + window), (260, 0, window - 1), (260, 0, window),
           (330, 63, 63 + window - 1), (330, 64, 64 + window)]
  for n, needle_at, ask_at in cases:
    toks = rng.integers(3, cfg_dict["vocab"], n).tolist()
    toks[needle_at], toks[ask_at] = 2, 1
    want = plain.forward(cfg_dict, w, toks)
    without = list(toks)
    without[needle_at] = 5
    decides[(needle_at, ask_at)] = np.abs(plain.forward(cfg_dict, w, without)[ask_at] - want[ask_at]).max() > 0.3
    for cuts in ([n], [ask_at, 1, n], [max(ask_at - 1, 1), 2, n], nx.cuts_of(n, [5, 2, 3, 64]),
                 [needle_at + 1, ask_at - needle_at - 1] + [1] * 8 + [n]):
      got = nx.run_cuts(engine, toks, [c for c in cuts if c > 0])
      nx.check_close(got, want, where[0], f"needle at {needle_at}, asked at {ask_at}, cuts {cuts[:3]}")
  # the needle decides the asker's logits exactly while the window holds it
  for (needle_at, ask_at), seen in decides.items():
    assert seen == (ask_at - needle_at < window), (needle_at, ask_at, seen)
  engine.ops.check_errors()


@pytest.mark.parametrize("where", WHERE)
def test_the_distance_bias_decides_between_equal_keys(where):
  """Two equal needles at different distances: without the bias the asker would weigh them alike;
  with it the nearer one wins by r1 log((1 + r2 d_far) / (1 + r2 d_near)).  Their values differ
  through the positions' neighbours only, so the test checks the engine against the plain model
  with a bias large enough to matter."""
  cfg_dict = nx.config([nx.biased(heads=2, kv_heads=1, dim=16, vdim=16, window=120, scale=0.5)], [None], width=32, vocab=50)
  cfg, t = nx.weights(cfg_dict, seed=4)
  nx.plant_needle(cfg_dict, t, 0, needle=2, asker=1, strength=3.0)
  t["l0.mix.r1"] = torch.tensor([2.5, 0.0]).to(torch.bfloat16)  # (the second head has no bias at all)
  t["l0.mix.r2"] = torch.tensor([3.0, 1.0]).to(torch.bfloat16)
  w = nx.as_numpy(t)
  engine, _ = engine_for(cfg_dict, where, tensors=t, page_size=8, max_seq_len=256)
  toks = np.random.default_rng(2).integers(3, 50, 130).tolist()
  toks[20], toks[100], toks[125] = 2, 2, 1
  want = plain.forward(cfg_dict, w, toks)
  flat = dict(w)
  flat["l0.mix.r1"] = np.zeros(2)
  assert np.abs(plain.forward(cfg_dict, flat, toks)[125] - want[125]).max() > 1e-2 * np.abs(want).max()
  for cuts in ([130], [125, 1, 4], nx.cuts_of(130, [9, 2, 31])):
    nx.check_close(nx.run_cuts(engine, toks, cuts), want, where[0], f"cuts {cuts[:3]}")


# ---- generation through the entry point and the scheduler -----------------------------------------

@pytest.mark.parametrize("where", [CPU, GPU32])
def test_greedy_generation_through_the_scheduler(where):
  cfg_dict = nx.CONFIG_B
  engine, t = engine_for(cfg_dict, where, seed=9, slots=2)
  w = nx.as_numpy(t)
  prompts = [tokens_for(cfg_dict, n, 30 + i) for i, n in enumerate((5, 17, 1, 26))]
  results = engine.generate(prompts, SamplingParams(temperature=0.0, max_decode_steps=12))
  for prompt, r in zip(prompts, results):
    toks = list(prompt)
    for _ in range(12):
      toks.append(int(np.argmax(plain.forward(cfg_dict, w, toks)[-1])))
    assert r.output_token_ids == toks[len(prompt):], (r.output_token_ids, toks[len(prompt):])
  assert engine.cache.all_pages_free()


@pytest.mark.gpu
@pytest.mark.parametrize("which,burst", [("a", 1), ("b", 5)])
def test_decoding_from_cuda_graphs(which, burst):
  """Three live requests decode from the graph of four rows (the fourth repeats the third),
  several steps per replay burst."""
  cfg_dict = CONFIGS[which]
  engine, t = engine_for(cfg_dict, ("float32", "cuda"), seed=13, slots=4, graphs=True, burst=burst)
  assert engine._decode_runner is not None, "the model's parts must all allow graph capture"
  w = nx.as_numpy(t)
  prompts = [tokens_for(cfg_dict, n, 40 + i) for i, n in enumerate((9, 3, 14))]
  results = engine.generate(prompts, SamplingParams(temperature=0.0, max_decode_steps=17))
  assert engine._decode_runner.bursts > 0
  for prompt, r in zip(prompts, results):
    toks = list(prompt)
    for _ in range(17):
      toks.append(int(np.argmax(plain.forward(cfg_dict, w, toks)[-1])))
    assert r.output_token_ids == toks[len(prompt):], (r.output_token_ids, toks[len(prompt):])
  engine.ops.check_errors()


@pytest.mark.gpu
def test_bfloat16_generation_runs_and_samples():
  engine, _ = engine_for(nx.CONFIG_A, ("bfloat16", "cuda"), seed=2, slots=3)
  prompts = [tokens_for(nx.CONFIG_A, n, i) for i, n in enumerate((4, 30, 11, 2, 19))]
  results = engine.generate(prompts, SamplingParams(temperature=0.8, top_k=20, max_decode_steps=20, seed=4))
  assert all(len(r.output_token_ids) == 20 for r in results)
  again = engine.generate(prompts, SamplingParams(temperature=0.8, top_k=20, max_decode_steps=20, seed=4))
  assert [r.output_token_ids for r in results][0] == [r.output_token_ids for r in again][0]
  engine.ops.check_errors()


@pytest.mark.gpu
def test_bfloat16_single_tokens_replayed_from_cuda_graphs():
  cfg_dict = nx.config(
      [nx.biased(heads=4, kv_heads=2, dim=64, vdim=64, window=50, scale=0.12),
       nx.rotated(heads=4, kv_heads=1, dim=32, vdim=32, dims=16, window=33, scale=0.2)],
      [nx.moe(experts=4, top=2, ff=32, shared=32), nx.dense(ff=64)], width=64, vocab=120, loop=(0, 1, 2))
  engine, t = engine_for(cfg_dict, ("bfloat16", "cuda"), seed=6, slots=4, graphs=True, page_size=16)
  assert engine._decode_runner is not None
  engine._decode_runner.keep_logits = True
  w = nx.as_numpy(t)
  requests = [tokens_for(cfg_dict, n, 50 + i) for i, n in enumerate((70, 41, 55))]
  want = [plain.forward(cfg_dict, w, r) for r in requests]
  slots = [engine.open_request() for _ in requests]
  heads = [len(r) - 30 for r in requests]
  engine.step_raw([StepEntry(s, r[:h], ()) for s, r, h in zip(slots, requests, heads)])
  got = [[] for _ in requests]
  for step in range(30):
    entries = [StepEntry(s, [r[h + step]], (0,)) for s, r, h in zip(slots, requests, heads)]
    logits = engine.step_raw(entries, from_graph=True).float().cpu().numpy()
    for i in range(len(requests)):
      got[i].append(logits[i])
  for i, h in enumerate(heads):
    nx.check_close(np.stack(got[i]), want[i][h:], "bfloat16", f"request {i}, replayed steps")
  engine.ops.check_errors()


# ---- configuration, model folders, the preset ---------------------------------------------------------

def test_config_round_trip_run_order_and_errors():
  cfg = config_from_dict(nx.CONFIG_A)
  assert config_from_dict(cfg.to_dict()) == cfg
  spec = cfg.model_spec()
  order = [(c.layer, c.stream_input) for c in spec.run_order]
  assert order == [("l0", ("loop", 0)), ("l1", None), ("l2", None), ("l0", ("loop", 1)), ("l1", None), ("l2", None),
                   ("l3", None)]
  assert len(set(spec.cache_names())) == 7  # every pass has a cache of its own
  spec_b = config_from_dict(nx.CONFIG_B).model_spec()
  assert [(c.layer, c.stream_input) for c in spec_b.run_order] == [
      ("l0", None), ("l1", ("loop", 0)), ("l1", ("loop", 1)), ("l1", ("loop", 2)), ("l2", None), ("l3", None)]
  spec_c = config_from_dict(nx.CONFIG_C).model_spec()
  assert [c.layer for c in spec_c.run_order] == ["l0", "l1"] and not spec_c.stream_inputs
  assert plain.run_order(nx.CONFIG_B) == [(0, None, False), (1, 0, True), (1, 1, True), (1, 2, True), (2, None, False),
                                          (3, None, False)]
  for change, text in [
      (lambda d: d["layers"][0].update(type="conv"), "unknown type"),
      (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
      (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=5), "rot.dims"),
      (lambda d: d["layers"][1]["mlp"]["router"].update(top=9), "router must choose"),
      (lambda d: d["layers"][1]["mlp"]["expert"].pop("limit"), "limit"),
      (lambda d: d["layers"][0]["mixer"].pop("mask"), "mask"),
      (lambda d: d.update(loop={"start": 2, "stop": 1, "times": 2}), "loop"),
      (lambda d: d["layers"][0]["mlp"].update(kind="sparse"), "unknown mlp kind"),
  ]:
    d = copy.deepcopy(nx.CONFIG_A)
    change(d)
    with pytest.raises(ConfigError, match=text):
      config_from_dict(d)


def test_model_folder_and_the_step_function_on_it(tmp_path):
  cfg = config_from_dict(nx.CONFIG_B)
  folder = write_model_folder(cfg, 4, str(tmp_path / "m"), matrix_std=0.2, scale_std=0.1)
  assert load_config(folder) == cfg
  with open(os.path.join(folder, "config.json")) as f:
    assert json.load(f)["architecture"] == "Nulezen"
  ec = EngineConfig(activation_dtype="float32", page_size=8, batch_size=2, max_seq_len=64, use_cuda_graphs=False)
  engine = Engine.from_folder(folder, ec, ops=ReferenceOps(torch.float32), device="cpu")
  from simply_b200.weights import safetensors_io as st
  entries = st.index_files(st.model_files(folder))
  reader = st.TensorReader(entries)
  w = {n: reader.read(n).float().numpy() for n in entries}
  toks = tokens_for(nx.CONFIG_B, 19, 3)
  slot = engine.open_request()
  got = engine.step_raw([StepEntry(slot, toks, tuple(range(len(toks))))]).numpy()
  engine.close_request(slot)
  nx.check_close(got, plain.forward(nx.CONFIG_B, w, toks), "float32", "a written folder")


def test_the_preset_generates_from_random_weights():
  from simply_b200.config import preset
  cfg = preset("nulezen-tiny")
  assert cfg.architecture == "Nulezen" and cfg.loop == (1, 3, 2)
  ec = EngineConfig(activation_dtype="float32", page_size=8, batch_size=2, max_seq_len=64, use_cuda_graphs=False)
  engine = Engine.from_config(cfg, 1, ec, matrix_std=0.2, ops=ReferenceOps(torch.float32), device="cpu")
  results = engine.generate([[1, 2, 3], [7]], SamplingParams(temperature=0.0, max_decode_steps=5))
  assert [len(r.output_token_ids) for r in results] == [5, 5]
