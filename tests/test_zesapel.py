"""The Zesapel decoder through the engine against the plain NumPy model.

Each scenario runs on the CPU with the plain PyTorch kernel statements (this checks the parts,
the configuration, the cache manager and the step function) and, marked `gpu`, with the CUDA
kernels in float32 and bfloat16."""

import copy
import json
import os

import numpy as np
import pytest
import torch

from simply_b200 import Engine, EngineConfig, SamplingParams
from simply_b200.config import ConfigError, config_from_dict, load_config
from simply_b200.weights import safetensors_io
from tests import zesapel_cases as zc
from tests.plain import zesapel_plain as plain
from tests.reference_ops import ReferenceOps

CPU = pytest.param(("float32", "cpu"), id="cpu")
GPU32 = pytest.param(("float32", "cuda"), id="gpu-f32", marks=pytest.mark.gpu)
GPU16 = pytest.param(("bfloat16", "cuda"), id="gpu-bf16", marks=pytest.mark.gpu)
WHERE = [CPU, GPU32, GPU16]
CONFIGS = {"a": zc.CONFIG_A, "b": zc.CONFIG_B, "c": zc.CONFIG_C, "d": zc.CONFIG_D}


def engine_for(cfg_dict, where, seed=0, tensors=None, **kw):
  dtype, device = where
  cfg, t = zc.weights(cfg_dict, seed)
  if tensors is not None:
    t = tensors
  ops = ReferenceOps(torch.float32) if device == "cpu" else None
  return zc.build_engine(cfg, t, dtype, device, ops, **kw), t


def tokens_for(cfg_dict, n, seed):
  return np.random.default_rng(seed).integers(0, cfg_dict["vocab"], n).tolist()


# ---- whole prompts, portions, decoding, batches -------------------------------------------------

@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("which", sorted(CONFIGS))
def test_whole_portions_and_decoding(which, where):
  cfg_dict = CONFIGS[which]
  engine, t = engine_for(cfg_dict, where, seed=3)
  toks = tokens_for(cfg_dict, 61, 1)
  want = plain.forward(cfg_dict, zc.as_numpy(t), toks)
  n = len(toks)
  for what, cuts in [
      ("whole", [n]),
      ("token by token", [1] * n),
      ("prompt then decoding", [n - 40] + [1] * 40),
      ("portions down to two tokens", zc.cuts_of(n, [7, 2, 5, 3, 11, 2, 13, 4, 2, 9])),
      ("portions of two", [2] * (n // 2) + [1]),
      ("one token, then the rest", [1, n - 1]),
  ]:
    zc.check_close(zc.run_cuts(engine, toks, cuts), want, where[0], f"{which}: {what}")
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
  w = zc.as_numpy(t)
  want = [plain.forward(cfg_dict, w, r) for r in requests]
  got = zc.run_mixed(engine, requests, seed=2)
  for i, (g, x) in enumerate(zip(got, want)):
    zc.check_close(g, x, where[0], f"request {i} in a mixed batch")
  # the same requests once more through the used slots and pages, each alone
  for i in (0, 4):
    zc.check_close(zc.run_cuts(engine, requests[i], [len(requests[i])]), want[i], where[0], f"request {i} again")
  engine.cache.check_invariants()
  assert engine.cache.all_pages_free()
  engine.ops.check_errors()


@pytest.mark.parametrize("where", WHERE)
def test_long_decoding_past_windows_and_pages(where):
  cfg_dict = zc.CONFIG_A
  engine, t = engine_for(cfg_dict, where, seed=7, page_size=4)
  toks = tokens_for(cfg_dict, 150, 4)
  want = plain.forward(cfg_dict, zc.as_numpy(t), toks)
  zc.check_close(zc.run_cuts(engine, toks, [3] + [1] * 147), want, where[0], "long decoding")
  engine.ops.check_errors()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_larger_sizes_and_pages_of_64(dtype):
  """330 tokens, windows that pass several pages of 64, head sizes that take the tensor-core tiles,
  states of 64 and 128 rows, two groups, a token with two experts."""
  cfg_dict = zc.config(
      [zc.latent(heads=8, dim=32, rot_dim=16, vdim=32, q_rank=48, kv_rank=64, dims=16, base=5000.0, scale=0.15, window=50),
       zc.delta(heads=3, dim=64),
       zc.mamba(heads=4, vdim=32, state=64, groups=2, norm_groups=2, conv=4),
       zc.latent(heads=6, dim=48, rot_dim=32, vdim=32, q_rank=72, kv_rank=128, dims=8, base=100.0, scale=0.1, window=130),
       zc.delta(heads=1, dim=128)],
      [zc.moe(experts=8, top=2, ff=64), zc.moe(experts=3, top=1, ff=128), None, zc.moe(experts=5, top=3, ff=32),
       zc.moe(experts=4, top=2, ff=64)],
      width=128, vocab=300, streams=2, taps=3, rank=16)
  # (matrices of this size at std 0.1 put the bfloat16 rounding noise of 99,000 logits at the bound itself)
  cfg, t = zc.weights(cfg_dict, seed=3, matrix_std=0.06)
  engine = zc.build_engine(cfg, t, dtype, "cuda", None, page_size=64, slots=2, max_seq_len=512)
  toks = tokens_for(cfg_dict, 330, 1)
  want = plain.forward(cfg_dict, zc.as_numpy(t), toks)
  for what, cuts in [("whole", [330]), ("portions", zc.cuts_of(330, [100, 2, 37, 64, 3, 129])),
                     ("decoding", [270] + [1] * 60)]:
    zc.check_close(zc.run_cuts(engine, toks, cuts), want, dtype, what)
  engine.ops.check_errors()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(1, 32, 16, 70), (2, 16, 16, 33), (20, 64, 16, 100), (24, 288, 32, 150),
                                   (5, 512, 64, None), (3, 96, 160, 64)])
def test_latent_rows_of_every_tile_shape(shape, dtype):
  """Attention over latents alone at shapes that take each form of its tensor-core kernel in
  bfloat16 (single tokens of up to 16, up to 32 and more rows; tiles of 32 and of 64 keys; one and
  two groups of value columns; heads that do not divide a tile), over several pages and tiles."""
  heads, kv_rank, rot_dim, window = shape
  cfg_dict = zc.config([zc.latent(heads=heads, dim=8, rot_dim=rot_dim, vdim=8, q_rank=24, kv_rank=kv_rank, dims=rot_dim // 2,
                                  scale=0.1, window=window)], [None], width=64, vocab=70, streams=0, taps=0)
  cfg, t = zc.weights(cfg_dict, seed=4)
  engine = zc.build_engine(cfg, t, dtype, "cuda", None, page_size=64, slots=2, max_seq_len=512)
  toks = tokens_for(cfg_dict, 300, 2)
  want = plain.forward(cfg_dict, zc.as_numpy(t), toks)
  for what, cuts in [("whole", [300]), ("portions", zc.cuts_of(300, [97, 2, 31, 64, 3, 1, 70])),
                     ("decoding", [230] + [1] * 70)]:
    zc.check_close(zc.run_cuts(engine, toks, cuts), want, dtype, f"{shape}: {what}")
  engine.ops.check_errors()


# ---- a key that stands out ----------------------------------------------------------------------

def needle_case(window, heads=3, tiles=False):
  """A one-layer model whose query of token 1 is answered by the key of token 2 alone.  `tiles`: cached
  rows of a size that the tensor-core kernel over latents takes."""
  sizes = dict(rot_dim=16, kv_rank=32) if tiles else dict(rot_dim=8)
  cfg_dict = zc.config([zc.latent(heads=heads, dim=12, vdim=10, dims=4, scale=1.0, window=window, **sizes)],
                       [None], width=32, vocab=50, streams=2, taps=0)
  cfg, t = zc.weights(cfg_dict, seed=11, matrix_std=0.12 if tiles else 0.25)  # (equal rounding noise at both sizes)
  zc.plant_needle(cfg_dict, t, 0, needle=2, asker=1)
  return cfg_dict, t


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("tiles", [False, True])
def test_a_key_that_stands_out_at_every_edge_of_the_window(tiles, where):
  window = 12
  cfg_dict, t = needle_case(window, tiles=tiles)
  w = zc.as_numpy(t)
  rng = np.random.default_rng(0)
  engine, _ = engine_for(cfg_dict, where, tensors=t, page_size=4)
  for distance in (0, 1, 3, 4, window - 2, window - 1, window, window + 1, 2 * window):
    for at in (0, 1, 3, 4, 7, 8, 30):  # first tokens, page borders (pages of 4), further in
      n = at + distance + 6
      toks = rng.integers(3, cfg_dict["vocab"], n).tolist()
      toks[at] = 2
      toks[at + distance] = 1 if distance else 2
      want = plain.forward(cfg_dict, w, toks)
      # the needle must matter inside the window: the logits with and without it differ
      if 0 < distance < window:
        other = list(toks)
        other[at] = 3
        assert np.abs(plain.forward(cfg_dict, w, other)[at + distance] - want[at + distance]).max() > 0.05 * np.abs(want).max()
      for what, cuts in [("whole", [n]), ("decoded", [at + 1] + [1] * (n - at - 1)),
                         ("cut after the needle", [at + 1, n - at - 1]),
                         ("portions of two", [2] * (n // 2 + 1))]:
        zc.check_close(zc.run_cuts(engine, toks, cuts), want, where[0], f"distance {distance} at {at}: {what}")
  engine.ops.check_errors()


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("tiles", [False, True])
def test_a_far_key_among_hundreds_without_a_window(tiles, where):
  cfg_dict, t = needle_case(None, heads=2, tiles=tiles)
  w = zc.as_numpy(t)
  rng = np.random.default_rng(1)
  engine, _ = engine_for(cfg_dict, where, tensors=t, page_size=16, max_seq_len=512, slots=2)
  n = 400
  toks = rng.integers(3, cfg_dict["vocab"], n).tolist()
  toks[5] = 2
  toks[390] = 1
  want = plain.forward(cfg_dict, w, toks)
  other = list(toks)
  other[5] = 3
  assert np.abs(plain.forward(cfg_dict, w, other)[390] - want[390]).max() > 0.05 * np.abs(want).max()
  for what, cuts in [("whole", [n]), ("decoded", [380] + [1] * 20), ("portions", zc.cuts_of(n, [150, 2, 97, 33]))]:
    zc.check_close(zc.run_cuts(engine, toks, cuts), want, where[0], what)
  engine.ops.check_errors()


# ---- configuration, folders, generation -----------------------------------------------------------

def test_config_round_trip_and_errors():
  cfg = config_from_dict(zc.CONFIG_A)
  assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
  spec = cfg.model_spec()
  assert [l.mixer.kind for l in spec.layers] == ["latent_attention", "generalized_delta_rule", "state_space_duality",
                                                 "latent_attention"]
  assert spec.layers[2].feed_forward.kind == "none"
  for breakage in (lambda d: d["layers"][0].update(type="unknown"), lambda d: d["layers"][0]["mixer"].pop("kv_rank"),
                   lambda d: d["layers"][2]["mixer"].update(groups=3), lambda d: d.pop("norm"),
                   lambda d: d["layers"][0]["mlp"]["router"].update(top=9)):
    bad = copy.deepcopy(zc.CONFIG_A)
    breakage(bad)
    with pytest.raises(ConfigError):
      config_from_dict(bad)


def test_sizes_come_from_the_tensors_where_the_config_names_none():
  """The rank of the decay's low-rank pair is the tensors' own."""
  bare = copy.deepcopy(zc.CONFIG_C)
  bare.pop("decay_rank")
  cfg, t = zc.weights(zc.CONFIG_C, seed=2)
  engine = zc.build_engine(config_from_dict(bare), t, "float32", "cpu", ReferenceOps(torch.float32))
  toks = tokens_for(bare, 19, 3)
  zc.check_close(zc.run_cuts(engine, toks, [19]), plain.forward(bare, zc.as_numpy(t), toks), "float32", "rank from tensors")


@pytest.mark.parametrize("where", WHERE)
def test_greedy_generation_from_a_folder_through_the_scheduler(where, tmp_path):
  dtype, device = where
  cfg_dict = zc.CONFIG_B
  cfg, t = zc.weights(cfg_dict, seed=9)
  folder = str(tmp_path / "model")
  os.makedirs(folder)
  with open(os.path.join(folder, "config.json"), "w") as f:
    json.dump(cfg.to_dict(), f)
  safetensors_io.write_file(os.path.join(folder, "model.safetensors"), t)
  assert load_config(folder).to_dict() == cfg.to_dict()
  ec = EngineConfig(activation_dtype=dtype, page_size=8, batch_size=3, max_seq_len=96, max_cache_tokens=3 * 96,
                    max_num_issue_tokens=16)
  ops = ReferenceOps(torch.float32) if device == "cpu" else None
  engine = Engine.from_folder(folder, ec, ops=ops, device=device)
  prompts = [tokens_for(cfg_dict, n, 20 + n) for n in (5, 31, 1, 18, 40)]
  results = engine.generate(prompts, SamplingParams(temperature=0.0, max_decode_steps=12))
  w = zc.as_numpy(t)
  for p, r in zip(prompts, results):
    g = list(r.output_token_ids)
    assert len(g) == 12
    logits = plain.forward(cfg_dict, w, (p + g)[:-1])
    scale = np.abs(logits).max()
    slack = 1e-4 if dtype == "float32" else 6e-2
    for i, tok in enumerate(g):
      row = logits[len(p) - 1 + i]
      assert row.max() - row[tok] <= slack * scale, (i, tok, int(row.argmax()))
  engine.cache.check_invariants()
  assert engine.cache.all_pages_free()
  engine.ops.check_errors()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_from_graphs_equals_decoding_step_by_step(dtype):
  cfg_dict = zc.CONFIG_A
  cfg, t = zc.weights(cfg_dict, seed=4)
  prompts = [tokens_for(cfg_dict, n, 40 + n) for n in (7, 22, 3)]
  outs = []
  for graphs, burst in ((False, 1), (True, 4)):
    engine = zc.build_engine(cfg, t, dtype, "cuda", None, graphs=graphs, burst=burst)
    results = engine.generate(prompts, SamplingParams(temperature=0.0, max_decode_steps=20))
    outs.append([list(r.output_token_ids) for r in results])
    engine.ops.check_errors()
  assert outs[0] == outs[1]


def test_the_preset_generates_from_random_weights():
  from simply_b200.config import preset
  cfg = preset("zesapel-tiny")
  assert cfg.architecture == "Zesapel" and cfg.streams == 2 and cfg.canon_taps == 3
  kinds = [layer.mixer.kind for layer in cfg.model_spec().layers]
  assert kinds == ["latent_attention", "generalized_delta_rule", "state_space_duality"]
  ec = EngineConfig(activation_dtype="float32", page_size=8, batch_size=2, max_seq_len=64, use_cuda_graphs=False)
  engine = Engine.from_config(cfg, 1, ec, matrix_std=0.2, ops=ReferenceOps(torch.float32), device="cpu")
  results = engine.generate([[1, 2, 3], [7]], SamplingParams(temperature=0.0, max_decode_steps=5))
  assert [len(r.output_token_ids) for r in results] == [5, 5]
