"""bin/trace_run on the GPU with Nulezen model folders, as a user runs it, against the plain model:
every request whole; most of it in one step and the last 32 tokens one by one; in portions of
changing size; and mixed with other requests in a pool so small that pages and slots are used again."""

import json
import os

import numpy as np
import pytest

from simply_b200.weights import safetensors_io as st
from tests import nulezen_cases as nx
from tests import replay_cases as cases
from tests import trace_util
from tests.plain import nulezen_plain as plain

pytestmark = pytest.mark.gpu

# A model of middling size whose loop lies in the middle (head sizes for the tcgen05 kernel, the
# mma.sync tiles and the general kernel; windows shorter and longer than a page of 64), and the
# small one without whole 16-byte groups.
MIDDLING = nx.config(
    [nx.biased(heads=8, kv_heads=4, dim=32, vdim=32, window=40, scale=0.18), nx.rotated(heads=8, kv_heads=1, dim=48, vdim=48, dims=24, base=5000.0, window=100, scale=0.15),
     nx.biased(heads=4, kv_heads=2, dim=64, vdim=64, window=70, scale=0.12), nx.rotated(heads=4, kv_heads=2, dim=32, vdim=40, dims=32, window=64, scale=0.2)],
    [nx.moe(experts=6, top=2, ff=48, shared=96), nx.dense(ff=192), nx.moe(experts=9, top=3, ff=40, shared=0), None],
    width=256, vocab=384, embed_scale=2.0, logit_scale=0.4, loop=(1, 3, 3))


@pytest.fixture(scope="module")
def models(tmp_path_factory):
  root = tmp_path_factory.mktemp("nulezen_models")
  out = {}
  for which, cfg_dict in (("a", MIDDLING), ("b", nx.CONFIG_C)):
    cfg, t = nx.weights(cfg_dict, seed=17, matrix_std=0.18 if which == "b" else 0.06)
    folder = str(root / which)
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as f:
      json.dump(cfg.to_dict(), f)
    st.write_file(os.path.join(folder, "model.safetensors"), t)
    requests = cases.make_requests(which, cfg_dict["vocab"])
    w = nx.as_numpy(t)
    expected = {rid: plain.forward(cfg_dict, w, toks) for rid, toks in requests.items()}
    out[which] = (folder, cfg_dict["vocab"], requests, expected)
  return out


def compare(got, requests, expected, dtype):
  assert got, "no logits came back"
  for key, rows in sorted(got.items()):
    rid = key.split(":")[1]
    assert sorted(rows) == list(range(len(requests[rid]))), f"{key}: positions missing"
    nx.check_close(np.stack([rows[p] for p in sorted(rows)]), expected[rid], dtype, key)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["a", "b"])
def test_trace_run_four_ways(models, tmp_path, which, dtype):
  folder, vocab, requests, expected = models[which]
  steps = cases.combined_trace(requests)
  out_dir = str(tmp_path / "out")
  trace_util.run_tool(folder, dtype, steps, out_dir, trace_util.tokens_needed(steps, 64))
  compare(trace_util.collect(steps, out_dir, vocab), requests, expected, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_small_pages_poisoned(models, tmp_path, dtype):
  """Pages of 8 tokens, freed pages filled with NaN, the pool exactly as large as the trace needs."""
  folder, vocab, requests, expected = models["a"]
  steps = cases.combined_trace(requests, modes=("mixed", "portions"))
  out_dir = str(tmp_path / "out")
  trace_util.run_tool(folder, dtype, steps, out_dir, trace_util.tokens_needed(steps, 8),
                      extra=("--page-size", "8", "--poison-freed-pages"))
  compare(trace_util.collect(steps, out_dir, vocab), requests, expected, dtype)
