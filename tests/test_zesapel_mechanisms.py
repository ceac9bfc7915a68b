"""Each mechanism of the Zesapel layers alone: calls of the kernel table (the CUDA kernels on a GPU,
their plain PyTorch statements on the CPU) against the functions of the plain NumPy model, and
one-layer models through the engine."""

import math

import numpy as np
import pytest
import torch

from simply_b200.engine.batch import StepEntry, pack_step
from tests import zesapel_cases as zc
from tests.plain import zesapel_plain as plain
from tests.reference_ops import ReferenceOps

CPU = pytest.param(("float32", "cpu"), id="cpu")
GPU32 = pytest.param(("float32", "cuda"), id="gpu-f32", marks=pytest.mark.gpu)
GPU16 = pytest.param(("bfloat16", "cuda"), id="gpu-bf16", marks=pytest.mark.gpu)
WHERE = [CPU, GPU32, GPU16]


def table(where):
  dtype, device = where
  if device == "cpu":
    return ReferenceOps(torch.float32), torch.float32
  from simply_b200.kernels.ops import CudaOps
  return CudaOps(getattr(torch, dtype)), getattr(torch, dtype)


def close(got, want, dtype, what, f32=2e-5, bf16=2e-2):
  got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
  bound = (f32 if dtype == torch.float32 else bf16) * max(np.abs(want).max(), 1e-6)
  assert np.isfinite(got).all(), what
  assert np.abs(got - want).max() <= bound, f"{what}: {np.abs(got - want).max():.3e} over {bound:.3e}"


def context(ops, device, lengths_before, new_counts, slots=None, page_size=8):
  entries = [StepEntry(slots[i] if slots else i, [0] * n, ()) for i, n in enumerate(new_counts)]
  return pack_step(entries, lengths_before, [], page_size, ops, device)


def held(x, dtype, device):
  """What the kernel table gets: values the storage type holds exactly; also returned as float64."""
  t = torch.from_numpy(np.asarray(x, np.float32)).to(dtype)
  return t.to(device), t.float().numpy().astype(np.float64)


def f32(x, device):
  t = torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(device)
  return t, t.cpu().numpy().astype(np.float64)


def walk_in_portions(lengths, slots, schedule, run):
  """Runs `run(rows, ctx_args)` over the schedule's steps; returns per sequence the rows' results.
  `schedule`: per step the number of new tokens of every sequence (0: left out of the step)."""
  starts = np.concatenate([[0], np.cumsum(lengths)[:-1]])
  done = [0] * len(lengths)
  got = [[] for _ in lengths]
  for portions in schedule:
    who = [i for i, p in enumerate(portions) if p]
    rows = np.concatenate([np.arange(starts[i] + done[i], starts[i] + done[i] + portions[i]) for i in who])
    out = run(rows, [done[i] for i in who], [portions[i] for i in who], [slots[i] for i in who])
    at = 0
    for i in who:
      got[i].append(out[at:at + portions[i]])
      at += portions[i]
      done[i] += portions[i]
  return [np.concatenate(g) for g in got]


SCHEDULE = ([5, 9, 64], [1, 0, 2], [1, 0, 1], [17, 0, 3])  # portions, single tokens, a sequence left out
LENGTHS = [24, 9, 70]
SLOTS = [3, 0, 4]  # not in order, slots between them that no request holds


# ---- the generalized delta rule's walk ------------------------------------------------------------

def plain_delta_walk(r, k, v, decay, take):
  t, heads, d = r.shape
  unit = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
  state = np.zeros((heads, d, d))
  o = np.zeros((t, heads, d))
  for i in range(t):
    for a in range(heads):
      old = state[a]
      state[a] = decay[i, a][:, None] * old - np.outer(take[i, a] * unit[i, a], unit[i, a] @ old) + np.outer(k[i, a], v[i, a])
      o[i, a] = state[a].T @ r[i, a]
  return o


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("sizes", [(2, 12), (3, 16), (1, 40), (2, 64), (1, 128), (1, 300), (5, 1), (3, 5)])
def test_the_delta_walk_carries_its_state_between_steps(sizes, where):
  heads, d = sizes
  ops, dtype = table(where)
  device = where[1]
  rng = np.random.default_rng(0)
  total, inner = sum(LENGTHS), heads * d
  scale = 1.0 / math.sqrt(d)
  raw = rng.standard_normal((total, 5 * inner + 3))  # r | k | v | gate | a | columns the walk skips
  raw[:, :3 * inner] *= scale ** 0.5
  pre, pre64 = held(raw, dtype, device)
  low, low64 = held(rng.standard_normal((total, inner)) * 2.0, dtype, device)
  decay_bias, db = f32(rng.standard_normal(inner), device)
  removal_bias, rb = f32(rng.standard_normal(inner), device)
  want, start = [], 0
  for length in LENGTHS:
    x, lw = pre64[start:start + length], low64[start:start + length]
    shape = (length, heads, d)
    decay = np.exp(-math.exp(-0.5) * plain.sigmoid(lw + db)).reshape(shape)
    take = plain.sigmoid(x[:, 4 * inner:5 * inner] + rb).reshape(shape)
    want.append(plain_delta_walk(x[:, :inner].reshape(shape), x[:, inner:2 * inner].reshape(shape),
                                 x[:, 2 * inner:3 * inner].reshape(shape), decay, take))
    start += length
  state = torch.full((5, heads, d, d), float("nan"), device=device)
  for s in SLOTS:
    state[s].zero_()

  def run(rows, before, new, slots):
    ctx = context(ops, device, before, new, slots=slots)
    idx = torch.from_numpy(rows).to(device)
    return ops.general_delta_scan(pre[idx].contiguous(), low[idx].contiguous(), decay_bias, removal_bias, state, ctx,
                                  num_heads=heads, head_dim=d).float().cpu().numpy()
  got = walk_in_portions(LENGTHS, SLOTS, SCHEDULE, run)
  for i, g in enumerate(got):
    close(g, want[i][:len(g)], torch.float32, f"sequence {i} of sizes {sizes}", f32=3e-5)
  assert torch.isnan(state[1]).all() and torch.isnan(state[2]).all(), "a slot no request holds was written"


# ---- the state-space walk -------------------------------------------------------------------------

@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("sizes", [(4, 6, 10, 2), (2, 16, 8, 1), (3, 8, 4, 3), (4, 64, 128, 2), (1, 3, 300, 1),
                                   (6, 1, 1, 3), (3, 5, 7, 1), (3, 5, 20, 1), (2, 40, 64, 2), (5, 16, 16, 1),
                                   (2, 24, 100, 1)])
def test_the_state_space_walk_carries_its_state_between_steps(sizes, where):
  heads, dv, n, groups = sizes
  ops, dtype = table(where)
  device = where[1]
  rng = np.random.default_rng(1)
  total, inner = sum(LENGTHS), heads * dv
  xbc, xbc64 = f32(rng.standard_normal((total, inner + 2 * groups * n)) / math.sqrt(math.sqrt(n)), device)
  pre, pre64 = held(rng.standard_normal((total, 2 + heads)), dtype, device)  # two columns the walk skips, then dt
  step_bias, sb = f32(rng.standard_normal(heads), device)
  rate_log = rng.standard_normal(heads) * 0.5 - 1.0
  neg_rate, nr = f32(-np.exp(rate_log), device)
  skip, sk = f32(rng.standard_normal(heads), device)
  per = heads // groups
  want, start = [], 0
  for length in LENGTHS:
    x = xbc64[start:start + length, :inner].reshape(length, heads, dv)
    bm = xbc64[start:start + length, inner:inner + groups * n].reshape(length, groups, n)
    cm = xbc64[start:start + length, inner + groups * n:].reshape(length, groups, n)
    dt = plain.softplus(pre64[start:start + length, 2:] + sb)
    s = np.zeros((heads, n, dv))
    y = np.zeros((length, heads, dv))
    for t in range(length):
      for a in range(heads):
        g = a // per
        s[a] = math.exp(nr[a] * dt[t, a]) * s[a] + dt[t, a] * np.outer(bm[t, g], x[t, a])
        y[t, a] = s[a].T @ cm[t, g] + sk[a] * x[t, a]
    want.append(y)
    start += length
  state = torch.full((5, heads, n, dv), float("nan"), device=device)
  for s in SLOTS:
    state[s].zero_()

  def run(rows, before, new, slots):
    ctx = context(ops, device, before, new, slots=slots)
    idx = torch.from_numpy(rows).to(device)
    return ops.state_space_scan(xbc[idx].contiguous(), pre[idx].contiguous(), 2, step_bias, neg_rate, skip, state, ctx,
                                num_heads=heads, value_dim=dv, state_dim=n, num_groups=groups).float().cpu().numpy()
  got = walk_in_portions(LENGTHS, SLOTS, SCHEDULE, run)
  for i, g in enumerate(got):
    close(g, want[i][:len(g)], torch.float32, f"sequence {i} of sizes {sizes}", f32=3e-5)
  assert torch.isnan(state[1]).all() and torch.isnan(state[2]).all(), "a slot no request holds was written"


# ---- the short convolution ------------------------------------------------------------------------

@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("sizes", [(2, 40, 0, True), (4, 36, 5, False), (3, 7, 0, False), (6, 16, 3, True), (1, 12, 0, True)])
def test_the_short_convolution_keeps_its_last_inputs_between_steps(sizes, where):
  taps, channels, offset, residual = sizes
  ops, dtype = table(where)
  device = where[1]
  rng = np.random.default_rng(2)
  total = sum(LENGTHS)
  x, x64 = held(rng.standard_normal((total, offset + channels + 2)), dtype, device)
  w, w64 = f32(rng.standard_normal((channels, taps)) * 0.5, device)
  b, b64 = (None, None) if residual else f32(rng.standard_normal(channels) * 0.3, device)
  want, start = [], 0
  for length in LENGTHS:
    xs = x64[start:start + length, offset:offset + channels]
    y = plain.causal_conv(xs, w64, b64)
    want.append(xs + y if residual else plain.silu(y))
    start += length
  state = torch.full((5, max(taps - 1, 1), channels), float("nan"), device=device) if taps > 1 else None
  if state is not None:
    for s in SLOTS:
      state[s].zero_()

  def run(rows, before, new, slots):
    ctx = context(ops, device, before, new, slots=slots)
    idx = torch.from_numpy(rows).to(device)
    return ops.short_conv(x[idx].contiguous(), w, b, state, ctx, activation=0 if residual else 1, residual=residual,
                          offset=offset, channels=channels, out_dtype=torch.float32).float().cpu().numpy()
  # single tokens first: steps shorter than the taps, where old inputs must move up in the state
  schedule = ([1, 1, 1], [1, 0, 2], [2, 3, 1], [20, 5, 60], [0, 0, 6])
  got = walk_in_portions(LENGTHS, SLOTS, schedule, run)
  for i, g in enumerate(got):
    close(g, want[i][:len(g)], torch.float32, f"sequence {i} of sizes {sizes}", f32=1e-5)
  if state is not None:
    assert torch.isnan(state[1]).all() and torch.isnan(state[2]).all(), "a slot no request holds was written"


# ---- the streams ------------------------------------------------------------------------------------

@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("sizes", [(1, 24), (2, 40), (3, 36), (4, 7), (5, 130)])
def test_streams_are_read_and_written_all_at_once(sizes, where):
  copies, width = sizes
  ops, dtype = table(where)
  device = where[1]
  rng = np.random.default_rng(3)
  t = 11
  x, x64 = f32(rng.standard_normal((t, width)), device)
  lanes = ops.spread_streams(x, copies)
  want = np.stack([x64] * copies)  # [S, T, W]
  eps = 1e-5
  for step in range(3):
    w_in, w_in64 = f32(rng.standard_normal(copies), device)
    mix, mix64 = f32(rng.standard_normal((copies, copies)) * 0.5 + np.eye(copies), device)
    w_out, w_out64 = f32(rng.standard_normal(copies), device)
    norm_w, norm64 = f32(rng.uniform(0.5, 1.5, width), device)
    branch, branch64 = held(rng.standard_normal((t, width)), dtype, device)
    want = plain.streams_write(want, branch64, mix64, w_out64)
    # a write and the next sublayer's read and norm are one call
    got = ops.streams_step(lanes, branch, mix, w_out, w_in, norm_w, eps, False, None)
    close(lanes.permute(1, 0, 2).cpu().numpy(), want, torch.float32, f"streams after write {step}", f32=1e-5)
    close(got.float().cpu().numpy(), plain.rms(plain.streams_read(want, w_in64), eps) * norm64[None, :], dtype,
          f"read {step}", f32=1e-5, bf16=1e-2)
  ones, ones64 = f32(np.ones(copies), device)
  close(ops.streams_step(lanes, None, None, None, ones, None, eps, False, None).cpu().numpy(), want.sum(0),
        torch.float32, "the sum of the streams", f32=1e-5)
  # only some rows, with the last write folded in and nothing written
  before = lanes.clone()
  rows = torch.tensor([7, 2, 10], dtype=torch.int32, device=device)
  branch, branch64 = held(rng.standard_normal((t, width)), dtype, device)
  got = ops.streams_step(lanes, branch, mix, w_out, ones, None, eps, False, rows)
  close(got.cpu().numpy(), plain.streams_write(want, branch64, mix64, w_out64).sum(0)[[7, 2, 10]], torch.float32,
        "rows of the sum", f32=1e-5)
  assert torch.equal(before, lanes)


# ---- norm in parts with a gate ----------------------------------------------------------------------

@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("sizes", [(24, 1), (24, 3), (30, 5), (128, 2), (7, 7), (520, 1)])
@pytest.mark.parametrize("kind", ["silu_before", "sigmoid_after", "none"])
def test_norm_in_equal_parts_with_the_gate_before_or_after(kind, sizes, where):
  n, groups = sizes
  ops, dtype = table(where)
  device = where[1]
  rng = np.random.default_rng(4)
  t, offset = 9, 3
  o, o64 = f32(rng.standard_normal((t, n)) * 3.0, device)
  gate, gate64 = held(rng.standard_normal((t, offset + n + 2)), dtype, device)
  w, w64 = f32(rng.uniform(0.5, 1.5, n), device)
  g = gate64[:, offset:offset + n]
  y = o64 * plain.silu(g) if kind == "silu_before" else o64
  y = plain.rms(y.reshape(t, groups, n // groups), 1e-5).reshape(t, n) * w64[None, :]
  if kind == "sigmoid_after":
    y = y * plain.sigmoid(g)
  got = ops.group_norm_gate(o, w, 1e-5, groups=groups, gate=gate if kind != "none" else None, gate_offset=offset,
                            gate_kind=kind)
  close(got.float().cpu().numpy(), y, dtype, f"{kind} {sizes}", f32=1e-5, bf16=1e-2)


# ---- table experts ----------------------------------------------------------------------------------

@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("sizes", [(5, 2, 16, 40), (3, 1, 24, 36), (7, 4, 8, 48), (4, 3, 12, 40), (2, 2, 9, 35)])
def test_experts_by_table_with_equal_weights(sizes, where):
  experts, top, ff, width = sizes
  ops, dtype = table(where)
  device = where[1]
  rng = np.random.default_rng(5)
  vocab, t = 30, 37
  tab = np.stack([rng.permutation(experts)[:top] for _ in range(vocab)]).astype(np.int32)
  ids = rng.integers(0, vocab, t).astype(np.int32)
  x, x64 = held(rng.standard_normal((t, width)), dtype, device)
  up, up64 = held(rng.standard_normal((experts, ff, width)) / math.sqrt(width), dtype, device)
  down, down64 = held(rng.standard_normal((experts, width, ff)) / math.sqrt(ff), dtype, device)
  w = {"p.table": tab}
  for e in range(experts):
    w[f"p.e{e}.up"], w[f"p.e{e}.down"] = up64[e], down64[e]
  want = plain.table_experts(x64, ids, {"router": {"top": top}}, w, "p")
  chosen, weight = ops.route_by_table(torch.from_numpy(ids).to(device), torch.from_numpy(tab).to(device), experts)
  assert torch.equal(chosen.cpu(), torch.from_numpy(tab[ids]))
  assert torch.allclose(weight.cpu(), torch.full((t, top), 1.0 / top))
  from simply_b200.registry import ACTIVATIONS
  from simply_b200.parts import experts as _  # noqa: F401  (registers the feed-forward and its activation)
  got = ops.mix_experts(x, chosen, weight, up.contiguous(), down.contiguous(), experts, ACTIVATIONS.get("gelu_erf"),
                        None, None, gated=False)
  close(got.float().cpu().numpy(), want, dtype, f"experts {sizes}", f32=2e-5, bf16=3e-2)
  if hasattr(ops, "expert_rows_for_dense_products"):
    # both ways of multiplying: expert by expert through the dense products, and the grouped kernel
    before = ops.expert_rows_for_dense_products
    for threshold in (0, 1):
      ops.expert_rows_for_dense_products = threshold
      got = ops.mix_experts(x, chosen, weight, up.contiguous(), down.contiguous(), experts, ACTIVATIONS.get("gelu_erf"),
                            None, None, gated=False)
      close(got.float().cpu().numpy(), want, dtype, f"experts {sizes}, threshold {threshold}", f32=2e-5, bf16=3e-2)
    ops.expert_rows_for_dense_products = before
    ops.check_errors()


# ---- one-layer models: every mixer alone at sizes of many kinds ------------------------------------------

ONE_LAYER = {
    "latent: dims below the rotated part": zc.latent(heads=3, dim=12, rot_dim=8, vdim=10, dims=4, window=6),
    "latent: the whole rotated part turns": zc.latent(heads=2, dim=8, rot_dim=12, vdim=8, dims=12, window=9),
    "latent: nothing turns": zc.latent(heads=2, dim=8, rot_dim=4, vdim=16, dims=0, window=4),
    "latent: one head, window of one": zc.latent(heads=1, dim=16, rot_dim=2, vdim=4, q_rank=3, kv_rank=5, dims=2, window=1),
    "latent: window of two": zc.latent(heads=5, dim=4, rot_dim=4, vdim=4, q_rank=8, kv_rank=6, dims=4, window=2),
    "latent: no window": zc.latent(heads=4, dim=8, rot_dim=8, vdim=12, dims=2, window=None),
    "latent: sizes of tensor-core tiles": zc.latent(heads=4, dim=32, rot_dim=16, vdim=32, q_rank=32, kv_rank=48, dims=16, window=20),
    "delta: one head": zc.delta(heads=1, dim=24),
    "delta: odd sizes": zc.delta(heads=5, dim=7),
    "delta: heads of 64": zc.delta(heads=2, dim=64),
    "state space: groups and norm groups": zc.mamba(heads=6, vdim=4, state=5, groups=3, norm_groups=4, conv=3),
    "state space: one of each": zc.mamba(heads=1, vdim=8, state=16, groups=1, norm_groups=1, conv=2),
    "state space: one tap": zc.mamba(heads=2, vdim=8, state=8, groups=2, norm_groups=2, conv=1),
    "state space: five taps": zc.mamba(heads=4, vdim=16, state=32, groups=1, norm_groups=2, conv=5),
}


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_one_layer_models(name, where):
  dtype, device = where
  for streams, taps, mlp in ((0, 0, None), (2, 3, zc.moe(experts=3, top=2, ff=8))):
    cfg_dict = zc.config([ONE_LAYER[name]], [mlp], width=32, vocab=41, streams=streams, taps=taps, rank=4)
    cfg, t = zc.weights(cfg_dict, seed=6)
    ops = ReferenceOps(torch.float32) if device == "cpu" else None
    engine = zc.build_engine(cfg, t, dtype, device, ops, page_size=4)
    toks = np.random.default_rng(8).integers(0, 41, 45).tolist()
    want = plain.forward(cfg_dict, zc.as_numpy(t), toks)
    for what, cuts in [("whole", [45]), ("decoded", [20] + [1] * 25), ("portions", zc.cuts_of(45, [3, 2, 9, 2, 14]))]:
      zc.check_close(zc.run_cuts(engine, toks, cuts), want, dtype, f"{name} (streams {streams}): {what}")
    engine.ops.check_errors()


@pytest.mark.parametrize("where", WHERE)
def test_the_sink_takes_its_share_and_the_gate_scales_heads(where):
  """A large sink on one head leaves that head's output near zero; without sinks the softmax sums to
  one.  The model's logits move accordingly, in the engine as in the plain model."""
  dtype, device = where
  cfg_dict = zc.config([zc.latent(heads=2, dim=8, rot_dim=4, vdim=8, dims=4, window=7)], [None], width=32, vocab=41,
                       streams=0, taps=0)
  cfg, t = zc.weights(cfg_dict, seed=12, matrix_std=0.25)
  toks = np.random.default_rng(9).integers(0, 41, 30).tolist()
  ops = ReferenceOps(torch.float32) if device == "cpu" else None
  seen = []
  for sink in ([-30.0, -30.0], [6.0, -30.0], [0.5, 2.0]):
    t["l0.mix.sink"] = torch.tensor(sink).to(torch.bfloat16)
    engine = zc.build_engine(cfg, t, dtype, device, ops)
    want = plain.forward(cfg_dict, zc.as_numpy(t), toks)
    got = zc.run_cuts(engine, toks, [11] + [1] * 19)
    zc.check_close(got, want, dtype, f"sinks {sink}")
    seen.append(want)
  assert np.abs(seen[0] - seen[1]).max() > 0.05 * np.abs(seen[0]).max()
  assert np.abs(seen[0] - seen[2]).max() > 0.05 * np.abs(seen[0]).max()


@pytest.mark.parametrize("where", WHERE)
def test_one_tap_on_the_input_and_four_streams(where):
  """Values that other tests leave out: a convolution of a single tap (no kept inputs at all) on what the
  mixer reads, four streams, a window as long as the sequence."""
  dtype, device = where
  cfg_dict = zc.config([zc.delta(heads=2, dim=8), zc.latent(heads=2, dim=8, rot_dim=8, vdim=8, q_rank=8, kv_rank=8, dims=8, window=45),
                        zc.mamba(heads=2, vdim=8, state=16, groups=1, norm_groups=1, conv=2)],
                       [zc.moe(experts=2, top=1, ff=8), None, zc.moe(experts=4, top=4, ff=8)], width=24, vocab=41, streams=4,
                       taps=1, rank=2)
  cfg, t = zc.weights(cfg_dict, seed=13)
  ops = ReferenceOps(torch.float32) if device == "cpu" else None
  engine = zc.build_engine(cfg, t, dtype, device, ops, page_size=4)
  toks = np.random.default_rng(3).integers(0, 41, 45).tolist()
  want = plain.forward(cfg_dict, zc.as_numpy(t), toks)
  for what, cuts in [("whole", [45]), ("decoded", [20] + [1] * 25), ("portions", zc.cuts_of(45, [3, 2, 9, 2, 14]))]:
    zc.check_close(zc.run_cuts(engine, toks, cuts), want, dtype, what)
  engine.ops.check_errors()
