"""Each mechanism of the Nulezen layers alone: one call of the kernel table (the CUDA kernels on a
GPU, their plain PyTorch statements on the CPU) against the function of the plain NumPy model, and
one-layer models through the engine with the stream after every layer call compared."""

import types

import numpy as np
import pytest
import torch

from simply_b200.cache import CacheManager, PagedKVNeed
from simply_b200.engine.batch import StepEntry
from simply_b200.parts.normed_attention import rotation_frequencies
from tests import nulezen_cases as nx
from tests.plain import nulezen_plain as plain
from tests.test_sapivik_mechanisms import close, context, held, table

CPU = pytest.param(("float32", "cpu"), id="cpu")
GPU32 = pytest.param(("float32", "cuda"), id="gpu-f32", marks=pytest.mark.gpu)
GPU16 = pytest.param(("bfloat16", "cuda"), id="gpu-bf16", marks=pytest.mark.gpu)
WHERE = [CPU, GPU32, GPU16]


def f32(x, device):
  return torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(device)


# ---- the norm without statistics, branches with a factor per channel ------------------------------------

@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("rows,width", [(5, 32), (3, 37), (70, 200), (2, 1030), (1, 6)])
def test_scaled_branches_and_the_tanh_norm(rows, width, where):
  ops, dtype = table(where)
  device = where[1]
  rng = np.random.default_rng(0)
  h64 = rng.standard_normal((rows, width)) * 3.0
  b1, b1_64 = held(rng.standard_normal((rows, width)), dtype, device)
  b2, b2_64 = held(rng.standard_normal((rows, width)), dtype, device)
  s1, s2 = rng.uniform(0.5, 1.5, width), rng.uniform(-1.0, 1.0, width)
  norm = types.SimpleNamespace(alpha=f32([0.6], device), weight=f32(rng.uniform(0.5, 1.5, width), device),
                               bias=f32(rng.standard_normal(width) * 0.3, device))
  a, w, b = (x.cpu().numpy().astype(np.float64) for x in (norm.alpha, norm.weight, norm.bias))
  s1_t, s2_t = f32(s1, device), f32(s2, device)
  s1, s2 = s1_t.cpu().numpy().astype(np.float64), s2_t.cpu().numpy().astype(np.float64)
  # both branches with factors, then the norm
  h = f32(h64, device)
  h64 = h.cpu().numpy().astype(np.float64)
  y = ops.scaled_residual_tanh(h, b1, s1_t, b2, s2_t, norm, None)
  want_h = h64 + s1 * b1_64 + s2 * b2_64
  close(h.cpu().numpy(), want_h, torch.float32, "the stream after both branches")
  close(y.float().cpu().numpy(), plain.dyt(want_h, a[0], w, b), dtype, "the normed stream")
  # one branch as it is, no norm; then the norm alone; then some rows only, the stream untouched
  h = f32(h64, device)
  assert ops.scaled_residual_tanh(h, None, None, b2, None, None, None) is None
  close(h.cpu().numpy(), h64 + b2_64, torch.float32, "a branch without factors")
  before = h.clone()
  y = ops.scaled_residual_tanh(h, None, None, None, None, norm, None)
  assert torch.equal(h, before)
  close(y.float().cpu().numpy(), plain.dyt(h64 + b2_64, a[0], w, b), dtype, "the norm alone")
  pick = [rows - 1, 0, rows - 1]
  y = ops.scaled_residual_tanh(h, b1, s1_t, None, None, norm, torch.tensor(pick, dtype=torch.int32, device=device))
  assert torch.equal(h, before), "a gathered read must leave the stream as it is"
  close(y.float().cpu().numpy(), plain.dyt((h64 + b2_64 + s1 * b1_64)[pick], a[0], w, b), dtype, "gathered rows")
  close(ops.scale_channels(b1, s2_t).float().cpu().numpy(), b1_64 * s2, dtype, "factors alone")


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("rows,width", [(3, 24), (40, 64), (200, 40)])
def test_the_stream_input_and_the_scaled_output_layer(rows, width, where):
  ops, dtype = table(where)
  device = where[1]
  rng = np.random.default_rng(1)
  x, x0 = f32(rng.standard_normal((rows, width)), device), f32(rng.standard_normal((rows, width)), device)
  w_in, w64 = held(rng.standard_normal((width, 2 * width)) * 0.2, dtype, device)
  step = f32(rng.standard_normal(width), device)
  both = ops.pack_pair(x, x0)
  assert both.shape == (rows, 2 * width) and both.dtype == dtype
  out = ops.linear_wide(both, w_in, step)
  assert out.dtype == torch.float32
  both64 = both.float().cpu().numpy().astype(np.float64)
  close(both64, np.concatenate([x.cpu().numpy(), x0.cpu().numpy()], axis=1), dtype, "side by side", bf16=4e-3)
  close(out.cpu().numpy(), both64 @ w64.T + step.cpu().numpy().astype(np.float64), torch.float32, "W [x; x0] + step",
        f32=2e-5 if dtype == torch.float32 else 1e-3)
  table_t, table64 = held(rng.standard_normal((50, width)), dtype, device)
  y, y64 = held(rng.standard_normal((rows, width)), dtype, device)
  close(ops.lm_head(y, table_t, 0.0, scale=0.3).cpu().numpy(), (y64 @ table64.T) * 0.3, torch.float32, "scaled logits",
        f32=2e-5 if dtype == torch.float32 else 1e-3)


# ---- feed-forwards -------------------------------------------------------------------------------------

@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("rows,width,hidden", [(3, 24, 20), (40, 64, 64), (200, 40, 24)])
def test_the_learned_activation(rows, width, hidden, where):
  ops, dtype = table(where)
  device = where[1]
  rng = np.random.default_rng(2)
  x, x64 = held(rng.standard_normal((rows, width)), dtype, device)
  up, up64 = held(rng.standard_normal((hidden, width)) * 0.5, dtype, device)
  for p, q in [(0.3, -0.8), (-2.0, 1.5), (0.0, 0.0)]:
    got = ops.linear_xielu(x, up, f32([p, q], device)).float().cpu().numpy()
    z = x64 @ up64.T
    if dtype == torch.bfloat16:  # (the product is stored in bfloat16 before the activation)
      z = torch.from_numpy(z).to(torch.bfloat16).double().numpy()
    close(got, plain.xielu(z, p, q), dtype, f"xielu with p {p}, q {q}")
    # with the host's factors a step of few tokens activates on the product's sums
    factors = (plain.softplus(p), 0.5 + plain.softplus(q))
    for n in (1, min(rows, 9), min(rows, 16), rows):
      got = ops.linear_xielu(x[:n].contiguous(), up, f32([p, q], device), factors).float().cpu().numpy()
      close(got, plain.xielu(z[:n], p, q), dtype, f"xielu with p {p}, q {q}, {n} rows, factors from the host")
  z = np.linspace(-30.0, 12.0, 85).reshape(1, -1)
  for v in (-1e-3, 0.0, 1e-3):
    z[0, int(abs(v) * 1e3) + 3] = v
  assert np.allclose(plain.xielu(z, 0.3, -0.8)[z <= 0], (0.5 + plain.softplus(-0.8)) * (np.exp(z[z <= 0]) - 1 - z[z <= 0]) + 0.5 * z[z <= 0])


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("sizes", [(8, 3, 24, 40), (37, 37, 16, 8), (3, 1, 72, 20), (2, 2, 64, 32)])
def test_routing_by_the_largest_logits_and_the_clamped_experts(sizes, where):
  experts, top, width, ff = sizes
  ops, dtype = table(where)
  device = where[1]
  rng = np.random.default_rng(4)
  rows = 200  # with few experts: more rows per expert than a tile holds
  w, w64 = {}, {}
  def put(name, value):
    w[name], w64[name] = held(value, dtype, device)
  for e in range(experts):
    put(f"m.e{e}.gate", rng.standard_normal((ff, width)) * 0.5)
    put(f"m.e{e}.up", rng.standard_normal((ff, width)) * 0.5)
    put(f"m.e{e}.down", rng.standard_normal((width, ff)) * 0.3)
  put("m.router", rng.standard_normal((experts, width)))
  put("m.router.b", rng.standard_normal(experts) * 2.0)  # large enough to change who is chosen
  for part, n in (("gate", 16), ("up", 16)):
    put(f"m.shared.{part}", rng.standard_normal((n, width)) * 0.5)
  put("m.shared.down", rng.standard_normal((width, 16)) * 0.3)
  x, x64 = held(rng.standard_normal((rows, width)), dtype, device)
  chosen64, weight64 = plain.route(x64, w64["m.router"], w64["m.router.b"], top)
  unbiased, _ = plain.route(x64, w64["m.router"], np.zeros(experts), top)
  assert top == experts or not np.array_equal(np.sort(unbiased, axis=1), np.sort(chosen64, axis=1)), \
      "the router's bias never changed a choice: the test's weights are too weak"
  chosen, weight, gate = ops.route_tokens(x, w["m.router"].float().contiguous(), None, None, top=top, scale=1.0,
                                          score=0, renormalize=True, bias=w["m.router.b"].float().contiguous())
  assert gate is None
  assert np.array_equal(chosen.cpu().numpy(), chosen64), "the chosen experts differ"
  close(weight.cpu().numpy(), weight64, torch.float32, "weights", f32=1e-4)
  assert np.allclose(weight.cpu().numpy().sum(axis=1), 1.0, atol=1e-5)
  mlp = {"kind": "moe", "expert": {"ff": ff, "limit": 0.9}, "router": {"experts": experts, "top": top},
         "shared": {"ff": 16, "limit": 1.7}}
  want = plain.moe_ff(x64, w64, "m", mlp)
  gate_up = torch.stack([torch.cat([w[f"m.e{e}.gate"], w[f"m.e{e}.up"]]) for e in range(experts)]).contiguous()
  down = torch.stack([w[f"m.e{e}.down"] for e in range(experts)]).contiguous()
  shared = ops.linear(ops.gated_linear(x, torch.cat([w["m.shared.gate"], w["m.shared.up"]]).contiguous(), 3, limit=1.7),
                      w["m.shared.down"])
  for dense_rows in (0, 1):  # the grouped kernel, and (bfloat16 on a GPU) every expert through the dense products
    if hasattr(ops, "expert_rows_for_dense_products"):
      ops.expert_rows_for_dense_products = dense_rows
    got = ops.mix_experts(x, chosen, weight, gate_up, down, experts, 3, shared, None, limit=0.9).float().cpu().numpy()
    close(got, want, dtype, f"experts and the shared expert (dense route from {dense_rows} rows)", f32=5e-5, bf16=4e-2)
  clamped = np.mean(np.abs(x64 @ w64["m.e0.gate"].T) > 0.9)
  assert 0.05 < clamped < 0.95, "the limit must cut some sums and leave others"


# ---- attention: biases, rotation by halves, value heads of another size, the distance bias, gates -----

@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("sizes", [(4, 2, 16, 16, 8, True), (3, 1, 20, 12, 20, True), (2, 2, 64, 64, 0, False), (6, 3, 12, 20, 4, True),
                                   (10, 2, 96, 96, 48, True)])
def test_biases_rotation_by_halves_and_the_stores(sizes, where):
  heads, kv_heads, d, dv, dims, with_bias = sizes
  ops, dtype = table(where)
  device = where[1]
  rng = np.random.default_rng(2)
  page_size, lengths_before, new = 8, [13, 0], [9, 5]
  need = PagedKVNeed(kv_heads, d, None, value_dim=None if dv == d else dv)
  mgr = CacheManager({"c": need}, page_size=page_size, max_slots=3, max_seq_len=64, max_cache_tokens=128, dtype=dtype,
                     device=device)
  slots = [mgr.acquire_slot(i) for i in range(2)]
  mgr.extend([(slots[0], lengths_before[0])])
  mgr.extend([(s, n) for s, n in zip(slots, new)])
  ctx = context(ops, device, lengths_before, new, slots=slots, tables=[g.tables for g in mgr.groups], page_size=page_size)
  total = sum(new)
  nq, nk, nv = heads * d, kv_heads * d, kv_heads * dv
  proj, proj64 = held(rng.standard_normal((total, nq + nk + nv + heads + 5)), dtype, device)
  bias = rng.standard_normal(nq + nk + nv) if with_bias else None
  bias_t = f32(bias, device) if with_bias else None
  bias64 = bias_t.cpu().numpy().astype(np.float64) if with_bias else np.zeros(nq + nk + nv)
  freq = torch.from_numpy(rotation_frequencies(dims, 300.0)).to(device) if dims else None
  storage = mgr.paged["c"].storage
  storage.fill_(float("nan"))
  more = {}
  if dv != d:
    more["value_dim"] = dv
  if with_bias:
    more["bias"] = bias_t
  q = ops.rotate_headnorm_store(proj, 0.0, 0.37, freq, interleaved=False, head_norm=False, tie_values=False,
                                num_heads=heads, num_kv_heads=kv_heads, head_dim=d, storage=storage,
                                block_table=ctx.block_tables[0], ctx=ctx, **more).float().cpu().numpy()
  positions = np.concatenate([np.arange(b, b + n) for b, n in zip(lengths_before, new)]).astype(np.float64)
  cols = proj64[:, :nq + nk + nv] + bias64
  want_q = plain.rotate_halves(cols[:, :nq].reshape(total, heads, d), positions, dims, 300.0) * 0.37
  want_k = plain.rotate_halves(cols[:, nq:nq + nk].reshape(total, kv_heads, d), positions, dims, 300.0)
  want_v = cols[:, nq + nk:].reshape(total, kv_heads, dv)
  close(q.reshape(total, heads, d), want_q, dtype, "queries", bf16=1e-2)
  flat = storage.float().cpu().numpy().reshape(storage.shape[0], -1)
  keys = flat[:, :kv_heads * page_size * d].reshape(-1, kv_heads, page_size, d)
  values = flat[:, kv_heads * page_size * d:].reshape(-1, kv_heads, page_size, dv)
  tables = mgr.groups[0].tables
  row = 0
  for s, b, n in zip(slots, lengths_before, new):
    for p in range(b, b + n):
      page = int(tables[s, p // page_size])
      close(keys[page, :, p % page_size, :], want_k[row], dtype, f"key at {p}", bf16=1e-2)
      close(values[page, :, p % page_size, :], want_v[row], dtype, f"value at {p}", bf16=1e-2)
      row += 1
  # one gate per head, read out of the same projection
  x, x64 = held(rng.standard_normal((total, heads * dv)), dtype, device)
  got = ops.sigmoid_gate(x.clone(), proj, nq + nk + nv, dv).float().cpu().numpy()
  want = x64.reshape(total, heads, dv) * plain.sigmoid(proj64[:, nq + nk + nv:nq + nk + nv + heads])[:, :, None]
  close(got, want.reshape(total, heads * dv), dtype, "a gate per head")


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("sizes", [(4, 2, 16, 16, 12), (3, 1, 20, 12, 40), (2, 2, 64, 64, 33), (6, 3, 12, 20, 1), (10, 2, 96, 96, 70),
                                   (8, 2, 64, 64, 200), (4, 2, 128, 128, 100), (16, 1, 64, 64, 50), (32, 1, 64, 64, 90),
                                   (8, 2, 64, 64, 4000)])
def test_windowed_attention_with_the_distance_bias(sizes, where):
  """Three sequences side by side: a prompt's portion that starts inside a page with older keys in
  the cache, a single token far into its sequence, and a first portion; keys and values are written
  into pages taken out of order."""
  heads, kv_heads, d, dv, window = sizes
  ops, dtype = table(where)
  device = where[1]
  rng = np.random.default_rng(5)
  page_size = 16
  lengths_before, new = [37, 150, 0], [21, 1, 45]
  need = PagedKVNeed(kv_heads, d, None, value_dim=None if dv == d else dv)
  mgr = CacheManager({"c": need}, page_size=page_size, max_slots=4, max_seq_len=256, max_cache_tokens=512, dtype=dtype,
                     device=device)
  slots = [mgr.acquire_slot(i) for i in range(3)]
  for s, b in zip(slots[::-1], lengths_before[::-1]):
    if b:
      mgr.extend([(s, b)])
  mgr.extend([(s, n) for s, n in zip(slots, new)])
  storage = mgr.paged["c"].storage
  storage.fill_(float("nan"))
  tables = mgr.groups[0].tables
  flat = storage.view(storage.shape[0], -1)
  keys = flat[:, :kv_heads * page_size * d].view(-1, kv_heads, page_size, d)
  values = flat[:, kv_heads * page_size * d:].view(-1, kv_heads, page_size, dv)
  r1, r2 = f32(rng.uniform(0.0, 2.0, heads), device), f32(rng.uniform(0.1, 3.0, heads), device)
  bias = (r1.cpu().numpy().astype(np.float64), r2.cpu().numpy().astype(np.float64))
  q_rows, want = [], []
  for s, b, n in zip(slots, lengths_before, new):
    t = b + n
    k, k64 = held(rng.standard_normal((t, kv_heads, d)), dtype, device)
    v, v64 = held(rng.standard_normal((t, kv_heads, dv)), dtype, device)
    q, q64 = held(rng.standard_normal((t, heads, d)) * 0.5, dtype, device)
    for p in range(t):
      page = int(tables[s, p // page_size])
      keys[page, :, p % page_size] = k[p]
      values[page, :, p % page_size] = v[p]
    q_rows.append(q[b:])
    want.append(plain.windowed_attention(q64, k64, v64, 1.0, window, bias)[b:].reshape(n, heads * dv))
  ctx = context(ops, device, lengths_before, new, slots=slots, tables=[g.tables for g in mgr.groups], page_size=page_size)
  more = {"value_dim": dv} if dv != d else {}
  got = ops.paged_attention(torch.cat(q_rows).contiguous(), storage, ctx.block_tables[0], ctx, num_heads=heads,
                            num_kv_heads=kv_heads, head_dim=d, logit_softcap=0.0, window=window,
                            distance_bias=torch.stack([r1, r2]).contiguous(), **more).float().cpu().numpy()
  close(got, np.concatenate(want), dtype, "attention with the distance bias", bf16=2e-2)
  if hasattr(ops, "prefill_tcgen05"):
    # once more with the prompt portions on the mma.sync tiles where the tcgen05 kernel took them
    ops.prefill_tcgen05 = False
    ctx = context(ops, device, lengths_before, new, slots=slots, tables=[g.tables for g in mgr.groups], page_size=page_size)
    got = ops.paged_attention(torch.cat(q_rows).contiguous(), storage, ctx.block_tables[0], ctx, num_heads=heads,
                              num_kv_heads=kv_heads, head_dim=d, logit_softcap=0.0, window=window,
                              distance_bias=torch.stack([r1, r2]).contiguous(), **more).float().cpu().numpy()
    close(got, np.concatenate(want), dtype, "attention with the distance bias, mma.sync tiles", bf16=2e-2)
  if hasattr(ops, "check_errors"):
    ops.check_errors()


# ---- one-layer models: the stream after every layer call -------------------------------------------------

ONE_LAYER = {
    "biased attention alone": nx.config([nx.biased(window=9)], [None], width=32, vocab=40),
    "rotated attention alone": nx.config([nx.rotated(window=9)], [None], width=32, vocab=40),
    "dense feed-forward": nx.config([nx.biased(window=3)], [nx.dense(ff=40)], width=32, vocab=40),
    "routed experts": nx.config([nx.rotated(window=3, dims=16)], [nx.moe(experts=5, top=2, ff=12, shared=20)], width=32, vocab=40),
    "one layer walked four times": nx.config([nx.biased(window=6)], [nx.dense(ff=24)], width=32, vocab=40, loop=(0, 1, 4)),
    "a walk of one pass": nx.config([nx.rotated(window=6)], [nx.dense(ff=24)], width=32, vocab=40, loop=(0, 1, 1)),
}


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_one_layer_models_layer_by_layer(name, where):
  from tests.test_nulezen import engine_for
  cfg_dict = ONE_LAYER[name]
  engine, t = engine_for(cfg_dict, where, seed=17)
  toks = np.random.default_rng(3).integers(0, cfg_dict["vocab"], 29).tolist()
  want_layers = []
  want = plain.forward(cfg_dict, nx.as_numpy(t), toks, want_layers)
  for cuts in ([29], [12] + [1] * 17, nx.cuts_of(29, [2, 9, 3])):
    nx.check_close(nx.run_cuts(engine, toks, cuts), want, where[0], f"{name}, cuts {cuts[:3]}")
  slot = engine.open_request()
  ctx = engine._prepare([StepEntry(slot, toks, ())])
  ctx.memo["layer_outputs"] = got_layers = []
  engine.model.forward(ctx, engine.caches)
  engine.close_request(slot)
  assert len(got_layers) == len(want_layers)
  for i, (g, x) in enumerate(zip(got_layers, want_layers)):
    close(g.float().cpu().numpy(), x, torch.float32 if where[0] == "float32" else torch.bfloat16, f"{name}: stream after call {i}",
          f32=3e-5, bf16=3e-2)
