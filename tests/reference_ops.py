"""Plain PyTorch statement of every kernel of the engine's kernel table.

Two uses.  The GPU tests call one CUDA kernel and the function of the same
name here on the same inputs.  The CPU tests hand an instance to the engine in
place of the CUDA table, so that the cache manager, the step function, the
scheduler and replay can be checked against the plain NumPy model on a machine
without a GPU.  Nothing in the package imports this file.

Every function computes in float32 (float64 where noted) from inputs of the
activation dtype and rounds once at the end, as the kernels do.
"""

from __future__ import annotations

import math

import numpy as np
import torch

from tests.plain import gemma2_plain as plain


class ReferenceOps:

  def __init__(self, dtype: torch.dtype = torch.float32):
    self.dtype = dtype
    self.name = "reference"

  # ---- checks ---------------------------------------------------------------
  def check_attention(self, head_dim, num_heads, num_kv_heads):
    pass

  # ---- dense ----------------------------------------------------------------
  def linear(self, x, w):
    return (x.float() @ w.float().t()).to(self.dtype)

  def gated_linear(self, x, w_gate_up, activation, limit=0.0):
    return self.gated_activation(self.linear(x, w_gate_up), activation, limit)

  def cast(self, x, dtype):
    return x.to(dtype)

  def check_errors(self):
    pass

  def embed(self, table, ids, scale, positions=None, position_table=None, round_scale=True):
    s = torch.tensor(scale, dtype=torch.float32)
    if table.dtype == torch.bfloat16 and round_scale:
      s = s.to(torch.bfloat16).float()
    out = table[ids.long()].float() * s
    if position_table is not None:
      out = out + position_table[positions.long()].float()
    return out

  def lm_head(self, x, table, cap, scale=1.0):
    logits = (x.float() @ table.float().t()) * scale
    if cap > 0:
      logits = cap * torch.tanh(logits / cap)
    return logits

  def gated_activation(self, gate_up, activation, limit=0.0):
    f = gate_up.shape[1] // 2
    g, u = gate_up[:, :f].float(), gate_up[:, f:].float()
    if activation == 3:
      g, u = torch.clamp(g, max=limit), torch.clamp(u, -limit, limit)
      return (g * torch.sigmoid(1.702 * g) * (u + 1.0)).to(self.dtype)
    if activation == 0:
      a = 0.5 * g * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (g + 0.044715 * g ** 3)))
    elif activation == 1:
      a = g * torch.sigmoid(g)
    elif activation == 2:
      a = torch.relu(g)
    else:
      raise ValueError(f"unknown activation code {activation}")
    return (a * u).to(self.dtype)

  # ---- norms ----------------------------------------------------------------
  @staticmethod
  def _rms(x, w, eps, plus_one):
    x = x.float()
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return y * (w.float() + 1.0 if plus_one else w.float())

  def rms_norm(self, x, w, eps, plus_one):
    return self._rms(x, w, eps, plus_one).to(self.dtype)

  def residual_norm(self, h, branch, post, pre, rows, branch2=None):
    if rows is not None:
      idx = rows.long()
      h = h[idx].clone()
      branch = branch[idx] if branch is not None else None
      branch2 = branch2[idx] if branch2 is not None else None
    if branch is not None:
      b = self._rms(branch, post.weight, post.eps, post.plus_one) if post is not None else branch.float()
      h += b
    if branch2 is not None:
      h += branch2.float()
    if pre is None:
      return None
    return self._rms(h, pre.weight, pre.eps, pre.plus_one).to(self.dtype)

  def scaled_residual_tanh(self, h, branch, scale, branch2, scale2, pre, rows):
    """h += scale * branch + scale2 * branch2 (float32, in place unless `rows` picks some);
    returns tanh(alpha h) w + b for the norm `pre`, or None without one."""
    if rows is not None:
      idx = rows.long()
      h = h[idx].float().clone()
      branch = branch[idx] if branch is not None else None
      branch2 = branch2[idx] if branch2 is not None else None
    elif h.dtype != torch.float32:
      h = h.float()
    add = None
    for b, s in ((branch, scale), (branch2, scale2)):
      if b is not None:
        term = b.float() * (s.float() if s is not None else 1.0)
        add = term if add is None else add + term
    if add is not None:
      h += add
    if pre is None:
      return None
    return (torch.tanh(pre.alpha.float() * h) * pre.weight.float() + pre.bias.float()).to(self.dtype)

  def scale_channels(self, x, w):
    return (x.float() * w.float()).to(self.dtype)

  def pack_pair(self, a, b):
    return torch.cat([a, b], dim=1).to(self.dtype)

  def linear_wide(self, x, w, row=None):
    out = x.float() @ w.float().t()
    return out + row.float() if row is not None else out

  def linear_xielu(self, x, w, act, factors=None):
    z = self.linear(x, w).float()
    ap = torch.nn.functional.softplus(act[0].float())
    an = 0.5 + torch.nn.functional.softplus(act[1].float())
    zn = torch.clamp(z, max=0.0)
    return torch.where(z > 0, ap * z * z + 0.5 * z, an * (torch.expm1(zn) - zn) + 0.5 * z).to(self.dtype)

  def gather_rows(self, x, rows):
    return x[rows.long()].clone()

  def add_to_residual(self, h, x):
    h += x.float()

  # ---- positions ------------------------------------------------------------
  def rotation_tables(self, positions, timescale, scale_factor):
    angle = positions.float()[:, None] / timescale[None, :] / np.float32(scale_factor)
    return torch.cos(angle), torch.sin(angle)

  def project_rotate_store(self, x, w_qkv, tables, q_scale, num_heads, num_kv_heads, head_dim, storage,
                           block_table, ctx):
    return self.rope_and_cache_write(self.linear(x, w_qkv), tables, q_scale, num_heads, num_kv_heads, head_dim,
                                     storage, block_table, ctx)

  def rope_and_cache_write(self, qkv, tables, q_scale, num_heads, num_kv_heads, head_dim, storage,
                           block_table, ctx):
    t = qkv.shape[0]
    nq = num_heads * head_dim
    nk = num_kv_heads * head_dim
    q = qkv[:, :nq].float().reshape(t, num_heads, head_dim)

    def rotate(x):
      if tables is None:
        return x
      cos, sin = tables[0][:, None, :], tables[1][:, None, :]
      half = head_dim // 2
      a, b = x[..., :half], x[..., half:]
      return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)

    q = (rotate(q) * np.float32(q_scale)).to(self.dtype)
    if storage is not None:
      k = rotate(qkv[:, nq:nq + nk].float().reshape(t, num_kv_heads, head_dim)).to(storage.dtype)
      v = qkv[:, nq + nk:nq + 2 * nk].reshape(t, num_kv_heads, head_dim).to(storage.dtype)
      pos = ctx.positions.long()
      page = block_table[ctx.token_seq.long(), pos // ctx.page_size].long()
      assert (page >= 0).all(), "a token would be written to a page its request does not hold"
      off = pos % ctx.page_size
      storage[page, 0, :, off, :] = k
      storage[page, 1, :, off, :] = v
    return q

  # ---- attention ------------------------------------------------------------
  def paged_attention(self, q, storage, block_table, ctx, *, num_heads, num_kv_heads, head_dim,
                      logit_softcap, window, value_dim=None, pooled=None, values_in_keys=False, sink=None,
                      distance_bias=None):
    if (pooled is not None or (value_dim is not None and value_dim != head_dim) or values_in_keys or sink is not None
        or distance_bias is not None):
      assert not logit_softcap
      return self._general_attention(q, storage, block_table, ctx, num_heads, num_kv_heads, head_dim,
                                     value_dim or head_dim, window, pooled, values_in_keys, sink, distance_bias)
    t = q.shape[0]
    out = torch.zeros(t, num_heads, head_dim, dtype=torch.float32, device=q.device)
    group = num_heads // num_kv_heads
    cu_q = ctx.host["cu_q"]
    q_start = ctx.host["q_start"]
    ps = ctx.page_size
    for b in range(ctx.num_seqs):
      r0, r1 = int(cu_q[b]), int(cu_q[b + 1])
      kv_len = int(q_start[b]) + (r1 - r0)
      q_pos = torch.arange(int(q_start[b]), kv_len, device=q.device)
      lo = 0 if window is None else max(int(q_start[b]) - window + 1, 0)
      k_pos = torch.arange(lo, kv_len, device=q.device)
      page = block_table[b, (k_pos // ps)].long()
      assert (page >= 0).all(), "attention would read a page the request does not hold"
      kv = storage[page, :, :, k_pos % ps, :].float()  # [Tk, 2, Hkv, dh]
      mask = k_pos[None, :] <= q_pos[:, None]
      if window is not None:
        mask &= (q_pos[:, None] - k_pos[None, :]) < window
      for n in range(num_heads):
        m = n // group
        s = q[r0:r1, n, :].float() @ kv[:, 0, m, :].t()
        if logit_softcap > 0:
          s = logit_softcap * torch.tanh(s / logit_softcap)
        s = torch.where(mask, s, torch.tensor(-0.5 * torch.finfo(torch.float32).max, device=q.device))
        p = torch.softmax(s, dim=-1)
        out[r0:r1, n, :] = p @ kv[:, 1, m, :]
    return out.reshape(t, num_heads * head_dim).to(self.dtype)

  # ---- attention with normed queries and keys, pooled blocks ------------------
  @staticmethod
  def _kv_views(storage, num_kv_heads, entries, head_dim, value_dim):
    """Keys [pages, G, entries, d] and values [pages, G, entries, dv] of a cache's storage."""
    flat = storage.view(storage.shape[0], -1)
    nk = num_kv_heads * entries * head_dim
    return (flat[:, :nk].view(-1, num_kv_heads, entries, head_dim),
            flat[:, nk:].view(-1, num_kv_heads, entries, value_dim))

  @staticmethod
  def _turn(x, angle):
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c, s = torch.cos(angle), torch.sin(angle)
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)

  def qk_norm_rotate_store(self, qkv, q_norm, k_norm, eps, head_scale, rot_freq, value_freq, num_heads,
                           num_kv_heads, head_dim, value_dim, storage, block_table, ctx):
    t = qkv.shape[0]
    nq, nk = num_heads * head_dim, num_kv_heads * head_dim
    pos = ctx.positions.float()

    def normed(x, w, heads):
      x = x.float()
      x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.float()
      x = x.reshape(t, heads, head_dim)
      if rot_freq is not None:
        dims = 2 * rot_freq.numel()
        angle = (pos[:, None] * rot_freq[None, :])[:, None, :]
        x = torch.cat([self._turn(x[..., :dims], angle), x[..., dims:]], dim=-1)
      return x

    q = (normed(qkv[:, :nq], q_norm, num_heads) * head_scale.float()[None, :, None]).to(self.dtype)
    if storage is not None and num_kv_heads:
      k = normed(qkv[:, nq:nq + nk], k_norm, num_kv_heads)
      v = qkv[:, nq + nk:nq + nk + num_kv_heads * value_dim].float().reshape(t, num_kv_heads, value_dim)
      if value_freq is not None:
        v = self._turn(v, (pos[:, None] * value_freq[None, :])[:, None, :])
      keys, values = self._kv_views(storage, num_kv_heads, ctx.page_size, head_dim, value_dim)
      p = ctx.positions.long()
      page = block_table[ctx.token_seq.long(), p // ctx.page_size].long()
      assert (page >= 0).all(), "a token would be written to a page its request does not hold"
      keys[page, :, p % ctx.page_size, :] = k.to(storage.dtype)
      values[page, :, p % ctx.page_size, :] = v.to(storage.dtype)
    return q

  def pool_blocks(self, storage, block_table, pool_storage, pool_table, ctx, num_kv_heads, head_dim, value_dim, pool):
    ps = ctx.page_size
    keys, values = self._kv_views(storage, num_kv_heads, ps, head_dim, value_dim)
    pk, pv = self._kv_views(pool_storage, num_kv_heads, -(-ps // pool), head_dim, value_dim)
    for b in range(ctx.num_seqs):
      start = int(ctx.host["q_start"][b])
      end = start + int(ctx.host["cu_q"][b + 1] - ctx.host["cu_q"][b])
      for c in range(start // pool, end // pool):
        j = torch.arange(c * pool, (c + 1) * pool, device=storage.device)
        page = block_table[b, j // ps].long()
        assert (page >= 0).all(), "a block would be pooled from a page its request does not hold"
        to = int(pool_table[b, (c * pool) // ps])
        assert to >= 0
        e = ((c * pool) % ps) // pool
        pk[to, :, e, :] = keys[page, :, j % ps, :].float().sum(0) / pool
        pv[to, :, e, :] = values[page, :, j % ps, :].float().sum(0) / pool

  def rotate_heads(self, x, positions, freq, num_heads, dim, inverse=False):
    t = x.shape[0]
    angle = (positions.float()[:, None] * freq[None, :])[:, None, :]
    y = self._turn(x.float().reshape(t, num_heads, dim), -angle if inverse else angle)
    return y.reshape(t, num_heads * dim).to(self.dtype)

  def _general_attention(self, q, storage, block_table, ctx, num_heads, num_kv_heads, head_dim, value_dim,
                         window, pooled, values_in_keys=False, sink=None, distance_bias=None):
    t = q.shape[0]
    ps = ctx.page_size
    if values_in_keys:  # one row per entry: the key, whose first value_dim numbers are the value
      keys = storage.view(storage.shape[0], num_kv_heads, ps, head_dim)
      values = keys[..., :value_dim]
    else:
      keys, values = self._kv_views(storage, num_kv_heads, ps, head_dim, value_dim)
    group = num_heads // num_kv_heads
    out = torch.zeros(t, num_heads, value_dim, dtype=torch.float32, device=q.device)
    q = q.reshape(t, num_heads, head_dim)
    for b in range(ctx.num_seqs):
      r0, r1 = int(ctx.host["cu_q"][b]), int(ctx.host["cu_q"][b + 1])
      start = int(ctx.host["q_start"][b])
      for r in range(r0, r1):
        i = start + r - r0
        lo = 0 if window is None else max(i - window + 1, 0)
        j = torch.arange(lo, i + 1, device=q.device)
        page = block_table[b, j // ps].long()
        assert (page >= 0).all(), "attention would read a page the request does not hold"
        k = keys[page, :, j % ps, :].float()
        v = values[page, :, j % ps, :].float()
        if pooled is not None:
          pool_storage, pool_table, pool = pooled
          pk, pv = self._kv_views(pool_storage, num_kv_heads, -(-ps // pool), head_dim, value_dim)
          nb = max((i - window + 1) // pool, 0)
          if nb:
            c = torch.arange(nb, device=q.device)
            pg = pool_table[b, (c * pool) // ps].long()
            assert (pg >= 0).all()
            e = ((c * pool) % ps) // pool
            k = torch.cat([pk[pg, :, e, :].float(), k], dim=0)
            v = torch.cat([pv[pg, :, e, :].float(), v], dim=0)
        for n in range(num_heads):
          m = n // group
          scores = k[:, m] @ q[r, n].float()
          if distance_bias is not None:  # [2, heads]: the score loses r1 log(1 + r2 distance)
            assert pooled is None
            scores = scores - distance_bias[0, n] * torch.log1p(distance_bias[1, n] * (i - j).float())
          if sink is None:
            p = torch.softmax(scores, dim=0)
          else:  # the denominator also holds exp(sink[n]), which has no value
            p = torch.softmax(torch.cat([scores, sink[n].float().reshape(1)]), dim=0)[:-1]
          out[r, n] = p @ v[:, m]
    return out.reshape(t, num_heads * value_dim).to(self.dtype)

  # ---- gated delta rule -------------------------------------------------------

  # ---- attention with heads normed one by one -----------------------------------
  def rotate_headnorm_store(self, proj, eps, q_scale, rot_freq, *, interleaved, head_norm, tie_values, num_heads,
                            num_kv_heads, head_dim, storage, block_table, ctx, value_dim=None, bias=None):
    t = proj.shape[0]
    value_dim = head_dim if value_dim is None else value_dim
    nq, nk, nv = num_heads * head_dim, num_kv_heads * head_dim, (0 if tie_values else num_kv_heads * value_dim)
    cols = proj[:, :nq + nk + nv].float()
    if bias is not None:  # on q, k and v, before anything else
      cols = cols + bias.float()
    q = cols[:, :nq].reshape(t, num_heads, head_dim)
    k_raw = cols[:, nq:nq + nk].reshape(t, num_kv_heads, head_dim)
    v = k_raw if tie_values else cols[:, nq + nk:].reshape(t, num_kv_heads, value_dim)

    def prepare(x):
      x = x.clone()
      if rot_freq is not None:
        dims = 2 * rot_freq.numel()
        angle = ctx.positions.float()[:, None, None] * rot_freq.float()[None, None, :]
        c, s = torch.cos(angle), torch.sin(angle)
        ia = torch.arange(0, dims, 2) if interleaved else torch.arange(0, dims // 2)
        ib = ia + 1 if interleaved else ia + dims // 2
        a, b = x[..., ia], x[..., ib]
        x[..., ia], x[..., ib] = a * c - b * s, b * c + a * s
      if head_norm:
        x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
      return x

    if storage is not None:
      ps = ctx.page_size
      pos = ctx.positions.long()
      page = block_table[ctx.token_seq.long(), pos // ps].long()
      assert (page >= 0).all(), "a token would be written to a page the request does not hold"
      keys, values = self._kv_views(storage, num_kv_heads, ps, head_dim, value_dim)
      keys[page, :, pos % ps, :] = prepare(k_raw).to(storage.dtype)
      values[page, :, pos % ps, :] = v.to(storage.dtype)
    return (prepare(q) * q_scale).to(self.dtype)

  def sigmoid_gate(self, x, proj, offset, per=1):
    gate = torch.sigmoid(proj[:, offset:offset + x.shape[1] // per].float())
    return (x.float() * gate.repeat_interleave(per, dim=1)).to(self.dtype)

  # ---- forget-gate recurrence -----------------------------------------------------
  def forget_gate_scan(self, pre, bias, lower, state, ctx, *, num_heads, head_dim, value_dim):
    t = pre.shape[0]
    n = num_heads * head_dim
    pq = pre[:, :n].float()
    q = (pq * torch.sigmoid(pq)).reshape(t, num_heads, head_dim)
    f = (lower + (1.0 - lower) * torch.sigmoid(pre[:, n:2 * n].float() + bias)).reshape(t, num_heads, head_dim)
    v = pre[:, 2 * n:2 * n + num_heads * value_dim].float().reshape(t, num_heads, value_dim)
    out = torch.empty(t, num_heads, value_dim, dtype=torch.float32, device=pre.device)
    for b in range(ctx.num_seqs):
      r0, r1 = int(ctx.host["cu_q"][b]), int(ctx.host["cu_q"][b + 1])
      slot = int(ctx.host["slots"][b])
      s = state[slot].clone()
      for r in range(r0, r1):
        s = f[r][:, :, None] * s + (1.0 - f[r])[:, :, None] * v[r][:, None, :]
        out[r] = torch.einsum("hdv,hd->hv", s, q[r])
      state[slot] = s
    return out

  # ---- routed experts ---------------------------------------------------------------
  def route_tokens(self, x, router, correction, shared_gate_w, *, top, scale, score=0, renormalize=False, bias=None):
    z = x.float() @ router.float().t()
    if bias is not None:
      z = z + bias.float()
    s = torch.softmax(z, dim=-1) if score == 0 else torch.sigmoid(z)
    choice = s + (correction.float() if correction is not None else 0.0)
    chosen = torch.argsort(-choice, dim=-1, stable=True)[:, :top]
    weight = torch.gather(s, 1, chosen)
    weight = weight / weight.sum(-1, keepdim=True) * scale if renormalize else weight * scale
    gate = torch.sigmoid(x.float() @ shared_gate_w.float()) if shared_gate_w is not None else None
    return chosen.to(torch.int32), weight, gate

  @staticmethod
  def _activation(g, activation):
    if activation == 4:
      return 0.5 * g * (1.0 + torch.erf(g / math.sqrt(2.0)))
    if activation == 0:
      return 0.5 * g * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (g + 0.044715 * g ** 3)))
    return g * torch.sigmoid(g) if activation == 1 else torch.relu(g)

  def route_by_table(self, token_ids, table, num_experts):
    chosen = table[token_ids.long()].to(torch.int32)
    return chosen, torch.full(chosen.shape, 1.0 / chosen.shape[1], dtype=torch.float32, device=chosen.device)

  def mix_experts(self, x, chosen, weight, gate_up, down, num_experts, activation, shared, shared_gate, gated=True,
                  limit=0.0):
    xf = x.float()
    out = torch.zeros_like(xf)
    for t in range(x.shape[0]):
      for j in range(chosen.shape[1]):
        e = int(chosen[t, j])
        if e < num_experts and not gated:
          h = self._activation(xf[t:t + 1] @ gate_up[e].float().t(), activation).to(self.dtype)
          y = (h.float() @ down[e].float().t()).to(self.dtype).float()[0]
        elif e < num_experts:
          h = self.gated_activation((xf[t:t + 1] @ gate_up[e].float().t()).to(self.dtype), activation, limit)
          y = (h.float() @ down[e].float().t()).to(self.dtype).float()[0]
        else:
          y = xf[t]
        out[t] += weight[t, j] * y
    if shared is not None:
      out += shared.float() * (shared_gate[:, None] if shared_gate is not None else 1.0)
    return out.to(self.dtype)

  def delta_rule_inputs(self, pre, low, conv_weight, conv_state, decay_bias, neg_rate, ctx, *, conv_taps,
                        num_heads, num_kv_heads, head_dim, value_dim):
    t = pre.shape[0]
    qk, vv = num_kv_heads * head_dim, num_heads * value_dim
    c = 2 * qk + vv
    x = pre[:, :c].float()
    y = torch.empty_like(x)
    for b in range(ctx.num_seqs):
      r0, r1 = int(ctx.host["cu_q"][b]), int(ctx.host["cu_q"][b + 1])
      slot = int(ctx.host["slots"][b])
      seen = torch.cat([conv_state[slot].float(), x[r0:r1]], dim=0)  # [taps - 1 + n, C]
      n = r1 - r0
      y[r0:r1] = sum(seen[j:j + n] * conv_weight[:, j][None, :] for j in range(conv_taps))
      if conv_taps > 1:
        conv_state[slot] = seen[-(conv_taps - 1):]
    y = y * torch.sigmoid(y)

    def unit(z):
      return z / torch.sqrt(z.pow(2).sum(-1, keepdim=True) + 1e-6)

    q = unit(y[:, :qk].reshape(t, num_kv_heads, head_dim)) * head_dim ** -0.5
    k = unit(y[:, qk:2 * qk].reshape(t, num_kv_heads, head_dim))
    v = y[:, 2 * qk:c].reshape(t, num_heads, value_dim)
    beta = torch.sigmoid(pre[:, c:c + num_heads].float())
    a = low[:, :num_heads * head_dim].float() + decay_bias[None, :]
    decay = torch.exp(neg_rate[None, :, None] * torch.nn.functional.softplus(a).reshape(t, num_heads, head_dim))
    return q.contiguous(), k.contiguous(), v.contiguous(), decay.contiguous(), beta.contiguous()

  def gated_delta_scan(self, q, k, v, decay, beta, state, ctx, *, num_heads, num_kv_heads, head_dim, value_dim):
    out = torch.empty(q.shape[0], num_heads, value_dim, dtype=torch.float32, device=q.device)
    rep = num_heads // num_kv_heads
    for b in range(ctx.num_seqs):
      r0, r1 = int(ctx.host["cu_q"][b]), int(ctx.host["cu_q"][b + 1])
      slot = int(ctx.host["slots"][b])
      for n in range(num_heads):
        s = state[slot, n].clone()
        for r in range(r0, r1):
          s = decay[r, n][:, None] * s
          u = beta[r, n] * (v[r, n] - s.t() @ k[r, n // rep])
          s = s + torch.outer(k[r, n // rep], u)
          out[r, n] = s.t() @ q[r, n // rep]
        state[slot, n] = s
    return out

  def gated_head_norm(self, o, low, gate_offset, weight, eps, num_heads, value_dim):
    t = o.shape[0]
    y = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * weight.float()[None, None, :]
    if low is None:
      return y.reshape(t, num_heads * value_dim).to(self.dtype)
    gate = torch.sigmoid(low[:, gate_offset:gate_offset + num_heads * value_dim].float())
    return (y.reshape(t, num_heads * value_dim) * gate).to(self.dtype)

  def normed_mean(self, branches, scales, eps):
    total = 0
    for x, w in zip(branches, scales):
      total = total + self._rms(x, w, eps, False)
    return (total / len(branches)).to(self.dtype)

  # ---- a stream kept several times ---------------------------------------------------
  def spread_streams(self, h, copies):
    return h[:, None, :].repeat(1, copies, 1).contiguous()

  def streams_step(self, lanes, branch, mix, out, weights, norm_weight, eps, plus_one, rows):
    """lanes [T, S, W] float32.  With `branch`: lanes[:, t] <- sum_s mix[s, t] lanes[:, s] + out[t] *
    branch (in place; with `rows` only those rows are computed and nothing is written).  With
    `weights`: returns rms(sum_s weights[s] lanes[:, s]) * norm_weight in the activation dtype
    (`norm_weight` None: the sum itself, float32)."""
    x = lanes if rows is None else lanes[rows.long()]
    if branch is not None:
      y = branch.float() if rows is None else branch[rows.long()].float()
      x = torch.einsum("sr,tsw->trw", mix.float(), x) + out.float()[None, :, None] * y[:, None, :]
      if rows is None:
        lanes.copy_(x)
    if weights is None:
      return None
    u = torch.einsum("s,tsw->tw", weights.float(), x)
    if norm_weight is None:
      return u
    return self._rms(u, norm_weight, eps, plus_one).to(self.dtype)

  # ---- short convolutions with their state ------------------------------------------------
  def short_conv(self, x, weight, bias, state, ctx, *, activation=0, residual=False, offset=0, channels=None,
                 out_dtype=None):
    """Causal convolution over time per channel on x[:, offset : offset + channels]: y_t = sum_j
    weight[:, j] * x_(t - K + 1 + j) (+ bias), the K - 1 inputs before a step's first token read from
    `state` [slots, K - 1, channels] (float32), which then takes the step's last inputs.  activation 1:
    silu.  residual: x + y."""
    channels = x.shape[1] - offset if channels is None else channels
    xs = x[:, offset:offset + channels].float()
    taps = weight.shape[1]
    y = torch.empty_like(xs)
    for b in range(ctx.num_seqs):
      r0, r1 = int(ctx.host["cu_q"][b]), int(ctx.host["cu_q"][b + 1])
      n = r1 - r0
      if taps > 1:
        slot = int(ctx.host["slots"][b])
        seen = torch.cat([state[slot].float(), xs[r0:r1]], dim=0)
        state[slot] = seen[-(taps - 1):]
      else:
        seen = xs[r0:r1]
      y[r0:r1] = sum(seen[j:j + n] * weight[:, j].float()[None, :] for j in range(taps))
    if bias is not None:
      y = y + bias.float()[None, :]
    if activation == 1:
      y = y * torch.sigmoid(y)
    if residual:
      y = xs + y
    return y.to(out_dtype or self.dtype)

  # ---- attention over latents -----------------------------------------------------------
  @staticmethod
  def _turn_part(x, positions, freq):
    """Dims i and i + n of the first 2n dims of x [T, ..., D] turn by positions * freq[i]."""
    if freq is None:
      return x
    n = freq.numel()
    angle = positions.float()[:, None] * freq.float()[None, :]
    while angle.dim() < x.dim():
      angle = angle[:, None]
    c, s = torch.cos(angle), torch.sin(angle)
    a, b = x[..., :n], x[..., n:2 * n]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., 2 * n:]], dim=-1)

  def latent_prepare(self, down, query_norm, kv_norm, eps, freq, *, query_rank, kv_rank, rotated_dim, storage,
                     block_table, ctx):
    d = down.float()
    cq = self._rms(d[:, :query_rank], query_norm, eps, False)
    c = self._rms(d[:, query_rank:query_rank + kv_rank], kv_norm, eps, False)
    kr = self._turn_part(d[:, query_rank + kv_rank:query_rank + kv_rank + rotated_dim], ctx.positions, freq)
    if storage is not None:
      ps = ctx.page_size
      pos = ctx.positions.long()
      page = block_table[ctx.token_seq.long(), pos // ps].long()
      assert (page >= 0).all(), "a token would be written to a page the request does not hold"
      rows = storage.view(storage.shape[0], ps, kv_rank + rotated_dim)
      rows[page, pos % ps] = torch.cat([c, kr], dim=1).to(storage.dtype)
    return cq.to(self.dtype)

  def latent_queries(self, q, key_up_t, freq, scale, ctx, *, num_heads, head_dim, rotated_dim):
    t = q.shape[0]
    qh = q.float().reshape(t, num_heads, head_dim + rotated_dim)
    plain = torch.einsum("thd,hrd->thr", qh[..., :head_dim], key_up_t.float())
    turned = self._turn_part(qh[..., head_dim:], ctx.positions, freq)
    return (torch.cat([plain, turned], dim=-1) * scale).reshape(t, -1).to(self.dtype)

  def head_linear(self, x, w):
    """x [T, H * Din] . w [H, Dout, Din]^T per head -> [T, H * Dout]."""
    h, dout, din = w.shape
    y = torch.einsum("thd,hod->tho", x.float().reshape(x.shape[0], h, din), w.float())
    return y.reshape(x.shape[0], h * dout).to(self.dtype)

  # ---- the generalized delta rule ---------------------------------------------------------
  def tanh_columns(self, x, offset, n):
    return torch.tanh(x[:, offset:offset + n].float()).to(self.dtype)

  def general_delta_scan(self, pre, low, decay_bias, removal_bias, state, ctx, *, num_heads, head_dim):
    t = pre.shape[0]
    inner = num_heads * head_dim
    shape = (t, num_heads, head_dim)
    r, k, v = (pre[:, i * inner:(i + 1) * inner].float().reshape(shape) for i in range(3))
    take = torch.sigmoid(pre[:, 4 * inner:5 * inner].float() + removal_bias).reshape(shape)
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(low[:, :inner].float() + decay_bias)).reshape(shape)
    unit = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    out = torch.empty(shape, dtype=torch.float32, device=pre.device)
    for b in range(ctx.num_seqs):
      r0, r1 = int(ctx.host["cu_q"][b]), int(ctx.host["cu_q"][b + 1])
      slot = int(ctx.host["slots"][b])
      s = state[slot].clone()  # [H, dk, dv]
      for i in range(r0, r1):
        seen = torch.einsum("hk,hkv->hv", unit[i], s)
        s = (decay[i][:, :, None] * s - (take[i] * unit[i])[:, :, None] * seen[:, None, :]
             + k[i][:, :, None] * v[i][:, None, :])
        out[i] = torch.einsum("hkv,hk->hv", s, r[i])
      state[slot] = s
    return out

  def group_norm_gate(self, o, weight, eps, *, groups, gate=None, gate_offset=0, gate_kind="none"):
    """o float32 [T, ...] of N numbers per token, RMS-normed in `groups` equal parts, times weight [N];
    the gate gate[:, gate_offset : gate_offset + N] acts as silu before the norm or as sigmoid after it."""
    t = o.shape[0]
    y = o.reshape(t, -1).float()
    n = y.shape[1]
    g = gate[:, gate_offset:gate_offset + n].float() if gate is not None and gate_kind != "none" else None
    if gate_kind == "silu_before":
      y = y * g * torch.sigmoid(g)
    y = y.reshape(t, groups, n // groups)
    y = (y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps)).reshape(t, n) * weight.float()[None, :]
    if gate_kind == "sigmoid_after":
      y = y * torch.sigmoid(g)
    return y.to(self.dtype)

  # ---- the state-space recurrence ---------------------------------------------------------
  def state_space_scan(self, xbc, pre, step_offset, step_bias, neg_rate, skip, state, ctx, *, num_heads, value_dim,
                       state_dim, num_groups):
    t = xbc.shape[0]
    inner, gn = num_heads * value_dim, num_groups * state_dim
    x = xbc[:, :inner].float().reshape(t, num_heads, value_dim)
    per = num_heads // num_groups
    bm = xbc[:, inner:inner + gn].float().reshape(t, num_groups, state_dim).repeat_interleave(per, dim=1)
    cm = xbc[:, inner + gn:inner + 2 * gn].float().reshape(t, num_groups, state_dim).repeat_interleave(per, dim=1)
    dt = torch.nn.functional.softplus(pre[:, step_offset:step_offset + num_heads].float() + step_bias[None, :],
                                      threshold=1e9)
    decay = torch.exp(neg_rate[None, :] * dt)
    out = torch.empty(t, num_heads, value_dim, dtype=torch.float32, device=xbc.device)
    for b in range(ctx.num_seqs):
      r0, r1 = int(ctx.host["cu_q"][b]), int(ctx.host["cu_q"][b + 1])
      slot = int(ctx.host["slots"][b])
      s = state[slot].clone()  # [H, N, dv]
      for i in range(r0, r1):
        s = decay[i][:, None, None] * s + (dt[i][:, None] * bm[i])[:, :, None] * x[i][:, None, :]
        out[i] = torch.einsum("hnv,hn->hv", s, cm[i]) + skip[:, None] * x[i]
      state[slot] = s
    return out

  # ---- sampling -------------------------------------------------------------
  def token_logprobs(self, logits, tokens, temperature, top_k, top_p):
    rows = [logits[i].float().cpu().numpy() for i in range(logits.shape[0])]
    lp = [plain.token_logprob(rows[i], int(tokens[i]), float(temperature), int(top_k), float(top_p))
          for i in range(len(rows))]
    return torch.tensor(lp, dtype=torch.float32, device=logits.device)

  def sample(self, logits, temperature, top_k, top_p, seed, position, logprobs=False):
    """logits f32 [R, V]; the other arguments are host sequences of length R."""
    rows = [logits[i].float().cpu().numpy() for i in range(logits.shape[0])]
    out = [
        plain.sample_token(rows[i], float(temperature[i]), int(top_k[i]), float(top_p[i]), int(seed[i]),
                           int(position[i]))
        for i in range(logits.shape[0])
    ]
    tokens = torch.tensor(out, dtype=torch.int32, device=logits.device)
    if not logprobs:
      return tokens
    lp = [plain.token_logprob(rows[i], out[i], float(temperature[i]), int(top_k[i]), float(top_p[i]))
          for i in range(logits.shape[0])]
    return tokens, torch.tensor(lp, dtype=torch.float32, device=logits.device)
