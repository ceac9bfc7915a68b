// What stands around attention with normed queries and keys: the norm over whole projections,
// rotations of keys, queries and values, the stores into the paged cache, the pooled blocks'
// means, and the turn back of a head's result.  Float32 arithmetic; T is the storage type.
//
//   x     = x / sqrt(mean_row x^2 + eps) * w                 over all heads of q (of k) at once
//   (a, b)= (a cos - b sin, b cos + a sin)                   pair (i, i + n/2), angle = pos * freq[i]
//   q    *= head_scale[head]
// A page of the cache holds all its key rows [kv head, entry, head_dim], then all its value
// rows [kv head, entry, value_dim].
#include "common.cuh"

// ---------------------------------------------------------------------------
// One block per token.  qkv row: q (H d) | k (G d) | v (G dv); G = 0: a layer without keys and
// values of its own.  rot_freq [rot_dims / 2] (null: no rotation), value_freq [dv / 2] (null:
// values are stored as they are).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
qk_norm_rotate_store_kernel(const T* __restrict__ qkv, int row_width, const float* __restrict__ q_norm,
                            const float* __restrict__ k_norm, float eps, const float* __restrict__ head_scale,
                            const float* __restrict__ rot_freq, int rot_dims, const float* __restrict__ value_freq,
                            T* __restrict__ q_out, T* __restrict__ cache, const int* __restrict__ block_table,
                            int max_pages, const int* __restrict__ token_seq, const int* __restrict__ positions,
                            int H, int G, int d, int dv, int page_size, int num_pages, int write_cache, int* err) {
  pdl_wait_block();
  pdl_launch_dependents();
  extern __shared__ float row[];  // (H + G) d floats, 33 scratch, cos and sin of rot_dims / 2 and of dv / 2 angles
  const int nq = H * d, nk = G * d;
  float* scratch = row + nq + nk;
  const int half = rot_dims / 2, vhalf = dv / 2;
  float* cs_qk = scratch + 33;    // [half] cos, [half] sin
  float* cs_v = cs_qk + 2 * half;  // [vhalf] cos, [vhalf] sin
  const int t = blockIdx.x;
  const T* x = qkv + (size_t)t * row_width;
  const float pos = (float)positions[t];
  // A token's angles are the same for all its heads: once per block.
  if (rot_freq != nullptr)
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * rot_freq[i], cs_qk + half + i, cs_qk + i);
  if (value_freq != nullptr && write_cache && nk > 0)
    for (int i = threadIdx.x; i < vhalf; i += blockDim.x) sincosf(pos * value_freq[i], cs_v + vhalf + i, cs_v + i);

  constexpr int N = Vec<T>::N;
  const bool vec = d % N == 0 && row_width % N == 0;  // whole 16-byte groups inside a head
  float ssq = 0.f, ssk = 0.f;
  if (vec) {
    for (int i = threadIdx.x * N; i < nq + nk; i += blockDim.x * N) {
      float v[N];
      Vec<T>::load(x + i, v);
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < N; ++e) {
        row[i + e] = v[e];
        ss = fmaf(v[e], v[e], ss);
      }
      if (i < nq) ssq += ss; else ssk += ss;
    }
  } else {
    for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) {
      const float v = to_f32<T>(x[i]);
      row[i] = v;
      if (i < nq) ssq = fmaf(v, v, ssq); else ssk = fmaf(v, v, ssk);
    }
  }
  ssq = block_sum(ssq, scratch);
  const float rq = 1.0f / sqrtf(ssq / (float)nq + eps);
  float rk = 0.f;
  if (nk > 0) {
    ssk = block_sum(ssk, scratch);
    rk = 1.0f / sqrtf(ssk / (float)nk + eps);
  }
  for (int i = threadIdx.x; i < nq + nk; i += blockDim.x)
    row[i] = i < nq ? row[i] * rq * q_norm[i] : row[i] * rk * k_norm[i - nq];
  __syncthreads();

  long long page = -1;
  int off = 0;
  if (write_cache && nk > 0) {
    const int p = positions[t];
    page = block_table[(size_t)token_seq[t] * max_pages + p / page_size];
    off = p % page_size;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(err, SB_ERR_BAD_PAGE);
      page = -1;
    }
  }
  const size_t page_stride = (size_t)G * page_size * (d + dv);
  if (vec) {
    for (int i0 = threadIdx.x * N; i0 < nq + nk; i0 += blockDim.x * N) {
      const int head = i0 / d, c0 = i0 - head * d;
      const float scale = i0 < nq ? head_scale[head] : 1.f;
      float o[N];
#pragma unroll
      for (int e = 0; e < N; ++e) {
        const int c = c0 + e;
        float v = row[i0 + e];
        if (rot_freq != nullptr && c < rot_dims) {
          const int pair = c < half ? c : c - half;
          const float cs = cs_qk[pair], sn = cs_qk[half + pair];
          const float a = row[i0 - c0 + pair], b = row[i0 - c0 + pair + half];
          v = c < half ? a * cs - b * sn : b * cs + a * sn;
        }
        o[e] = v * scale;
      }
      if (i0 < nq)
        Vec<T>::store(q_out + (size_t)t * nq + i0, o);
      else if (page >= 0)
        Vec<T>::store(cache + page * page_stride + ((size_t)(head - H) * page_size + off) * d + c0, o);
    }
  }
  for (int i = threadIdx.x; i < (vec ? 0 : nq + nk); i += blockDim.x) {
    const int head = i / d, c = i % d;
    float v = row[i];
    if (rot_freq != nullptr && c < rot_dims) {
      const int pair = c < half ? c : c - half;
      const float cs = cs_qk[pair], sn = cs_qk[half + pair];
      const float a = row[i - c + pair], b = row[i - c + pair + half];
      v = c < half ? a * cs - b * sn : b * cs + a * sn;
    }
    if (i < nq) {
      q_out[(size_t)t * nq + i] = from_f32<T>(v * head_scale[head]);
    } else if (page >= 0) {
      const int m = head - H;
      cache[page * page_stride + ((size_t)m * page_size + off) * d + c] = from_f32<T>(v);
    }
  }
  if (page >= 0) {
    const T* vx = x + nq + nk;
    T* dst = cache + page * page_stride + (size_t)G * page_size * d;
    const bool vec_v = vec && dv % N == 0 && (value_freq == nullptr || vhalf % N == 0) && (nq + nk) % N == 0;
    if (vec_v) {
      for (int i0 = threadIdx.x * N; i0 < G * dv; i0 += blockDim.x * N) {
        const int m = i0 / dv, c0 = i0 - m * dv;
        float own[N], other[N], o[N];
        Vec<T>::load(vx + i0, own);
        if (value_freq != nullptr) {
          Vec<T>::load(vx + (c0 < vhalf ? i0 + vhalf : i0 - vhalf), other);
#pragma unroll
          for (int e = 0; e < N; ++e) {
            const int pair = c0 < vhalf ? c0 + e : c0 + e - vhalf;
            const float cs = cs_v[pair], sn = cs_v[vhalf + pair];
            o[e] = c0 < vhalf ? own[e] * cs - other[e] * sn : own[e] * cs + other[e] * sn;
          }
        } else {
#pragma unroll
          for (int e = 0; e < N; ++e) o[e] = own[e];
        }
        Vec<T>::store(dst + ((size_t)m * page_size + off) * dv + c0, o);
      }
    }
    for (int i = threadIdx.x; i < (vec_v ? 0 : G * dv); i += blockDim.x) {
      const int m = i / dv, c = i % dv;
      float v = to_f32<T>(vx[i]);
      if (value_freq != nullptr) {
        const int pair = c < vhalf ? c : c - vhalf;
        const float cs = cs_v[pair], sn = cs_v[vhalf + pair];
        const float a = to_f32<T>(vx[i - c + pair]), b = to_f32<T>(vx[i - c + pair + vhalf]);
        v = c < vhalf ? a * cs - b * sn : b * cs + a * sn;
      }
      dst[((size_t)m * page_size + off) * dv + c] = from_f32<T>(v);
    }
  }
}

extern "C" int sb_qk_norm_rotate_store(const void* qkv, int row_width, int dtype, const float* q_norm,
                                       const float* k_norm, float eps, const float* head_scale,
                                       const float* rot_freq, int rot_dims, const float* value_freq, void* q_out,
                                       void* cache, const int* block_table, int max_pages, const int* token_seq,
                                       const int* positions, int num_tokens, int H, int G, int d, int dv,
                                       int page_size, int num_pages, int write_cache, int* err,
                                       cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  const size_t smem = ((size_t)(H + G) * d + 33 + rot_dims + dv) * sizeof(float);
  if (smem > 200 * 1024) return -2;
  if (rot_dims % 2 || rot_dims > d || (value_freq != nullptr && dv % 2)) return -4;
  if (dtype == SB_DTYPE_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(qk_norm_rotate_store_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb_launch(qk_norm_rotate_store_kernel<float>, num_tokens, 256, smem, stream, (const float*)qkv, row_width,
              q_norm, k_norm, eps, head_scale, rot_freq, rot_dims, value_freq, (float*)q_out, (float*)cache,
              block_table, max_pages, token_seq, positions, H, G, d, dv, page_size, num_pages, write_cache, err);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(qk_norm_rotate_store_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb_launch(qk_norm_rotate_store_kernel<bf16>, num_tokens, 256, smem, stream, (const bf16*)qkv, row_width,
              q_norm, k_norm, eps, head_scale, rot_freq, rot_dims, value_freq, (bf16*)q_out, (bf16*)cache,
              block_table, max_pages, token_seq, positions, H, G, d, dv, page_size, num_pages, write_cache, err);
  }
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// Pooled blocks: for every block of P tokens whose last token arrived in this step, the mean of
// its keys and of its values as the cache holds them, summed in float32 in the tokens' order,
// into the storage of block entries.  Grid (block within the step, sequence, kv head).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(1024)
pool_blocks_kernel(const T* __restrict__ cache, const int* __restrict__ block_table, int max_pages, int num_pages,
                   T* __restrict__ pool, const int* __restrict__ pool_table, int pool_max_pages,
                   int pool_pages, const int* __restrict__ cu_q, const int* __restrict__ q_start, int G, int d,
                   int dv, int page_size, int P, int* err) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int b = blockIdx.y, m = blockIdx.z;
  const int start = q_start[b], end = start + cu_q[b + 1] - cu_q[b];
  const int c = start / P + blockIdx.x;
  if (c >= end / P) return;
  const int first = c * P;
  const int entries = (page_size + P - 1) / P;
  const long long to = pool_table[(size_t)b * pool_max_pages + first / page_size];
  if (to < 0 || to >= pool_pages) {
    if (threadIdx.x == 0) atomicOr(err, SB_ERR_BAD_PAGE);
    return;
  }
  const size_t page_stride = (size_t)G * page_size * (d + dv);
  const size_t pool_stride = (size_t)G * entries * (d + dv);
  const size_t entry = (size_t)m * entries + (first % page_size) / P;
  // Where the block's tokens live: worked out once per 64 tokens, by the first threads.
  __shared__ long long where[64];  // the token's page times the page's size; -1: not held
  __shared__ int row_in_page[64];
  float sums[4] = {0.f, 0.f, 0.f, 0.f};  // this thread's channels: threadIdx.x, + 128, ...
  bool ok = true;
  for (int j0 = 0; j0 < P; j0 += 64) {
    const int count = min(64, P - j0);
    __syncthreads();
    if ((int)threadIdx.x < count) {
      const int p = first + j0 + threadIdx.x;
      const long long page = block_table[(size_t)b * max_pages + p / page_size];
      where[threadIdx.x] = (page < 0 || page >= num_pages) ? -1 : page * (long long)page_stride;
      row_in_page[threadIdx.x] = p % page_size;
    }
    __syncthreads();
#pragma unroll
    for (int turn = 0; turn < 4; ++turn) {
      const int ch = turn * blockDim.x + threadIdx.x;
      if (ch >= d + dv) break;
      const bool is_key = ch < d;
      const int cc = is_key ? ch : ch - d, width = is_key ? d : dv;
      const size_t base = (is_key ? 0 : (size_t)G * page_size * d) + (size_t)m * page_size * width + cc;
      float sum = sums[turn];
      for (int j = 0; j < count; j += 8) {  // eight tokens' loads together, added in the tokens' order
        float x[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          x[u] = 0.f;
          if (j + u < count) {
            const long long at = where[j + u];
            if (at < 0) ok = false;
            else x[u] = to_f32<T>(cache[at + base + (size_t)row_in_page[j + u] * width]);
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (j + u < count) sum += x[u];
      }
      sums[turn] = sum;
    }
  }
  if (!ok) atomicOr(err, SB_ERR_BAD_PAGE);
#pragma unroll
  for (int turn = 0; turn < 4; ++turn) {
    const int ch = turn * blockDim.x + threadIdx.x;
    if (ch >= d + dv || !ok) break;
    const bool is_key = ch < d;
    const int cc = is_key ? ch : ch - d, width = is_key ? d : dv;
    T* dst = pool + to * pool_stride + (is_key ? 0 : (size_t)G * entries * d) + entry * width + cc;
    *dst = from_f32<T>(sums[turn] / (float)P);
  }
}

extern "C" int sb_pool_blocks(const void* cache, int dtype, const int* block_table, int max_pages, int num_pages,
                              void* pool, const int* pool_table, int pool_max_pages, int pool_pages,
                              const int* cu_q, const int* q_start, int num_seqs, int max_blocks, int G, int d,
                              int dv, int page_size, int P, int* err, cudaStream_t stream) {
  if (num_seqs == 0 || max_blocks <= 0) return 0;
  if (P <= 0) return -13;
  const dim3 grid(max_blocks, num_seqs, G);
  // a thread keeps up to four channels' sums: wider heads get wider blocks
  int threads = 128;
  while (threads * 4 < d + dv && threads < 1024) threads *= 2;
  if (threads * 4 < d + dv) return -13;
  if (dtype == SB_DTYPE_F32)
    sb_launch(pool_blocks_kernel<float>, grid, threads, 0, stream, (const float*)cache, block_table, max_pages,
              num_pages, (float*)pool, pool_table, pool_max_pages, pool_pages, cu_q, q_start, G, d, dv, page_size, P, err);
  else
    sb_launch(pool_blocks_kernel<bf16>, grid, threads, 0, stream, (const bf16*)cache, block_table, max_pages,
              num_pages, (bf16*)pool, pool_table, pool_max_pages, pool_pages, cu_q, q_start, G, d, dv, page_size, P, err);
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// Turns every head of x [T, H, n] by its token's position: pair (i, i + n/2) by
// sign * pos * freq[i].  One block per token.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
rotate_heads_kernel(const T* __restrict__ x, const int* __restrict__ positions, const float* __restrict__ freq,
                    float sign, int H, int n, T* __restrict__ out) {
  pdl_wait_block();
  pdl_launch_dependents();
  extern __shared__ float cs[];  // [n / 2] cos, [n / 2] sin: a token's angles are the same for all its heads
  const int t = blockIdx.x, half = n / 2;
  const float pos = sign * (float)positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * freq[i], cs + half + i, cs + i);
  __syncthreads();
  constexpr int N = Vec<T>::N;
  if (half % N == 0) {
    for (int i0 = threadIdx.x * N; i0 < H * half; i0 += blockDim.x * N) {
      const int h = i0 / half, pair = i0 - h * half;
      const size_t at = ((size_t)t * H + h) * n + pair;
      float a[N], b[N], lo[N], hi[N];
      Vec<T>::load(x + at, a);
      Vec<T>::load(x + at + half, b);
#pragma unroll
      for (int e = 0; e < N; ++e) {
        const float c = cs[pair + e], s = cs[half + pair + e];
        lo[e] = a[e] * c - b[e] * s;
        hi[e] = b[e] * c + a[e] * s;
      }
      Vec<T>::store(out + at, lo);
      Vec<T>::store(out + at + half, hi);
    }
    return;
  }
  for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
    const int h = i / half, pair = i % half;
    const size_t at = ((size_t)t * H + h) * n + pair;
    const float c = cs[pair], s = cs[half + pair];
    const float a = to_f32<T>(x[at]), b = to_f32<T>(x[at + half]);
    out[at] = from_f32<T>(a * c - b * s);
    out[at + half] = from_f32<T>(b * c + a * s);
  }
}

extern "C" int sb_rotate_heads(const void* x, int dtype, const int* positions, const float* freq, float sign,
                               int num_tokens, int H, int n, void* out, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (n % 2) return -4;
  if (dtype == SB_DTYPE_F32)
    sb_launch(rotate_heads_kernel<float>, num_tokens, 256, (size_t)n * sizeof(float), stream, (const float*)x, positions, freq, sign, H, n,
              (float*)out);
  else
    sb_launch(rotate_heads_kernel<bf16>, num_tokens, 256, (size_t)n * sizeof(float), stream, (const bf16*)x, positions, freq, sign, H, n,
              (bf16*)out);
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// Attention whose heads are normed one by one after rotation.  One block per token, a warp per
// head.  Row of `proj`: q (H d) | k (G d) | [v (G dv)] | whatever follows (a gate, which this
// kernel does not read).
//   (a, b) = (a cos - b sin, b cos + a sin)     neighbours (2i, 2i + 1) for `interleaved`, else
//                                               (i, i + rot_dims/2); angle = pos * rot_freq[i]
//   x      = x / sqrt(mean_head x^2 + eps)      (no scale; `head_norm` = 0 skips it)
//   q     *= q_scale
// Keys go to the cache rotated and normed.  Values: with `tie_values` a key head as the projection
// left it (before rotation and norm) is also the value head; otherwise the v columns as they are.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
rotate_headnorm_store_kernel(const T* __restrict__ proj, int row_width, const float* __restrict__ bias, float eps, float q_scale,
                             const float* __restrict__ rot_freq, int rot_dims, int interleaved, int head_norm,
                             int tie_values, T* __restrict__ q_out, T* __restrict__ cache,
                             const int* __restrict__ block_table, int max_pages, const int* __restrict__ token_seq,
                             const int* __restrict__ positions, int H, int G, int d, int dv, int page_size,
                             int num_pages, int write_cache, int* err) {
  pdl_wait_block();
  pdl_launch_dependents();
  extern __shared__ float row[];  // (H + G) d floats, then cos and sin of rot_dims / 2 angles
  const int nq = H * d, nk = G * d, half = rot_dims / 2;
  float* cs = row + nq + nk;
  const int t = blockIdx.x;
  const T* x = proj + (size_t)t * row_width;
  const float pos = (float)positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * rot_freq[i], cs + half + i, cs + i);
  // `bias`: a learned offset on q, k and (untied) v, added in float32 before anything else
  for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) row[i] = to_f32<T>(x[i]) + (bias != nullptr ? bias[i] : 0.f);
  __syncthreads();

  long long page = -1;
  int off = 0;
  if (write_cache && nk > 0) {
    const int p = positions[t];
    page = block_table[(size_t)token_seq[t] * max_pages + p / page_size];
    off = p % page_size;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(err, SB_ERR_BAD_PAGE);
      page = -1;
    }
  }
  const size_t page_stride = (size_t)G * page_size * (d + dv);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int head = warp; head < H + G; head += nwarps) {
    float* v = row + (size_t)head * d;
    const bool is_q = head < H;
    T* value_dst = nullptr;
    T* key_dst = nullptr;
    if (!is_q && page >= 0) {
      key_dst = cache + page * page_stride + ((size_t)(head - H) * page_size + off) * d;
      value_dst = cache + page * page_stride + (size_t)G * page_size * d + ((size_t)(head - H) * page_size + off) * dv;
      if (tie_values)  // the head as projected, before this warp turns it
        for (int c = lane; c < d; c += 32) value_dst[c] = from_f32<T>(v[c]);
    }
    __syncwarp();
    for (int i = lane; i < half; i += 32) {
      const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
      const float a = v[ia], b = v[ib], c = cs[i], sn = cs[half + i];
      v[ia] = a * c - b * sn;
      v[ib] = b * c + a * sn;
    }
    __syncwarp();
    float scale = is_q ? q_scale : 1.0f;
    if (head_norm) {
      float ss = 0.f;
      for (int c = lane; c < d; c += 32) ss = fmaf(v[c], v[c], ss);
      ss = warp_sum(ss);
      scale *= 1.0f / sqrtf(ss / (float)d + eps);
    }
    if (is_q) {
      T* dst = q_out + (size_t)t * nq + (size_t)head * d;
      for (int c = lane; c < d; c += 32) dst[c] = from_f32<T>(v[c] * scale);
    } else if (key_dst != nullptr) {
      for (int c = lane; c < d; c += 32) key_dst[c] = from_f32<T>(v[c] * scale);
    }
  }
  if (!tie_values && page >= 0) {
    const T* vx = x + nq + nk;
    T* dst = cache + page * page_stride + (size_t)G * page_size * d;
    for (int i = threadIdx.x; i < G * dv; i += blockDim.x) {
      const int m = i / dv, c = i - m * dv;
      dst[((size_t)m * page_size + off) * dv + c] =
          bias != nullptr ? from_f32<T>(to_f32<T>(vx[i]) + bias[nq + nk + i]) : vx[i];
    }
  }
}

extern "C" int sb_rotate_headnorm_store(const void* proj, int row_width, int dtype, const float* bias, float eps, float q_scale,
                                        const float* rot_freq, int rot_dims, int interleaved, int head_norm,
                                        int tie_values, void* q_out, void* cache, const int* block_table,
                                        int max_pages, const int* token_seq, const int* positions, int num_tokens,
                                        int H, int G, int d, int dv, int page_size, int num_pages, int write_cache,
                                        int* err, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (rot_freq == nullptr) rot_dims = 0;
  const size_t smem = ((size_t)(H + G) * d + rot_dims) * sizeof(float);
  if (smem > 200 * 1024) return -2;
  if (rot_dims % 2 || rot_dims > d || (tie_values && dv != d)) return -4;
  if (dtype == SB_DTYPE_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(rotate_headnorm_store_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb_launch(rotate_headnorm_store_kernel<float>, num_tokens, 256, smem, stream, (const float*)proj, row_width, bias, eps,
              q_scale, rot_freq, rot_dims, interleaved, head_norm, tie_values, (float*)q_out, (float*)cache,
              block_table, max_pages, token_seq, positions, H, G, d, dv, page_size, num_pages, write_cache, err);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(rotate_headnorm_store_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb_launch(rotate_headnorm_store_kernel<bf16>, num_tokens, 256, smem, stream, (const bf16*)proj, row_width, bias, eps,
              q_scale, rot_freq, rot_dims, interleaved, head_norm, tie_values, (bf16*)q_out, (bf16*)cache,
              block_table, max_pages, token_seq, positions, H, G, d, dv, page_size, num_pages, write_cache, err);
  }
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// Output gate: x[t, c] *= sigmoid(gate[t, c]), the gate read from a wider row (a column range of
// the fused projection).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(T* __restrict__ x, const T* __restrict__ gate, int gate_width, int width, int per) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int t = blockIdx.y;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < width; c += gridDim.x * blockDim.x) {
    const float g = to_f32<T>(gate[(size_t)t * gate_width + c / per]);  // one gate per `per` neighbours
    const size_t at = (size_t)t * width + c;
    x[at] = from_f32<T>(to_f32<T>(x[at]) / (1.0f + expf(-g)));
  }
}

extern "C" int sb_sigmoid_gate(void* x, const void* gate, int gate_width, int dtype, int num_tokens, int width,
                               int per, cudaStream_t stream) {
  if (num_tokens == 0 || width == 0) return 0;
  if (per < 1) return -13;
  for (int t0 = 0; t0 < num_tokens; t0 += 65535) {
    const dim3 grid((unsigned)min((width + 255) / 256, 64), (unsigned)min(65535, num_tokens - t0));
    if (dtype == SB_DTYPE_F32)
      sb_launch(sigmoid_gate_kernel<float>, grid, 256, 0, stream, (float*)x + (size_t)t0 * width,
                (const float*)gate + (size_t)t0 * gate_width, gate_width, width, per);
    else
      sb_launch(sigmoid_gate_kernel<bf16>, grid, 256, 0, stream, (bf16*)x + (size_t)t0 * width,
                (const bf16*)gate + (size_t)t0 * gate_width, gate_width, width, per);
  }
  SB_LAUNCH_CHECK();
  return 0;
}
