// Ragged paged attention, general form: any head size, page size, grouping and
// storage type.  One block of four warps per (token, query head); keys are visited in
// tiles of 32 that start at a multiple of 32 of the absolute key position, tile number i
// by warp i mod 4, and the warps' parts are merged in warp order, so a token's result is
// the same whatever else the step holds.
//
//   s = q . k                 (q is already rotated and scaled)
//   s = cap * tanh(s / cap)   if cap > 0          simply/model_lib.py:621-626
//   keep k_pos <= q_pos and, with a window W, q_pos - k_pos < W
//                                                 simply/model_lib.py:469-515
//   p = softmax(s) in float32, o = p . v          simply/model_lib.py:633-637
//   query head n reads kv head n / (Hq / Hkv)     simply/model_lib.py:2306-2310
//
// Options beyond that (`sb_paged_attention_general`): value heads of another size than key heads
// (a page then holds all its key rows, then all its value rows), and pooled blocks: with a
// window W and blocks of P tokens, position i also sees, ahead of its window and under the same
// softmax, one key and value per block c with c*P + P - 1 <= i - W, read from a second paged
// storage that holds one entry per P tokens in the page of the block's first token.  Blocks
// are visited in tiles of 32 by block number, before the tokens.  `tied`: an entry has one row of
// head_dim numbers whose first v_dim are its value as well (a cache of latents; a page then holds
// key rows only).  `sink`: one learned number per query head whose exponential joins the softmax's
// denominator; it has no key and no value.  `distance`: two learned numbers r1, r2 per query head
// ([2, heads]); the score of query i and key j loses r1 * log(1 + r2 * (i - j)) (float32, log1pf).
//
// This is the true 32-bit path's attention and the fallback of the bfloat16
// path for shapes its tensor-core kernels refuse.
#include <float.h>

#include "common.cuh"

#define GEN_WARPS 4
#define GEN_MAX_DPL 16  // dims per lane: head_dim <= 512

template <typename T> struct Vec16;  // 16-byte vector loads of storage type T
template <> struct Vec16<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float* out) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  }
};
template <> struct Vec16<bf16> {
  static constexpr int N = 8;
  __device__ static void load(const bf16* p, float* out) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      out[2 * i] = __uint_as_float(w[i] << 16);
      out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

// One tile of up to 32 keys, one per lane: scores, the running softmax, and the values' sum.
// `kr` / `vr` are this lane's key and value rows (null where the lane has no key).
template <typename KT>
__device__ __forceinline__ void gen_tile(const KT* kr, const KT* vr, const float* qs, int head_dim, int v_dim,
                                         float cap, float minus, int lane, float& m_run, float& l_run, float* acc) {
  constexpr int VN = Vec16<KT>::N;
  const float NEG = -0.5f * FLT_MAX;  // the reference's mask value, simply/utils/common.py:543-551
  const bool valid = kr != nullptr;
  float s = NEG;
  if (valid) {
    float dot = 0.f;
    int d = 0;
    if ((head_dim % VN) == 0) {
      for (; d < head_dim; d += VN) {
        float kf[VN];
        Vec16<KT>::load(kr + d, kf);
#pragma unroll
        for (int e = 0; e < VN; ++e) dot = fmaf(qs[d + e], kf[e], dot);
      }
    } else {
      for (; d < head_dim; ++d) dot = fmaf(qs[d], to_f32<KT>(kr[d]), dot);
    }
    s = (cap > 0.f ? cap * tanhf(dot / cap) : dot) - minus;
  }
  const float m_new = fmaxf(m_run, warp_max(s));
  const float alpha = expf(m_run - m_new);
  const float p = valid ? expf(s - m_new) : 0.f;
  l_run = l_run * alpha + warp_sum(p);
  m_run = m_new;
#pragma unroll
  for (int i = 0; i < GEN_MAX_DPL; ++i) acc[i] *= alpha;
  const unsigned valid_mask = __ballot_sync(0xffffffffu, valid);
  // Four keys at a time: their values are fetched together, then added in the keys' order (eight
  // at a time cost registers and were slower).
  constexpr int KEYS = 4;
  for (int j0 = 0; j0 < 32; j0 += KEYS) {
    const unsigned four = (valid_mask >> j0) & ((1u << KEYS) - 1u);  // uniform over the warp
    if (!four) continue;
    float pj[KEYS];
    const KT* vj[KEYS];
#pragma unroll
    for (int u = 0; u < KEYS; ++u) {
      pj[u] = __shfl_sync(0xffffffffu, p, j0 + u);
      vj[u] = reinterpret_cast<const KT*>(__shfl_sync(0xffffffffu, (unsigned long long)vr, j0 + u));
    }
#pragma unroll
    for (int i = 0; i < GEN_MAX_DPL; ++i) {
      const int d = lane + 32 * i;
      if (d < v_dim) {
        float x[KEYS];
#pragma unroll
        for (int u = 0; u < KEYS; ++u) x[u] = ((four >> u) & 1u) ? to_f32<KT>(vj[u][d]) : 0.f;
#pragma unroll
        for (int u = 0; u < KEYS; ++u)
          if ((four >> u) & 1u) acc[i] = fmaf(pj[u], x[u], acc[i]);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(GEN_WARPS * 32)
paged_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ cache,
                               const int* __restrict__ block_table, int max_pages,
                               const int* __restrict__ token_seq, const int* __restrict__ positions,
                               T* __restrict__ out, int num_tokens, int num_q_heads, int num_kv_heads,
                               int head_dim, int v_dim, int page_size, int num_pages, float cap, int window,
                               const T* __restrict__ pool, const int* __restrict__ pool_table,
                               int pool_max_pages, int pool_len, int pool_pages, int tied,
                               const float* __restrict__ sink, const float* __restrict__ distance, int* err) {
  const float r1 = distance != nullptr ? distance[blockIdx.x % num_q_heads] : 0.f;  // (weights: before the wait)
  const float r2 = distance != nullptr ? distance[num_q_heads + blockIdx.x % num_q_heads] : 0.f;
  pdl_wait_block();
  pdl_launch_dependents();
  // head_dim floats of q, then per warp its running maximum, sum and v_dim partial results
  extern __shared__ float smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long item = blockIdx.x;
  const int t = (int)(item / num_q_heads), n = (int)(item % num_q_heads);
  const int m = n / (num_q_heads / num_kv_heads);
  const int b = token_seq[t], pos = positions[t];
  float* qs = smem;
  float* part = smem + head_dim;
  const T* qp = q + ((size_t)t * num_q_heads + n) * head_dim;
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) qs[d] = to_f32<T>(qp[d]);
  __syncthreads();

  const int lo = window > 0 ? max(pos - window + 1, 0) : 0;
  float m_run = -0.5f * FLT_MAX, l_run = 0.f;
  float acc[GEN_MAX_DPL];
#pragma unroll
  for (int i = 0; i < GEN_MAX_DPL; ++i) acc[i] = 0.f;

  if (pool != nullptr && window > 0 && pool_len > 0) {
    // Blocks that lie wholly before the window: c * P + P - 1 <= pos - window.
    const int num_blocks = pos - window + 1 > 0 ? (pos - window + 1) / pool_len : 0;
    const int entries = (page_size + pool_len - 1) / pool_len;
    const size_t page_stride = (size_t)num_kv_heads * entries * (head_dim + v_dim);
    for (int tile = 32 * warp; tile < num_blocks; tile += 32 * GEN_WARPS) {  // tile i belongs to warp i % 4
      const int c = tile + lane;
      const T* kr = nullptr;
      const T* vr = nullptr;
      if (c < num_blocks) {
        const long long start = (long long)c * pool_len;
        const long long page = pool_table[(size_t)b * pool_max_pages + start / page_size];
        if (page < 0 || page >= pool_pages) {
          atomicOr(err, SB_ERR_BAD_PAGE);
        } else {
          const size_t row = (size_t)m * entries + (start % page_size) / pool_len;
          kr = pool + page * page_stride + row * head_dim;
          vr = pool + page * page_stride + (size_t)num_kv_heads * entries * head_dim + row * v_dim;
        }
      }
      gen_tile<T>(kr, vr, qs, head_dim, v_dim, cap, 0.f, lane, m_run, l_run, acc);
    }
  }

  const size_t page_stride = (size_t)num_kv_heads * page_size * (tied ? head_dim : head_dim + v_dim);
  const size_t value_base = (size_t)num_kv_heads * page_size * head_dim;
  for (int tile = (lo / 32) * 32; tile <= pos; tile += 32) {
    if (((tile >> 5) & (GEN_WARPS - 1)) != warp) continue;  // by the tile's absolute number
    const int j = tile + lane;
    const T* kr = nullptr;
    const T* vr = nullptr;
    if (j >= lo && j <= pos) {
      const long long page = block_table[(size_t)b * max_pages + j / page_size];
      if (page < 0 || page >= num_pages) {
        atomicOr(err, SB_ERR_BAD_PAGE);
      } else {
        const size_t row = (size_t)m * page_size + j % page_size;
        kr = cache + page * page_stride + row * head_dim;
        vr = tied ? kr : cache + page * page_stride + value_base + row * v_dim;
      }
    }
    const float minus = distance != nullptr && j <= pos ? r1 * log1pf(r2 * (float)(pos - j)) : 0.f;
    gen_tile<T>(kr, vr, qs, head_dim, v_dim, cap, minus, lane, m_run, l_run, acc);
  }
  // The warps' parts meet in warp order (the same order whatever the step holds).
  float* mine = part + (size_t)warp * (v_dim + 2);
  if (lane == 0) {
    mine[0] = m_run;
    mine[1] = l_run;
  }
#pragma unroll
  for (int i = 0; i < GEN_MAX_DPL; ++i) {
    const int d = lane + 32 * i;
    if (d < v_dim) mine[2 + d] = acc[i];
  }
  __syncthreads();
  if (warp != 0) return;
  float m_all = part[0];
#pragma unroll
  for (int w = 1; w < GEN_WARPS; ++w) m_all = fmaxf(m_all, part[(size_t)w * (v_dim + 2)]);
  if (sink != nullptr) m_all = fmaxf(m_all, sink[n]);
  float scale[GEN_WARPS], l_all = 0.f;
#pragma unroll
  for (int w = 0; w < GEN_WARPS; ++w) {
    scale[w] = expf(part[(size_t)w * (v_dim + 2)] - m_all);
    l_all += part[(size_t)w * (v_dim + 2) + 1] * scale[w];
  }
  if (sink != nullptr) l_all += expf(sink[n] - m_all);
  T* op = out + ((size_t)t * num_q_heads + n) * v_dim;
  const float inv = 1.0f / l_all;
  for (int d = lane; d < v_dim; d += 32) {
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < GEN_WARPS; ++w) sum += part[(size_t)w * (v_dim + 2) + 2 + d] * scale[w];
    op[d] = from_f32<T>(sum * inv);
  }
}

extern "C" int sb_paged_attention_general(const void* q, int dtype, const void* cache, const int* block_table,
                                          int max_pages, const int* token_seq, const int* positions,
                                          void* out, int num_tokens, int num_q_heads, int num_kv_heads,
                                          int head_dim, int v_dim, int page_size, int num_pages, float cap,
                                          int window, const void* pool, const int* pool_table,
                                          int pool_max_pages, int pool_len, int pool_pages, int tied,
                                          const float* sink, const float* distance, int* err,
                                          cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (distance != nullptr && pool != nullptr) return -13;
  if (tied && (pool != nullptr || v_dim > head_dim)) return -13;
  // (the values' sums live in registers, GEN_MAX_DPL per lane; a key row only passes through)
  if (head_dim <= 0 || head_dim > 4096 || v_dim <= 0 || v_dim > 32 * GEN_MAX_DPL) return -7;
  if (num_kv_heads <= 0 || num_q_heads % num_kv_heads) return -8;
  const long long items = (long long)num_tokens * num_q_heads;
  if (items > 0x7fffffffLL) return -6;
  const unsigned blocks = (unsigned)items;
  const size_t smem = ((size_t)head_dim + (size_t)GEN_WARPS * (v_dim + 2)) * sizeof(float);
  if (dtype == SB_DTYPE_F32)
    sb_launch(paged_attention_generic_kernel<float>, blocks, GEN_WARPS * 32, smem, stream, (const float*)q,
        (const float*)cache, block_table, max_pages, token_seq, positions, (float*)out, num_tokens,
        num_q_heads, num_kv_heads, head_dim, v_dim, page_size, num_pages, cap, window, (const float*)pool, pool_table,
        pool_max_pages, pool_len, pool_pages, tied, sink, distance, err);
  else
    sb_launch(paged_attention_generic_kernel<bf16>, blocks, GEN_WARPS * 32, smem, stream, (const bf16*)q,
        (const bf16*)cache, block_table, max_pages, token_seq, positions, (bf16*)out, num_tokens,
        num_q_heads, num_kv_heads, head_dim, v_dim, page_size, num_pages, cap, window, (const bf16*)pool, pool_table,
        pool_max_pages, pool_len, pool_pages, tied, sink, distance, err);
  SB_LAUNCH_CHECK();
  return 0;
}

extern "C" int sb_paged_attention_generic(const void* q, int dtype, const void* cache, const int* block_table,
                                          int max_pages, const int* token_seq, const int* positions,
                                          void* out, int num_tokens, int num_q_heads, int num_kv_heads,
                                          int head_dim, int page_size, int num_pages, float cap, int window,
                                          int* err, cudaStream_t stream) {
  return sb_paged_attention_general(q, dtype, cache, block_table, max_pages, token_seq, positions, out, num_tokens,
                                    num_q_heads, num_kv_heads, head_dim, head_dim, page_size, num_pages, cap,
                                    window, nullptr, nullptr, 0, 0, 0, 0, nullptr, nullptr, err, stream);
}
