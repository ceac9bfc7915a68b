// Attention over a paged cache of latents on tensor cores (bfloat16 in, float32 scores, softmax
// and sums), compiled once per shape: -DSB_LATENT_KD=N (numbers per cached row: the latent, then
// the rotated key part) and -DSB_LATENT_VD=M (the latent's size: a row's first M numbers are its
// value as well).
//
// All H query heads read the one cached row per token, so a block's rows are (token, head) pairs
// of one sequence in the order they lie in memory, BM at a time, whatever H is.  Per row at
// position i, over the keys j <= i (with a window W: i - j < W):
//
//   s_j = q . row_j                    (q is already scaled; its first M numbers ask the latent)
//   p   = exp(s_j - max) / (sum_j exp(s_j - max) + exp(sink_h - max))
//   o   = sum_j p_j row_j[:M]
//
// A block's warps are WM row groups of 16 rows x WN key groups that split every tile of BN keys
// x NS value groups that each own M / NS columns of the result (a row group's sums over 512
// columns do not fit one warp's registers; its NS warps each compute the scores themselves).
// The key groups' parts merge at the end in the groups' order.  The launch picks (WM, WN) by the
// longest portion of the step: single tokens take one row group and four key groups.
// Key tiles come through the block table with 16-byte cp.async copies, the next tile under way
// while this one is used; rows outside what a tile's rows can see are zero-filled, never read.
// Blocks find their tile by walking the step's sequences, so the launch needs no list from the
// host and a captured graph replays it as it is.
#include <cuda.h>
#include <float.h>

#include "common.cuh"

#ifndef SB_LATENT_KD
#define SB_LATENT_KD 576
#endif
#ifndef SB_LATENT_VD
#define SB_LATENT_VD 512
#endif

namespace {

constexpr int KD = SB_LATENT_KD, VD = SB_LATENT_VD;
constexpr int NS = (VD + 255) / 256;  // value groups
constexpr int VDS = VD / NS;          // columns of the result per warp
constexpr int PITCH = KD + 8;         // elements; the 16-byte pad spreads 8 consecutive rows over all banks
constexpr int CPR = KD / 8;           // 16-byte chunks per row
constexpr int BN_WIDE = KD > 256 ? 32 : 64;
constexpr float LOG2E = 1.4426950408889634f;

static_assert(KD % 16 == 0 && KD <= 768, "a cached row has a multiple of 16 numbers, at most 768");
static_assert(VD % (16 * NS) == 0 && VD <= KD && VD <= 512, "the latent is a multiple of 16, at most 512 and the row");

struct LatentParams {
  const bf16* q;      // [T, H, KD]
  const bf16* cache;  // [P, page, KD]
  const int* block_table;
  int max_pages;
  const int* cu_q;     // [B + 1]
  const int* q_start;  // [B]
  bf16* out;           // [T, H * VD]
  const float* sink;   // [H] or null
  int num_heads, page_size, num_pages, window, num_seqs;
  int* err;
  // With gridDim.y > 1 every tile's keys are split over that many blocks, which leave (max, sum) and
  // unnormalised sums per row for `latent_combine_kernel`: part_ml [rows, splits, 2], part_o [rows, splits, VD].
  float* part_ml;
  float* part_o;
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0: nothing is read, the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t r[4], const bf16* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t r[4], const bf16* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void mma16816(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// Scores of one warp's 16 query rows against NKT * 8 keys that start at row `key0` of the tile.
template <int NKT>
__device__ __forceinline__ void scores(float (&s)[NKT][4], const bf16* sq_rows, const bf16* sk, int key0) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int i = 0; i < NKT; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[i][e] = 0.f;
#pragma unroll 4
  for (int ks = 0; ks < KD / 16; ++ks) {
    uint32_t a[4];
    ldmatrix_x4(a, sq_rows + (lane & 15) * PITCH + ks * 16 + (lane >> 4) * 8);
#pragma unroll
    for (int np = 0; np < NKT / 2; ++np) {
      uint32_t r[4];
      ldmatrix_x4(r, sk + (key0 + np * 16 + (lane >> 4) * 8 + (lane & 7)) * PITCH + ks * 16 + ((lane >> 3) & 1) * 8);
      mma16816(s[2 * np], a, r[0], r[1]);
      mma16816(s[2 * np + 1], a, r[2], r[3]);
    }
  }
}

// Mask, online softmax update and P . V for one warp's columns [col0, col0 + VDS) of the values.
// `pos_a`, `pos_b`: positions of the thread's two query rows (-1 for a padding row).  `j0`:
// position of the first of the NKT * 8 keys.  m_* are kept in log2 units.
template <int NKT>
__device__ __forceinline__ void softmax_pv(float (&s)[NKT][4], float (&o)[VDS / 8][4], float& m_a, float& m_b,
                                           float& l_a, float& l_b, int pos_a, int pos_b, int j0, int window,
                                           const bf16* sk, int key0, int col0, bool need_mask) {
  const int lane = threadIdx.x & 31, t = lane & 3;
  float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
  for (int i = 0; i < NKT; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int j = j0 + i * 8 + 2 * t + (e & 1);
      const int pos = e < 2 ? pos_a : pos_b;
      const bool keep = !need_mask || (j <= pos && (window <= 0 || pos - j < window));
      const float v = keep ? s[i][e] * LOG2E : -INFINITY;
      s[i][e] = v;
      if (e < 2) mx_a = fmaxf(mx_a, v); else mx_b = fmaxf(mx_b, v);
    }
  mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
  mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
  mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
  mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
  const float new_a = fmaxf(m_a, mx_a), new_b = fmaxf(m_b, mx_b);
  const float use_a = new_a == -INFINITY ? 0.f : new_a, use_b = new_b == -INFINITY ? 0.f : new_b;
  const float alpha_a = fast_exp2(m_a - use_a), alpha_b = fast_exp2(m_b - use_b);
  m_a = new_a;
  m_b = new_b;
  float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
  for (int i = 0; i < NKT; ++i) {
    s[i][0] = fast_exp2(s[i][0] - use_a);
    s[i][1] = fast_exp2(s[i][1] - use_a);
    s[i][2] = fast_exp2(s[i][2] - use_b);
    s[i][3] = fast_exp2(s[i][3] - use_b);
    sum_a += s[i][0] + s[i][1];
    sum_b += s[i][2] + s[i][3];
  }
  l_a = l_a * alpha_a + sum_a;  // per-thread share of the row sum; the quad is added up at the end
  l_b = l_b * alpha_b + sum_b;
  if (__any_sync(0xffffffffu, alpha_a != 1.f || alpha_b != 1.f)) {  // the running maxima rarely move
#pragma unroll
    for (int d = 0; d < VDS / 8; ++d) {
      o[d][0] *= alpha_a;
      o[d][1] *= alpha_a;
      o[d][2] *= alpha_b;
      o[d][3] *= alpha_b;
    }
  }
#pragma unroll
  for (int kk = 0; kk < NKT / 2; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int dp = 0; dp < VDS / 16; ++dp) {
      uint32_t r[4];
      ldmatrix_x4_trans(r, sk + (key0 + kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * PITCH + col0 + dp * 16 + (lane >> 4) * 8);
      mma16816(o[2 * dp], a, r[0], r[1]);
      mma16816(o[2 * dp + 1], a, r[2], r[3]);
    }
  }
}

template <int WM, int WN, int BN>
__global__ void __launch_bounds__(WM * WN * NS * 32) latent_attention_kernel(const LatentParams p) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int BM = WM * 16, THREADS = WM * WN * NS * 32, KEYS = BN / WN, NKT = KEYS / 8;
  static_assert(NKT >= 2 && NKT % 2 == 0, "a key group takes whole steps of 16 keys");
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sq = reinterpret_cast<bf16*>(smem_raw);  // [BM][PITCH]
  bf16* sk = sq + BM * PITCH;                    // [2][BN][PITCH]
  __shared__ long long row_src[2][BN];
  __shared__ int s_item[2];
  const int H = p.num_heads;
  if (threadIdx.x == 0) {
    // tile number blockIdx.x of the step: sequences in order, BM rows of one sequence at a time
    int left = blockIdx.x, b = 0, r0 = -1;
    for (; b < p.num_seqs; ++b) {
      const int tiles = ((p.cu_q[b + 1] - p.cu_q[b]) * H + BM - 1) / BM;
      if (left < tiles) {
        r0 = left * BM;
        break;
      }
      left -= tiles;
    }
    s_item[0] = b;
    s_item[1] = r0;
  }
  __syncthreads();
  const int b = s_item[0], r0 = s_item[1];
  if (r0 < 0) return;  // the grid is an upper bound of the number of tiles
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int vs = warp / (WM * WN), wm = (warp % (WM * WN)) % WM, wn = (warp % (WM * WN)) / WM;
  const int row0 = p.cu_q[b], q_len = p.cu_q[b + 1] - row0, qs = p.q_start[b];
  const int rows_valid = min(BM, q_len * H - r0);
  const size_t first_row = (size_t)row0 * H + r0;  // of q and of the result

  for (int i = threadIdx.x; i < BM * CPR; i += THREADS) {
    const int row = i / CPR, c = i - row * CPR;
    const bool valid = row < rows_valid;
    cp_async16(sq + row * PITCH + c * 8, p.q + (first_row + (valid ? row : 0)) * KD + c * 8, valid);
  }
  const int p0 = qs + r0 / H, p1 = qs + (r0 + rows_valid - 1) / H;  // positions of the first and last row
  const int lo = p.window > 0 ? max(p0 - p.window + 1, 0) : 0;      // lowest key this tile can see
  const int kv_hi = p1 + 1;
  const int tile0 = (lo / BN) * BN;
  const int n_tiles = (kv_hi - tile0 + BN - 1) / BN;
  const int splits = gridDim.y, per_split = (n_tiles + splits - 1) / splits;
  const int it_lo = blockIdx.y * per_split, it_hi = min(n_tiles, it_lo + per_split);  // this block's tiles
  // Brings keys [tile0 + it BN, + BN) to shared memory: first where each row lives (one block-table
  // lookup per row), then 16 bytes per thread and turn.  Contains one __syncthreads.
  auto load_tile = [&](int it, int stage) {
    bf16* dst = sk + stage * BN * PITCH;
    for (int row = threadIdx.x; row < BN; row += THREADS) {
      const int j = tile0 + it * BN + row;
      long long src = -1;
      if (j >= lo && j < kv_hi) {
        const int page_index = j / p.page_size;
        const long long page = p.block_table[(size_t)b * p.max_pages + page_index];
        if (page < 0 || page >= p.num_pages)
          atomicOr(p.err, SB_ERR_BAD_PAGE);
        else
          src = (page * p.page_size + (j - page_index * p.page_size)) * (long long)KD;
      }
      row_src[stage][row] = src;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < BN * CPR; i += THREADS) {
      const int row = i / CPR, c = i - row * CPR;
      const long long src = row_src[stage][row];
      const bool valid = src >= 0;
      cp_async16(dst + row * PITCH + c * 8, p.cache + (valid ? src : 0) + c * 8, valid);
    }
  };
  if (it_lo < it_hi) load_tile(it_lo, 0);
  cp_async_commit();

  const int ra = wm * 16 + g, rb = ra + 8;
  const int pos_a = ra < rows_valid ? qs + (r0 + ra) / H : -1;
  const int pos_b = rb < rows_valid ? qs + (r0 + rb) / H : -1;
  // Positions of this warp's first and last row, for deciding whether a tile needs masking.
  const bool rows_full = wm * 16 + 15 < rows_valid;
  const int warp_pos_lo = qs + (r0 + wm * 16) / H, warp_pos_hi = qs + (r0 + wm * 16 + 15) / H;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  float o[VDS / 8][4];
#pragma unroll
  for (int d = 0; d < VDS / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

  for (int it = it_lo; it < it_hi; ++it) {
    const int stage = (it - it_lo) & 1;
    if (it + 1 < it_hi) {
      load_tile(it + 1, stage ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int j0 = tile0 + it * BN + wn * KEYS;  // this warp's first key of the tile
    // Every key visible to every row of the warp: none above the lowest row's position, all inside the
    // highest row's window.
    const bool need_mask = !rows_full || j0 + KEYS - 1 > warp_pos_lo || (p.window > 0 && warp_pos_hi - j0 >= p.window);
    float s[NKT][4];
    scores<NKT>(s, sq + wm * 16 * PITCH, sk + stage * BN * PITCH, wn * KEYS);
    softmax_pv<NKT>(s, o, m_a, m_b, l_a, l_b, pos_a, pos_b, j0, p.window, sk + stage * BN * PITCH, wn * KEYS,
                    vs * VDS, need_mask);
    __syncthreads();
  }
  cp_async_wait<0>();  // (a block without tiles of its own still has its query rows under way)
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  if (WN > 1) {
    // The key groups of a row group merge in their order: group 1, 2, ... hand (max, sum, result) to
    // group 0 through the shared memory that held the tiles.
    float* xm = reinterpret_cast<float*>(smem_raw);  // [NS][BM] max, [NS][BM] sum, then [NS][BM][VDS]
    float* xl = xm + NS * BM;
    float* xo = xl + NS * BM;
    const int xa = vs * BM + ra, xb = vs * BM + rb;
    for (int step = 1; step < WN; ++step) {
      if (wn == step) {
        if (t == 0) {
          xm[xa] = m_a; xm[xb] = m_b;
          xl[xa] = l_a; xl[xb] = l_b;
        }
#pragma unroll
        for (int d = 0; d < VDS / 8; ++d) {
          *reinterpret_cast<float2*>(xo + (size_t)xa * VDS + d * 8 + 2 * t) = make_float2(o[d][0], o[d][1]);
          *reinterpret_cast<float2*>(xo + (size_t)xb * VDS + d * 8 + 2 * t) = make_float2(o[d][2], o[d][3]);
        }
      }
      __syncthreads();
      if (wn == 0) {
        const float om_a = xm[xa], om_b = xm[xb];
        const float nm_a = fmaxf(m_a, om_a), nm_b = fmaxf(m_b, om_b);
        const float ua = nm_a == -INFINITY ? 0.f : nm_a, ub = nm_b == -INFINITY ? 0.f : nm_b;
        const float sa = fast_exp2(m_a - ua), sb = fast_exp2(m_b - ub);    // scale of this warp's part
        const float ta = fast_exp2(om_a - ua), tb = fast_exp2(om_b - ub);  // scale of the other's
        l_a = l_a * sa + xl[xa] * ta;
        l_b = l_b * sb + xl[xb] * tb;
        m_a = nm_a;
        m_b = nm_b;
#pragma unroll
        for (int d = 0; d < VDS / 8; ++d) {
          const float2 oa = *reinterpret_cast<const float2*>(xo + (size_t)xa * VDS + d * 8 + 2 * t);
          const float2 ob = *reinterpret_cast<const float2*>(xo + (size_t)xb * VDS + d * 8 + 2 * t);
          o[d][0] = o[d][0] * sa + oa.x * ta;
          o[d][1] = o[d][1] * sa + oa.y * ta;
          o[d][2] = o[d][2] * sb + ob.x * tb;
          o[d][3] = o[d][3] * sb + ob.y * tb;
        }
      }
      __syncthreads();
    }
    if (wn != 0) return;
  }
  if (splits > 1) {
    // this block's part of every row; the sink and the division wait for the combine
    if (ra < rows_valid) {
      const size_t at = (first_row + ra) * splits + blockIdx.y;
      if (t == 0 && vs == 0) { p.part_ml[2 * at] = m_a; p.part_ml[2 * at + 1] = l_a; }
#pragma unroll
      for (int d = 0; d < VDS / 8; ++d)
        *reinterpret_cast<float2*>(p.part_o + at * VD + vs * VDS + d * 8 + 2 * t) = make_float2(o[d][0], o[d][1]);
    }
    if (rb < rows_valid) {
      const size_t at = (first_row + rb) * splits + blockIdx.y;
      if (t == 0 && vs == 0) { p.part_ml[2 * at] = m_b; p.part_ml[2 * at + 1] = l_b; }
#pragma unroll
      for (int d = 0; d < VDS / 8; ++d)
        *reinterpret_cast<float2*>(p.part_o + at * VD + vs * VDS + d * 8 + 2 * t) = make_float2(o[d][2], o[d][3]);
    }
    return;
  }
  if (p.sink != nullptr) {
    // exp(sink_h) joins the sum; it has no value, so the result only shrinks
    const float ka = p.sink[(r0 + min(ra, rows_valid - 1)) % H] * LOG2E, kb = p.sink[(r0 + min(rb, rows_valid - 1)) % H] * LOG2E;
    const float na = fmaxf(m_a, ka), nb = fmaxf(m_b, kb);
    const float sa = fast_exp2(m_a - na), sb = fast_exp2(m_b - nb);
    l_a = l_a * sa + fast_exp2(ka - na);
    l_b = l_b * sb + fast_exp2(kb - nb);
#pragma unroll
    for (int d = 0; d < VDS / 8; ++d) {
      o[d][0] *= sa;
      o[d][1] *= sa;
      o[d][2] *= sb;
      o[d][3] *= sb;
    }
  }
  const float inv_a = l_a > 0.f ? 1.0f / l_a : 0.f, inv_b = l_b > 0.f ? 1.0f / l_b : 0.f;
  if (ra < rows_valid) {
    bf16* op = p.out + (first_row + ra) * VD + vs * VDS;
#pragma unroll
    for (int d = 0; d < VDS / 8; ++d)
      *reinterpret_cast<uint32_t*>(op + d * 8 + 2 * t) = pack_bf16(o[d][0] * inv_a, o[d][1] * inv_a);
  }
  if (rb < rows_valid) {
    bf16* op = p.out + (first_row + rb) * VD + vs * VDS;
#pragma unroll
    for (int d = 0; d < VDS / 8; ++d)
      *reinterpret_cast<uint32_t*>(op + d * 8 + 2 * t) = pack_bf16(o[d][2] * inv_b, o[d][3] * inv_b);
  }
}

// Merges the parts of a row's key splits in their order, adds the sink to the sum and divides.
constexpr int MAX_SPLITS = 16;
__global__ void __launch_bounds__(128) latent_combine_kernel(const float* __restrict__ part_ml,
                                                             const float* __restrict__ part_o, const float* __restrict__ sink,
                                                             bf16* __restrict__ out, int num_heads, int splits) {
  pdl_wait();
  pdl_launch_dependents();
  const size_t row = blockIdx.x;
  float m_all = sink != nullptr ? sink[row % num_heads] * LOG2E : -INFINITY;
  for (int s = 0; s < splits; ++s) m_all = fmaxf(m_all, part_ml[2 * (row * splits + s)]);
  float scale[MAX_SPLITS], l_all = sink != nullptr ? fast_exp2(sink[row % num_heads] * LOG2E - m_all) : 0.f;
#pragma unroll
  for (int s = 0; s < MAX_SPLITS; ++s) {
    scale[s] = 0.f;
    if (s < splits) {
      const float m = part_ml[2 * (row * splits + s)];
      scale[s] = m == -INFINITY ? 0.f : fast_exp2(m - m_all);
      l_all += part_ml[2 * (row * splits + s) + 1] * scale[s];
    }
  }
  const float inv = l_all > 0.f ? 1.0f / l_all : 0.f;
  for (int c = threadIdx.x; c < VD; c += blockDim.x) {
    float sum = 0.f;
#pragma unroll
    for (int s = 0; s < MAX_SPLITS; ++s)
      if (s < splits) sum = fmaf(part_o[(row * splits + s) * VD + c], scale[s], sum);
    out[row * VD + c] = __float2bfloat16(sum * inv);
  }
}

template <int WM, int WN, int BN>
int launch(const LatentParams& p, int num_tokens, int splits, cudaStream_t stream) {
  constexpr int BM = WM * 16;
  const size_t smem = (size_t)(BM + 2 * BN) * PITCH * sizeof(bf16);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(latent_attention_kernel<WM, WN, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const long long tiles = ((long long)num_tokens * p.num_heads + BM - 1) / BM + p.num_seqs;
  if (tiles > 0x7fffffffLL) return -6;
  sb_launch(latent_attention_kernel<WM, WN, BN>, dim3((unsigned)tiles, (unsigned)splits), WM * WN * NS * 32, smem, stream, p);
  SB_LAUNCH_CHECK();
  if (splits > 1) {
    sb_launch(latent_combine_kernel, dim3((unsigned)(num_tokens * p.num_heads)), 128, 0, stream, (const float*)p.part_ml,
              (const float*)p.part_o, p.sink, p.out, p.num_heads, splits);
    SB_LAUNCH_CHECK();
  }
  return 0;
}

}  // namespace

#define SB_CAT5_(a, b, c, d, e) a##b##c##d##e
#define SB_CAT5(a, b, c, d, e) SB_CAT5_(a, b, c, d, e)

// q [T, H, KD] scaled, cache [P, page, KD], out [T, H * VD]; `max_q_len`: the longest portion of the step.
// `splits` > 1 (steps of few rows per sequence only): every tile's keys over that many blocks, with
// part_ml [T H, splits, 2] and part_o [T H, splits, VD] float32 as their meeting place.
extern "C" int SB_CAT5(sb_latent_attention_k, SB_LATENT_KD, _v, SB_LATENT_VD, )(
    const void* q, const void* cache, const int* block_table, int max_pages, const int* cu_q, const int* q_start,
    void* out, const float* sink, int num_tokens, int num_seqs, int max_q_len, int num_heads, int page_size,
    int num_pages, int window, int splits, float* part_ml, float* part_o, int* err, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (num_heads <= 0 || num_seqs <= 0 || page_size <= 0 || splits < 1 || splits > MAX_SPLITS) return -8;
  if (splits > 1 && (part_ml == nullptr || part_o == nullptr)) return -8;
  LatentParams p{};
  p.q = (const bf16*)q; p.cache = (const bf16*)cache; p.block_table = block_table; p.max_pages = max_pages;
  p.cu_q = cu_q; p.q_start = q_start; p.out = (bf16*)out; p.sink = sink; p.num_heads = num_heads;
  p.page_size = page_size; p.num_pages = num_pages; p.window = window; p.num_seqs = num_seqs; p.err = err;
  p.part_ml = part_ml; p.part_o = part_o;
  const long long rows = (long long)max_q_len * num_heads;
  if (rows <= 16) return launch<1, 4, 64>(p, num_tokens, splits, stream);
  if (rows <= 32) return launch<2, 2, BN_WIDE>(p, num_tokens, splits, stream);
  return launch<4, 1, BN_WIDE>(p, num_tokens, splits, stream);
}
