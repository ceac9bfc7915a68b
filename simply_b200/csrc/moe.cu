// Feed-forward layers made of routed experts.  Five kernels, none of which needs the host to
// know how the tokens were dealt out, so a step can be captured in a CUDA graph:
//
//   route    per token: router logits z = W_r x (+ a learned offset per expert) (float32), scores
//            s = softmax(z) (or sigmoid),
//            the `top` experts with the largest s + correction, weights s * scale (optionally
//            divided by their sum), and the shared expert's gate sigmoid(w_sg . x)
//   group    the (token, choice) pairs sorted by expert, cut into tiles of TILE_M rows of one
//            expert each; experts with index >= E ("identity" experts) take no rows
//   product  out[r, :] = A[row(r), :] . W[expert of r's tile]^T over those tiles, once with two
//            sets of weight rows and act(gate) * up on the sums, once plain
//   combine  y[t] = sum_j weight[t, j] * (expert output of pair (t, j), or x[t] for an identity
//            expert) + gate[t] * shared[t], summed in the order of j
//
// bfloat16 products run on tensor cores (mma.sync through nvcuda::wmma) with float32 sums; the
// float32 path uses CUDA cores only.  A row's result does not depend on which rows share its tile.
#include <mma.h>

#include "common.cuh"

#define MOE_TILE_M 64   // rows of a tile
#define MOE_TILE_N 32   // output columns of one set of weight rows

// ---------------------------------------------------------------------------
// route: one block per token.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(1024)
moe_route_kernel(const T* __restrict__ x, int width, const float* __restrict__ router_w,
                 const float* __restrict__ correction, const float* __restrict__ shared_gate_w,
                 const float* __restrict__ bias, int NE, int top,
                 float scale, int score_fn, int renormalize, int* __restrict__ chosen, float* __restrict__ weight,
                 float* __restrict__ shared_gate) {
  pdl_wait_block();
  pdl_launch_dependents();
  extern __shared__ __align__(16) float route_smem[];  // x [width], z [NE + 1], choice [NE]
  float* xs = route_smem;
  float* z = xs + width;
  float* choice = z + NE + 1;
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) xs[c] = to_f32<T>(x[(size_t)t * width + c]);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int rows = NE + (shared_gate_w != nullptr ? 1 : 0);
  // A row's loads go out together (a few rows per warp, each a chain of fetches otherwise); the
  // sum's order depends on the width alone.
  const bool vec = width % 4 == 0;
  for (int e = warp; e < rows; e += nwarps) {
    const float* w = e < NE ? router_w + (size_t)e * width : shared_gate_w;
    float acc = 0.f;
    if (vec) {
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll 4
      for (int c = lane * 4; c < width; c += 128) {
        const float4 wv = *reinterpret_cast<const float4*>(w + c);
        const float4 xv = *reinterpret_cast<const float4*>(xs + c);
        a0 = fmaf(wv.x, xv.x, a0); a1 = fmaf(wv.y, xv.y, a1); a2 = fmaf(wv.z, xv.z, a2); a3 = fmaf(wv.w, xv.w, a3);
      }
      acc = (a0 + a1) + (a2 + a3);
    } else {
#pragma unroll 4
      for (int c = lane; c < width; c += 32) acc = fmaf(w[c], xs[c], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) z[e] = acc + (bias != nullptr && e < NE ? bias[e] : 0.f);
  }
  __syncthreads();
  if (warp != 0) return;
  if (shared_gate_w != nullptr && lane == 0) shared_gate[t] = 1.0f / (1.0f + expf(-z[NE]));
  if (score_fn == 0) {
    float m = -INFINITY;
    for (int e = lane; e < NE; e += 32) m = fmaxf(m, z[e]);
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < NE; e += 32) sum += expf(z[e] - m);
    sum = warp_sum(sum);
    for (int e = lane; e < NE; e += 32) z[e] = expf(z[e] - m) / sum;
  } else {
    for (int e = lane; e < NE; e += 32) z[e] = 1.0f / (1.0f + expf(-z[e]));
  }
  for (int e = lane; e < NE; e += 32) choice[e] = z[e] + (correction != nullptr ? correction[e] : 0.f);
  __syncwarp();
  float total = 0.f;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < NE; e += 32) {
      const float v = choice[e];
      if (v > best || (v == best && e < at)) { best = v; at = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at >= NE) at = 0;  // (only if every score is NaN)
    const float s = z[at];
    total += s;
    if (lane == 0) {
      chosen[(size_t)t * top + j] = at;
      weight[(size_t)t * top + j] = s * scale;
      choice[at] = -INFINITY;
    }
    __syncwarp();
  }
  if (renormalize && lane == 0)
    for (int j = 0; j < top; ++j) weight[(size_t)t * top + j] /= total;
}

extern "C" int sb_moe_route(const void* x, int dtype, int num_tokens, int width, const float* router_w,
                            const float* correction, const float* shared_gate_w, const float* bias, int NE, int top,
                            float scale, int score_fn, int renormalize, int* chosen, float* weight,
                            float* shared_gate, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  const size_t smem = ((size_t)width + 2 * NE + 1) * sizeof(float);
  if (top < 1 || top > NE || smem > 200 * 1024) return -13;
  // A warp per router row where a block can hold them (at least 8, at most 32 warps): a row's
  // fetches are then one round for all rows instead of one round after the other.
  int warps = NE + (shared_gate_w != nullptr ? 1 : 0);
  warps = warps < 8 ? 8 : (warps > 32 ? 32 : warps);
  if (dtype == SB_DTYPE_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb_launch(moe_route_kernel<float>, num_tokens, 32 * warps, smem, stream, (const float*)x, width, router_w, correction,
              shared_gate_w, bias, NE, top, scale, score_fn, renormalize, chosen, weight, shared_gate);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb_launch(moe_route_kernel<bf16>, num_tokens, 32 * warps, smem, stream, (const bf16*)x, width, router_w, correction,
              shared_gate_w, bias, NE, top, scale, score_fn, renormalize, chosen, weight, shared_gate);
  }
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// group: one block.  P pairs (pair p = token p / top, choice p % top), E experts with rows.
//   sorted_pair [P]: the pairs of expert 0, then of expert 1, ... (unused entries at the end: -1)
//   pos_of_pair [P]: where pair p stands in sorted_pair, or -1 for an identity expert's pair
//   tile_expert / tile_row0 / tile_rows [max_tiles]: the tiles; unused ones have expert -1
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int* __restrict__ chosen, int P, int E, int max_tiles, int* __restrict__ sorted_pair,
                 int* __restrict__ pos_of_pair, int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                 int* __restrict__ tile_rows) {
  pdl_wait_block();
  pdl_launch_dependents();
  extern __shared__ int group_smem[];  // counts [E], offsets [E], tile_base [E], cursor [E]
  int* counts = group_smem;
  int* offsets = counts + E;
  int* tile_base = offsets + E;
  int* cursor = tile_base + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = cursor[e] = 0;
  for (int k = threadIdx.x; k < max_tiles; k += blockDim.x) tile_expert[k] = -1;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = chosen[p];
    if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int rows = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = rows;
      tile_base[e] = tiles;
      rows += counts[e];
      tiles += (counts[e] + MOE_TILE_M - 1) / MOE_TILE_M;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int n = counts[e];
    for (int i = 0, k = tile_base[e]; i < n && k < max_tiles; i += MOE_TILE_M, ++k) {
      tile_expert[k] = e;
      tile_row0[k] = offsets[e] + i;
      tile_rows[k] = min(MOE_TILE_M, n - i);
    }
  }
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = chosen[p];
    int r = -1;
    if (e >= 0 && e < E) {
      r = offsets[e] + atomicAdd(&cursor[e], 1);
      sorted_pair[r] = p;
    }
    pos_of_pair[p] = r;
  }
}

extern "C" int sb_moe_group(const int* chosen, int P, int E, int max_tiles, int* sorted_pair, int* pos_of_pair,
                            int* tile_expert, int* tile_row0, int* tile_rows, cudaStream_t stream) {
  if (P == 0) return 0;
  const size_t smem = (size_t)4 * (E > 0 ? E : 1) * sizeof(int);
  if (smem > 48 * 1024) return -13;
  sb_launch(moe_group_kernel, 1, 1024, smem, stream, chosen, P, E, max_tiles, sorted_pair, pos_of_pair, tile_expert,
            tile_row0, tile_rows);
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// product over the tiles.  Grid (tiles, column tiles).  Row r of a tile reads row
// `row_pair[r] / pair_div` of A (row_pair null: row r itself) and writes row r of `out`.  A block
// forms two sets of sums: weight rows n0 + c and `second` + n0 + c (c < 32).  GATED: out[r, n0 + c] =
// act(set 0) * set 1.  Otherwise the sets are 64 neighbouring output columns (`second` = 32).
// ---------------------------------------------------------------------------
__device__ __forceinline__ float moe_activation(float g, int act) {
  if (act == 0) {
    const float c = 0.7978845608028654f;
    return 0.5f * g * (1.0f + tanhf(c * (g + 0.044715f * g * g * g)));
  }
  if (act == 1) return g / (1.0f + expf(-g));
  if (act == 4) return 0.5f * g * (1.0f + erff(g * 0.7071067811865476f));  // the exact gelu
  return fmaxf(g, 0.f);
}

// act(gate) * up; activation 3 is the clamped form, which acts on both halves:
// g' = min(g, limit), u' = clamp(u, -limit, limit), g' sigmoid(1.702 g') (u' + 1).
__device__ __forceinline__ float moe_gated_pair(float g, float u, int act, float limit) {
  if (act == 3) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
  }
  return moe_activation(g, act) * u;
}

// 16 bytes from global memory (16-byte aligned) into a tile row (bfloat16 rows are, float rows are not).
__device__ __forceinline__ void moe_copy16(bf16* dst, const bf16* src) {
  *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
}
__device__ __forceinline__ void moe_copy16(float* dst, const float* src) {
  const float4 v = *reinterpret_cast<const float4*>(src);
  dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
}

template <typename T> struct MoeTile;
template <> struct MoeTile<bf16> { static constexpr int K = 64, LD = 72; };
template <> struct MoeTile<float> { static constexpr int K = 32, LD = 33; };

// Stages of the ring of tiles that feeds the products: bfloat16 tiles come by cp.async, up to
// two k-steps ahead of the one being multiplied; float32 tiles are fetched as they are needed.
template <typename T> struct MoeStages;
template <> struct MoeStages<bf16> { static constexpr int N = 3; };
template <> struct MoeStages<float> { static constexpr int N = 1; };

template <typename T>
constexpr size_t moe_product_smem() {
  const size_t ring = (size_t)MoeStages<T>::N * (MOE_TILE_M + 2 * MOE_TILE_N) * MoeTile<T>::LD * sizeof(T);
  const size_t sums = (size_t)2 * MOE_TILE_M * (MOE_TILE_N + 4) * sizeof(float);
  return ring > sums ? ring : sums;
}

__device__ __forceinline__ void moe_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}

template <typename T, bool GATED>
__global__ void __launch_bounds__(256)
moe_product_kernel(const T* __restrict__ A, const int* __restrict__ row_pair, int pair_div,
                   const T* __restrict__ W, size_t expert_stride, int second, int K, int N,
                   const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                   const int* __restrict__ tile_rows, int act, float limit, T* __restrict__ out) {
  pdl_wait_block();
  pdl_launch_dependents();
  constexpr int BK = MoeTile<T>::K, LD = MoeTile<T>::LD, NST = MoeStages<T>::N;
  constexpr int STAGE = (MOE_TILE_M + 2 * MOE_TILE_N) * LD;  // elements: the A tile, then the two W tiles
  extern __shared__ __align__(128) unsigned char moe_smem[];
  T* ring = reinterpret_cast<T*>(moe_smem);
  float* Cs = reinterpret_cast<float*>(moe_smem);  // the sums, once the ring is done with
  __shared__ int src_row[MOE_TILE_M];
  constexpr int CLD = MOE_TILE_N + 4;
  const int e = tile_expert[blockIdx.x];
  if (e < 0) return;
  const int row0 = tile_row0[blockIdx.x], rows = tile_rows[blockIdx.x];
  const int n0 = blockIdx.y * (GATED ? MOE_TILE_N : 2 * MOE_TILE_N);
  const T* We = W + (size_t)e * expert_stride;
  if (threadIdx.x < MOE_TILE_M) {
    int r = -1;
    if ((int)threadIdx.x < rows) r = row_pair != nullptr ? row_pair[row0 + threadIdx.x] / pair_div : row0 + threadIdx.x;
    src_row[threadIdx.x] = r;
  }
  __syncthreads();
  constexpr int V = 16 / sizeof(T);  // elements of a 16-byte piece
  const bool vec = K % V == 0;

  // The ring starts as zeros: rows of the tile that hold no pair, and weight rows beyond the
  // matrix, are never fetched and stay zero (a step of single tokens has a few rows per tile).
  for (int i = threadIdx.x; i < (int)(NST * STAGE * sizeof(T) / 16); i += blockDim.x)
    reinterpret_cast<uint4*>(moe_smem)[i] = make_uint4(0u, 0u, 0u, 0u);
  __syncthreads();

  // Fetches k-step k0 into a stage: the tile's `rows` rows of A, then the two sets of weight rows;
  // 16-byte pieces where a whole one lies inside the matrix (bfloat16: asynchronously), the ragged
  // end of K by plain stores with zeros behind it.  A thread fetches the same pieces in every
  // k-step: where they come from and go to is worked out once.
  constexpr int PIECES = BK / V;
  constexpr int MINE = (MOE_TILE_M + 2 * MOE_TILE_N) * PIECES / 256;  // pieces per thread (256 threads)
  const T* piece_src[MINE];
  int piece_dst[MINE], piece_col[MINE];
#pragma unroll
  for (int p = 0; p < MINE; ++p) {
    const int idx = threadIdx.x + p * 256;
    const int a_pieces = rows * PIECES;
    piece_src[p] = nullptr;
    piece_col[p] = (idx % PIECES) * V;
    int j = 0;
    if (idx < a_pieces) {
      j = idx / PIECES;
      piece_src[p] = A + (size_t)src_row[j] * K;
    } else if (idx < a_pieces + 2 * MOE_TILE_N * PIECES) {
      const int w = (idx - a_pieces) / PIECES, set = w / MOE_TILE_N, jj = w - set * MOE_TILE_N;
      const int n = n0 + (GATED ? 0 : set * MOE_TILE_N) + jj;  // output column
      j = MOE_TILE_M + w;
      if (n < N) piece_src[p] = We + (size_t)(GATED ? set * second + n : n) * K;
    }
    piece_dst[p] = j * LD + piece_col[p];
  }
  auto fetch = [&](T* stage, int k0) {
#pragma unroll
    for (int p = 0; p < MINE; ++p) {
      if (piece_src[p] == nullptr) continue;
      const int c = piece_col[p];
      T* dst = stage + piece_dst[p];
      const T* src = piece_src[p] + k0 + c;
      if (vec && k0 + c + V <= K) {
        if constexpr (sizeof(T) == 2) moe_async16(dst, src);
        else moe_copy16(dst, src);
      } else {
#pragma unroll
        for (int q = 0; q < V; ++q) dst[q] = k0 + c + q < K ? src[q] : from_f32<T>(0.f);
      }
    }
  };

  [[maybe_unused]] const int warp = threadIdx.x >> 5;
  // float32: thread (ty, tx) owns rows 4 ty .. 4 ty + 3 and columns 2 tx, 2 tx + 1 of both sets
  [[maybe_unused]] const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  [[maybe_unused]] float acc[2][4][2];
#pragma unroll
  for (int s = 0; s < 2; ++s)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[s][i][0] = acc[s][i][1] = 0.f;
  [[maybe_unused]] nvcuda::wmma::fragment<nvcuda::wmma::accumulator, 16, 16, 16, float> cfrag[2];
  if constexpr (sizeof(T) == 2) {
    nvcuda::wmma::fill_fragment(cfrag[0], 0.f);
    nvcuda::wmma::fill_fragment(cfrag[1], 0.f);
  }

  const int steps = (K + BK - 1) / BK;
  if constexpr (NST > 1) {
#pragma unroll
    for (int p = 0; p < NST - 1; ++p) {
      if (p < steps) fetch(ring + p * STAGE, p * BK);
      asm volatile("cp.async.commit_group;\n" ::);
    }
  }
  for (int kt = 0; kt < steps; ++kt) {
    const T* As = ring + (kt % NST) * STAGE;
    const T* Ws = As + MOE_TILE_M * LD;
    if constexpr (NST > 1) {
      // the stage that k-step kt + NST - 1 goes to was multiplied in the step before this one
      if (kt + NST - 1 < steps) fetch(ring + ((kt + NST - 1) % NST) * STAGE, (kt + NST - 1) * BK);
      asm volatile("cp.async.commit_group;\n" ::);
      asm volatile("cp.async.wait_group %0;\n" ::"n"(NST - 1));
    } else {
      fetch(ring, kt * BK);
    }
    __syncthreads();
    if constexpr (sizeof(T) == 2) {
      using namespace nvcuda;
      const int wr = warp & 3, wc = warp >> 2;
      if (wr * 16 < rows)  // (a warp whose 16 rows hold no pair has nothing to multiply)
#pragma unroll
      for (int kk = 0; kk < BK; kk += 16) {
        wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> a;
        wmma::load_matrix_sync(a, reinterpret_cast<const bf16*>(As) + wr * 16 * LD + kk, LD);
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::col_major> b;
          wmma::load_matrix_sync(b, reinterpret_cast<const bf16*>(Ws) + (s * MOE_TILE_N + wc * 16) * LD + kk, LD);
          wmma::mma_sync(cfrag[s], a, b, cfrag[s]);
        }
      }
    } else {
      const float* Af = reinterpret_cast<const float*>(As);
      const float* Wf = reinterpret_cast<const float*>(Ws);
#pragma unroll 8
      for (int kk = 0; kk < BK; ++kk) {
        float a[4], b[2][2];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = Af[(ty * 4 + i) * LD + kk];
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          b[s][0] = Wf[(s * MOE_TILE_N + tx * 2) * LD + kk];
          b[s][1] = Wf[(s * MOE_TILE_N + tx * 2 + 1) * LD + kk];
        }
#pragma unroll
        for (int s = 0; s < 2; ++s)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            acc[s][i][0] = fmaf(a[i], b[s][0], acc[s][i][0]);
            acc[s][i][1] = fmaf(a[i], b[s][1], acc[s][i][1]);
          }
      }
    }
    __syncthreads();
  }
  if constexpr (NST > 1) asm volatile("cp.async.wait_group 0;\n" ::);
  if constexpr (sizeof(T) == 2) {
    const int wr = warp & 3, wc = warp >> 2;
#pragma unroll
    for (int s = 0; s < 2; ++s)
      nvcuda::wmma::store_matrix_sync(Cs + (s * MOE_TILE_M + wr * 16) * CLD + wc * 16, cfrag[s], CLD,
                                      nvcuda::wmma::mem_row_major);
  } else {
#pragma unroll
    for (int s = 0; s < 2; ++s)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        Cs[(s * MOE_TILE_M + ty * 4 + i) * CLD + tx * 2] = acc[s][i][0];
        Cs[(s * MOE_TILE_M + ty * 4 + i) * CLD + tx * 2 + 1] = acc[s][i][1];
      }
  }
  __syncthreads();
  if (GATED) {
    for (int idx = threadIdx.x; idx < rows * MOE_TILE_N; idx += blockDim.x) {
      const int r = idx / MOE_TILE_N, c = idx - r * MOE_TILE_N;
      if (n0 + c < N)
        out[(size_t)(row0 + r) * N + n0 + c] =
            from_f32<T>(moe_gated_pair(Cs[r * CLD + c], Cs[(MOE_TILE_M + r) * CLD + c], act, limit));
    }
  } else {
    for (int idx = threadIdx.x; idx < rows * 2 * MOE_TILE_N; idx += blockDim.x) {
      const int r = idx / (2 * MOE_TILE_N), c = idx - r * 2 * MOE_TILE_N;
      const int s = c / MOE_TILE_N, cc = c - s * MOE_TILE_N;
      if (n0 + c < N) {
        const float v = Cs[(s * MOE_TILE_M + r) * CLD + cc];
        out[(size_t)(row0 + r) * N + n0 + c] = from_f32<T>(act >= 0 ? moe_activation(v, act) : v);
      }
    }
  }
}

// gated = 1: W [E, 2 N, K] (gate rows, then up rows), out [P, N] = act(gate) * up;
// gated = 0: W [E, N, K], out [P, N] = act(sums), act -1: the sums themselves.
// act: 0 gelu (tanh form), 1 silu, 2 relu, 3 the clamped form with `limit` (gated only), 4 the exact gelu.
extern "C" int sb_moe_product(const void* A, const int* row_pair, int pair_div, const void* W, int dtype, int gated,
                              int K, int N, const int* tile_expert, const int* tile_row0, const int* tile_rows,
                              int max_tiles, int act, float limit, void* out, cudaStream_t stream) {
  if (max_tiles == 0 || N == 0) return 0;
  if (K <= 0 || act < (gated ? 0 : -1) || act > 4 || (act == 3 && !(gated && limit > 0.f)) || pair_div < 1) return -13;
  const size_t stride = (size_t)(gated ? 2 : 1) * N * K;
  const int per_block = gated ? MOE_TILE_N : 2 * MOE_TILE_N;
  const dim3 grid(max_tiles, (N + per_block - 1) / per_block);
#define SB_MOE_PRODUCT(T_, G_)                                                                                  \
  do {                                                                                                          \
    if (moe_product_smem<T_>() > 48 * 1024)                                                                     \
      cudaFuncSetAttribute(moe_product_kernel<T_, G_>, cudaFuncAttributeMaxDynamicSharedMemorySize,             \
                           (int)moe_product_smem<T_>());                                                        \
    sb_launch(moe_product_kernel<T_, G_>, grid, 256, moe_product_smem<T_>(), stream, (const T_*)A, row_pair,    \
              pair_div, (const T_*)W, stride, G_ ? N : MOE_TILE_N, K, N, tile_expert, tile_row0, tile_rows,     \
              act, limit, (T_*)out);                                                                            \
  } while (0)
  if (dtype == SB_DTYPE_F32) {
    if (gated) SB_MOE_PRODUCT(float, true);
    else SB_MOE_PRODUCT(float, false);
  } else {
    if (gated) SB_MOE_PRODUCT(bf16, true);
    else SB_MOE_PRODUCT(bf16, false);
  }
#undef SB_MOE_PRODUCT
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// combine: a block per token and slice of columns.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const T* __restrict__ x, const T* __restrict__ y_pair, const int* __restrict__ chosen,
                   const float* __restrict__ weight, const int* __restrict__ pos_of_pair,
                   const T* __restrict__ shared, const float* __restrict__ shared_gate, int E, int top, int width,
                   T* __restrict__ out) {
  pdl_wait_block();
  pdl_launch_dependents();
  // Grid (token, slice of 256 columns): one column per thread.
  const int t = blockIdx.x;
  const float sg = shared == nullptr ? 0.f : (shared_gate != nullptr ? shared_gate[t] : 1.0f);
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c < width) {
    float acc = 0.f;
    for (int j = 0; j < top; ++j) {
      const int p = t * top + j;
      const int pos = pos_of_pair[p];
      const float v = pos >= 0 ? to_f32<T>(y_pair[(size_t)pos * width + c]) : to_f32<T>(x[(size_t)t * width + c]);
      acc = fmaf(weight[p], v, acc);
    }
    if (shared != nullptr) acc = fmaf(sg, to_f32<T>(shared[(size_t)t * width + c]), acc);
    out[(size_t)t * width + c] = from_f32<T>(acc);
  }
}

extern "C" int sb_moe_combine(const void* x, const void* y_pair, int dtype, const int* chosen, const float* weight,
                              const int* pos_of_pair, const void* shared, const float* shared_gate, int E, int top,
                              int num_tokens, int width, void* out, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  const dim3 grid((unsigned)num_tokens, (unsigned)((width + 255) / 256));
  if (dtype == SB_DTYPE_F32)
    sb_launch(moe_combine_kernel<float>, grid, 256, 0, stream, (const float*)x, (const float*)y_pair, chosen,
              weight, pos_of_pair, (const float*)shared, shared_gate, E, top, width, (float*)out);
  else
    sb_launch(moe_combine_kernel<bf16>, grid, 256, 0, stream, (const bf16*)x, (const bf16*)y_pair, chosen,
              weight, pos_of_pair, (const bf16*)shared, shared_gate, E, top, width, (bf16*)out);
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// The experts of a long prompt portion, one after the other through the dense products, issued
// from here so that the host pays one call, not two per expert: rows [starts[i], starts[i] +
// counts[i]) of xs (sorted by expert) go through expert experts[i]:
//   h = act(xs W_gate^T) * (xs W_up^T)   the tcgen05 gated product (gemm_gated_tc.cu)
//   y = h W_down^T                        the library's product (gemm_library.cu)
// Returns -9 (nothing launched for that expert or any after it) when a product does not take the
// shape; the caller then runs those experts through the kernel table's own methods.
// One expert's products fill a part of the GPU only (32 tiles of 256 x 128 for 512 rows and 2,048
// features, on 74 pairs of SMs): with `workspace2` every other expert goes to a second stream, which
// starts after what `stream` holds so far and which `stream` waits for at the end.
// ---------------------------------------------------------------------------
extern "C" int sb_gemm_gated_tc(const void* x, const void* w, void* out, int M, int F, int K, int act, float limit,
                                int blocks, int pairs, int* err, cudaStream_t stream);
extern "C" int sb_gemm_library_bf16(const void* x, const void* w, void* out, int M, int N, int K, int out_f32,
                                    void* workspace, long long workspace_bytes, cudaStream_t stream);

// h <- act(h) in place, eight numbers per thread (experts without a gate on the dense route).
__global__ void __launch_bounds__(256) activate_rows_kernel(bf16* __restrict__ h, long long groups, int act) {
  pdl_wait();
  pdl_launch_dependents();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= groups) return;
  uint4 v = reinterpret_cast<uint4*>(h)[i];
  __nv_bfloat162* pair = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __bfloat1622float2(pair[e]);
    pair[e] = __floats2bfloat162_rn(moe_activation(f.x, act), moe_activation(f.y, act));
  }
  reinterpret_cast<uint4*>(h)[i] = v;
}

// `gated` 0: experts without a gate, gate_up [E, hidden, width]: the library's product, the
// activation in place, the library's product.
extern "C" int sb_experts_dense_bf16(const void* xs, const void* gate_up, const void* down, void* h, void* y,
                                     const int* starts, const int* counts, const int* experts, int num, int width,
                                     int hidden, int act, float limit, int gated, int blocks, int pairs, void* workspace,
                                     void* workspace2, long long workspace_bytes, int* done, int* err,
                                     cudaStream_t stream) {
  *done = 0;
  static cudaStream_t side = nullptr;
  static cudaEvent_t fork_event = nullptr, join_event = nullptr;
  bool two = workspace2 != nullptr && num > 1;
  if (two && side == nullptr) {
    if (cudaStreamCreateWithFlags(&side, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&fork_event, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&join_event, cudaEventDisableTiming) != cudaSuccess) {
      side = nullptr;
      two = false;
    }
  }
  if (two) {
    cudaEventRecord(fork_event, stream);
    cudaStreamWaitEvent(side, fork_event, 0);
  }
  // (whatever happens below, `stream` waits for the second stream before this returns)
  struct Join {
    bool on; cudaStream_t main, other; cudaEvent_t event;
    ~Join() { if (on) { cudaEventRecord(event, other); cudaStreamWaitEvent(main, event, 0); } }
  } join{two, stream, side, join_event};
  cudaStream_t main_stream = stream;
  void* main_workspace = workspace;
  for (int i = 0; i < num; ++i) {
    stream = (two && (i & 1)) ? side : main_stream;
    workspace = (two && (i & 1)) ? workspace2 : main_workspace;
    const size_t row = (size_t)starts[i];
    const bf16* x_i = (const bf16*)xs + row * width;
    bf16* h_i = (bf16*)h + row * hidden;
    const bf16* gu = (const bf16*)gate_up + (size_t)experts[i] * (gated ? 2 : 1) * hidden * width;
    const bf16* dn = (const bf16*)down + (size_t)experts[i] * width * hidden;
    int rc;
    if (gated) {
      rc = sb_gemm_gated_tc(x_i, gu, h_i, counts[i], hidden, width, act, limit, blocks, pairs, err, stream);
      if (rc != 0) return rc;
    } else {
      rc = sb_gemm_library_bf16(x_i, gu, h_i, counts[i], hidden, width, 0, workspace, workspace_bytes, stream);
      if (rc != 0) return rc;
      const long long groups = (long long)counts[i] * hidden / 8;  // (hidden is a multiple of 8, rows start on 16 bytes)
      sb_launch(activate_rows_kernel, dim3((unsigned)((groups + 255) / 256)), 256, 0, stream, h_i, groups, act);
      SB_LAUNCH_CHECK();
    }
    rc = sb_gemm_library_bf16(h_i, dn, (bf16*)y + row * width, counts[i], width, hidden, 0, workspace, workspace_bytes,
                              stream);
    if (rc != 0) return rc;  // (h_i is computed; the caller redoes this expert whole)
    *done = i + 1;
  }
  return 0;
}
