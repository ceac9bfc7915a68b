// Walks of two recurrent mixers whose state is a matrix per head and request (float32, in a state
// slot): the generalized delta rule and the state-space recurrence of Mamba-2.
//
//   generalized delta rule   S [d, d] per head;  per token, with decay w, unit key u, removal rate a:
//                              p   = u^T S                       (the old state)
//                              S  <- diag(w) S - (a * u) p + k v^T
//                              o   = S^T r
//   state-space recurrence   S [N, dv] per head;  S <- exp(-exp(A) dt) S + dt B x^T;  y = S^T C + D x
//
// Both share one layout: a block owns `cols` columns of one (head, sequence) and walks the
// sequence's tokens of this step in order; a column of S is held by RS neighbouring lanes with ROWS
// rows each in registers (row rs + RS r), sums over rows are butterfly sums over those lanes in an
// order that does not depend on the step's shape; the tokens' vectors come to shared memory by
// cp.async, a chunk of tokens at a time, the next chunk under way while this one is walked.  The
// state is read once and written once per step, by the first row of its slot (a decode graph pads
// its batch by repeating a request).  Everything is float32.
#include "common.cuh"

#define SB_ERR_BAD_SLOT 16

__device__ __forceinline__ bool owns_slot(const int* slots, int b) {
  const int slot = slots[b];
  for (int i = 0; i < b; ++i)
    if (slots[i] == slot) return false;
  return true;
}

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

__device__ __forceinline__ void stage4(float* smem, const float* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void stage16(float* smem, const float* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}
// n floats; `wide`: both addresses are 16-byte aligned and n is a multiple of 4.
__device__ __forceinline__ void stage_row(float* smem, const float* gmem, int n, bool wide) {
  if (wide) {
    for (int c = threadIdx.x * 4; c < n; c += blockDim.x * 4) stage16(smem + c, gmem + c);
  } else {
    for (int c = threadIdx.x; c < n; c += blockDim.x) stage4(smem + c, gmem + c);
  }
}

// ---------------------------------------------------------------------------
// Inputs of the generalized delta rule, once per token.  pre [T, pre_width] = r | k | v | gate | a | ...
// (each H d), low [T, low_width] = the decay's low-rank output (H d).  A warp per (token, head):
//   vecs [T, H, 5, d] = w, u, a * u, k, r ;  vals [T, H, d] = v ;  dots [T, H, 2] = r . (a u), r . k
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
general_delta_inputs_kernel(const T* __restrict__ pre, int pre_width, const T* __restrict__ low, int low_width,
                            const float* __restrict__ decay_bias, const float* __restrict__ removal_bias, int H,
                            int d, int num_tokens, float* __restrict__ vecs, float* __restrict__ vals,
                            float* __restrict__ dots) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)num_tokens * H) return;
  const int t = (int)(item / H), h = (int)(item - (long long)t * H);
  const int inner = H * d;
  const T* row = pre + (size_t)t * pre_width + (size_t)h * d;
  const T* lrow = low + (size_t)t * low_width + (size_t)h * d;
  float kk = 0.f;
  for (int c = lane; c < d; c += 32) {
    const float k = to_f32<T>(row[inner + c]);
    kk = fmaf(k, k, kk);
  }
  const float inv = 1.0f / sqrtf(warp_sum(kk) + 1e-6f);
  const float rate = 0.6065306597126334f;  // e^(-1/2)
  float* out = vecs + (size_t)item * 5 * d;
  float ra = 0.f, rk = 0.f;
  for (int c = lane; c < d; c += 32) {
    const float r = to_f32<T>(row[c]), k = to_f32<T>(row[inner + c]);
    const float a = sigmoidf_(to_f32<T>(row[4 * inner + c]) + removal_bias[h * d + c]);
    const float w = expf(-rate * sigmoidf_(to_f32<T>(lrow[c]) + decay_bias[h * d + c]));
    const float u = k * inv, au = a * u;
    out[c] = w;
    out[d + c] = u;
    out[2 * d + c] = au;
    out[3 * d + c] = k;
    out[4 * d + c] = r;
    vals[(size_t)item * d + c] = to_f32<T>(row[2 * inner + c]);
    ra = fmaf(r, au, ra);
    rk = fmaf(r, k, rk);
  }
  ra = warp_sum(ra);
  rk = warp_sum(rk);
  if (lane == 0) {
    dots[(size_t)item * 2] = ra;
    dots[(size_t)item * 2 + 1] = rk;
  }
}

template <int RS, int ROWS>
__global__ void __launch_bounds__(128)
general_delta_scan_kernel(const float* __restrict__ vecs, const float* __restrict__ vals,
                          const float* __restrict__ dots, float* __restrict__ state, const int* __restrict__ cu_q,
                          const int* __restrict__ slots, int num_slots, int H, int d, int cols, int chunk,
                          float* __restrict__ out, int* err) {
  pdl_wait_block();
  pdl_launch_dependents();
  extern __shared__ __align__(16) float stage[];  // two buffers of chunk x (5 d | cols_pad | 4)
  const int h = blockIdx.x, b = blockIdx.y, col0 = blockIdx.z * cols;
  const int rs = threadIdx.x % RS, col_local = threadIdx.x / RS;
  const int col = col0 + col_local;
  const bool on = col_local < cols && col < d;
  const int first = cu_q[b], n = cu_q[b + 1] - first;
  const int slot = slots[b];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(err, SB_ERR_BAD_SLOT);
    return;
  }
  const int cols_pad = (cols + 3) & ~3;
  const int per_token = 5 * d + cols_pad + 4;
  const bool wide = (d & 3) == 0;

  // Staging a chunk, where rows are whole 16-byte groups: a thread takes a piece of a token (16 bytes of
  // the five vectors, one value, one of the two dot products) and copies it for every token of the
  // chunk, one copy and two additions per token; all threads walking every token's rows in turn cost more
  // instructions than the walk itself.
  const int vec_pieces = (5 * d) >> 2, pieces = vec_pieces + cols + 2;
  auto issue_pieces = [&](float* buf, int base, int count) {
    for (int k = threadIdx.x; k < pieces; k += blockDim.x) {
      const float* src;
      size_t stride;
      int dst_off;
      const bool sixteen = k < vec_pieces;
      if (sixteen) {
        src = vecs + ((size_t)(first + base) * H + h) * 5 * d + 4 * k; stride = (size_t)H * 5 * d; dst_off = 4 * k;
      } else if (k < vec_pieces + cols) {
        const int c = k - vec_pieces;
        src = vals + ((size_t)(first + base) * H + h) * d + min(col0 + c, d - 1); stride = (size_t)H * d; dst_off = 5 * d + c;
      } else {
        const int j = k - vec_pieces - cols;
        src = dots + ((size_t)(first + base) * H + h) * 2 + j; stride = (size_t)2 * H; dst_off = 5 * d + cols_pad + j;
      }
      float* dst = buf + dst_off;
      for (int i = 0; i < count; ++i, src += stride, dst += per_token) {
        if (sixteen) stage16(dst, src);
        else stage4(dst, src);
      }
    }
  };
  auto issue = [&](int which, int base) {
    float* buf = stage + (size_t)which * chunk * per_token;
    const int count = min(chunk, n - base);
    if (wide) {
      issue_pieces(buf, base, count);
      asm volatile("cp.async.commit_group;\n" ::);
      return;
    }
    for (int i = 0; i < count; ++i) {
      const size_t at = (size_t)(first + base + i) * H + h;
      float* dst = buf + (size_t)i * per_token;
      stage_row(dst, vecs + at * 5 * d, 5 * d, wide);
      for (int c = threadIdx.x; c < cols; c += blockDim.x) stage4(dst + 5 * d + c, vals + at * d + min(col0 + c, d - 1));
      if (threadIdx.x < 2) stage4(dst + 5 * d + cols_pad + threadIdx.x, dots + at * 2 + threadIdx.x);
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };

  if (n > 0) issue(0, 0);
  float* S = state + ((size_t)slot * H + h) * d * d;
  float s[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int row = rs + RS * r;
    s[r] = (on && row < d) ? S[(size_t)row * d + col] : 0.f;
  }
  int which = 0;
  for (int base = 0; base < n; base += chunk, which ^= 1) {
    const int count = min(chunk, n - base);
    if (base + chunk < n) {
      issue(which ^ 1, base + chunk);
      asm volatile("cp.async.wait_group 1;\n" ::);
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::);
    }
    __syncthreads();
    const float* buf = stage + (size_t)which * chunk * per_token;
    // A token's vectors are fetched into registers while the token before it is worked on: the walk
    // is a chain of dependent steps per token, and the fetches' latency would otherwise be part of it.
    float cw[ROWS], cu[ROWS], ca[ROWS], ck[ROWS], cr[ROWS], cv, cra, crk;
    auto fetch = [&](int i, float (&fw)[ROWS], float (&fu)[ROWS], float (&fa)[ROWS], float (&fk)[ROWS],
                     float (&fr)[ROWS], float& fv, float& fra, float& frk) {
      const float* w = buf + (size_t)i * per_token;
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const int row = min(rs + RS * r, d - 1);
        fw[r] = w[row];
        fu[r] = w[d + row];
        fa[r] = w[2 * d + row];
        fk[r] = w[3 * d + row];
        fr[r] = w[4 * d + row];
      }
      fv = w[5 * d + min(col_local, cols - 1)];
      fra = w[5 * d + cols_pad];
      frk = w[5 * d + cols_pad + 1];
    };
    constexpr bool AHEAD = ROWS <= 8;  // (two tokens' vectors of 32 rows do not fit the registers)
    if constexpr (AHEAD) fetch(0, cw, cu, ca, ck, cr, cv, cra, crk);
    for (int i = 0; i < count; ++i) {
      float nw[ROWS], nu[ROWS], na[ROWS], nk[ROWS], nr[ROWS], nv, nra, nrk;
      const float* here = buf + (size_t)i * per_token;  // (32 rows per lane: read where they are used)
      if constexpr (AHEAD) {
        fetch(min(i + 1, count - 1), nw, nu, na, nk, nr, nv, nra, nrk);
      } else {
        cv = here[5 * d + min(col_local, cols - 1)];
        cra = here[5 * d + cols_pad];
        crk = here[5 * d + cols_pad + 1];
      }
      // One pass over the old state gives both sums: o = r . (w * s) - p (r . a u) + v_j (r . k).
      float p = 0.f, od = 0.f;
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const int row = rs + RS * r;
        if (row < d) {
          p = fmaf(AHEAD ? cu[r] : here[d + row], s[r], p);
          s[r] *= AHEAD ? cw[r] : here[row];
          od = fmaf(AHEAD ? cr[r] : here[4 * d + row], s[r], od);
        }
      }
#pragma unroll
      for (int o = 1; o < RS; o <<= 1) {
        p += __shfl_xor_sync(0xffffffffu, p, o);
        od += __shfl_xor_sync(0xffffffffu, od, o);
      }
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const int row = rs + RS * r;
        if (row < d) s[r] = fmaf(AHEAD ? ck[r] : here[3 * d + row], cv, fmaf(-(AHEAD ? ca[r] : here[2 * d + row]), p, s[r]));
      }
      if (on && rs == 0) out[((size_t)(first + base + i) * H + h) * d + col] = fmaf(cv, crk, fmaf(-p, cra, od));
      if constexpr (AHEAD) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          cw[r] = nw[r]; cu[r] = nu[r]; ca[r] = na[r]; ck[r] = nk[r]; cr[r] = nr[r];
        }
        cv = nv; cra = nra; crk = nrk;
      }
    }
    __syncthreads();  // the buffer is filled again two chunks on
  }
  if (on && owns_slot(slots, b)) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int row = rs + RS * r;
      if (row < d) S[(size_t)row * d + col] = s[r];
    }
  }
}

// The delta rule's walk with a patch of the state per lane (4 rows x 4 columns), for prompt portions
// with heads of 16 to 128 channels in whole groups of four: a fetched element of a vector serves four
// multiply-adds.  RG lanes (a power of two, 4 to 32) stand over the rows, 32 / RG groups of four
// columns per warp.  The sums u^T S of a lane's four columns are needed by every lane of the group
// before the update (a butterfly over the RG lanes); the sums for the output wait for nobody and meet in
// a butterfly that halves what is passed on in its first two steps.
template <int RG>
__global__ void __launch_bounds__(128)
general_delta_patch_kernel(const float* __restrict__ vecs, const float* __restrict__ vals,
                           const float* __restrict__ dots, float* __restrict__ state, const int* __restrict__ cu_q,
                           const int* __restrict__ slots, int num_slots, int H, int d, int chunk,
                           float* __restrict__ out, int* err) {
  pdl_wait_block();
  pdl_launch_dependents();
  constexpr int CG = 32 / RG, NP = RG * 4;
  extern __shared__ __align__(16) float stage[];  // two buffers of chunk x (w, u, a u, k, r: NP each | v: cols | 4)
  const int warps = blockDim.x >> 5, cols = warps * CG * 4;
  const int h = blockIdx.x, b = blockIdx.y, col0 = blockIdx.z * cols;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rg = lane % RG, cg = warp * CG + lane / RG;
  const int row_first = rg * 4, col_local = cg * 4, col_first = col0 + col_local;
  const int first = cu_q[b], n = cu_q[b + 1] - first;
  const int slot = slots[b];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(err, SB_ERR_BAD_SLOT);
    return;
  }
  const int per_token = 5 * NP + cols + 4;
  const int cols_here = max(0, min(cols, d - col0));
  for (int i = threadIdx.x; i < 2 * chunk * per_token; i += blockDim.x) stage[i] = 0.f;  // rows and columns past d stay zero
  __syncthreads();
  const int d4 = d >> 2, vec_pieces = 5 * d4, pieces = vec_pieces + cols_here + 2;
  auto issue = [&](int which, int base) {
    float* buf = stage + (size_t)which * chunk * per_token;
    const int count = min(chunk, n - base);
    for (int k = threadIdx.x; k < pieces; k += blockDim.x) {
      const float* src;
      size_t stride;
      int dst_off;
      const bool sixteen = k < vec_pieces;
      if (sixteen) {
        const int j = k / d4, within = k - j * d4;
        src = vecs + ((size_t)(first + base) * H + h) * 5 * d + (size_t)j * d + 4 * within; stride = (size_t)H * 5 * d;
        dst_off = j * NP + 4 * within;
      } else if (k < vec_pieces + cols_here) {
        const int c = k - vec_pieces;
        src = vals + ((size_t)(first + base) * H + h) * d + col0 + c; stride = (size_t)H * d; dst_off = 5 * NP + c;
      } else {
        const int j = k - vec_pieces - cols_here;
        src = dots + ((size_t)(first + base) * H + h) * 2 + j; stride = (size_t)2 * H; dst_off = 5 * NP + cols + j;
      }
      float* dst = buf + dst_off;
      for (int i = 0; i < count; ++i, src += stride, dst += per_token) {
        if (sixteen) stage16(dst, src);
        else stage4(dst, src);
      }
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };

  if (n > 0) issue(0, 0);
  float* S = state + ((size_t)slot * H + h) * d * d;
  float s[4][4];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int q = 0; q < 4; ++q)
      s[r][q] = (row_first + r < d && col_first + q < d) ? S[(size_t)(row_first + r) * d + col_first + q] : 0.f;
  const bool low1 = rg & 1, low2 = rg & 2;
  int which = 0;
  for (int base = 0; base < n; base += chunk, which ^= 1) {
    const int count = min(chunk, n - base);
    if (base + chunk < n) {
      issue(which ^ 1, base + chunk);
      asm volatile("cp.async.wait_group 1;\n" ::);
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::);
    }
    __syncthreads();
    const float* buf = stage + (size_t)which * chunk * per_token;
#pragma unroll 2
    for (int i = 0; i < count; ++i) {
      const float* tok = buf + (size_t)i * per_token;
      const float4 w4 = *reinterpret_cast<const float4*>(tok + row_first);
      const float4 u4 = *reinterpret_cast<const float4*>(tok + NP + row_first);
      const float4 a4 = *reinterpret_cast<const float4*>(tok + 2 * NP + row_first);
      const float4 k4 = *reinterpret_cast<const float4*>(tok + 3 * NP + row_first);
      const float4 r4 = *reinterpret_cast<const float4*>(tok + 4 * NP + row_first);
      const float4 v4 = *reinterpret_cast<const float4*>(tok + 5 * NP + col_local);
      const float ra = tok[5 * NP + cols], rk = tok[5 * NP + cols + 1];
      const float w[4] = {w4.x, w4.y, w4.z, w4.w}, u[4] = {u4.x, u4.y, u4.z, u4.w}, au[4] = {a4.x, a4.y, a4.z, a4.w};
      const float k[4] = {k4.x, k4.y, k4.z, k4.w}, rr[4] = {r4.x, r4.y, r4.z, r4.w}, v[4] = {v4.x, v4.y, v4.z, v4.w};
      // one pass over the old state gives both sums: o = r . (w * s) - p (r . a u) + v (r . k)
      float p[4] = {0.f, 0.f, 0.f, 0.f}, od[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          p[q] = fmaf(u[r], s[r][q], p[q]);
          s[r][q] *= w[r];
          od[q] = fmaf(rr[r], s[r][q], od[q]);
        }
#pragma unroll
      for (int o = 1; o < RG; o <<= 1)
#pragma unroll
        for (int q = 0; q < 4; ++q) p[q] += __shfl_xor_sync(0xffffffffu, p[q], o);
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int q = 0; q < 4; ++q) s[r][q] = fmaf(k[r], v[q], fmaf(-au[r], p[q], s[r][q]));
      // lanes with an odd rg go on with columns 2, 3, the others with 0, 1; then one column each
      const float t0 = __shfl_xor_sync(0xffffffffu, low1 ? od[0] : od[2], 1);
      const float t1 = __shfl_xor_sync(0xffffffffu, low1 ? od[1] : od[3], 1);
      const float a0 = (low1 ? od[2] : od[0]) + t0, a1 = (low1 ? od[3] : od[1]) + t1;
      const float t2 = __shfl_xor_sync(0xffffffffu, low2 ? a0 : a1, 2);
      float sum = (low2 ? a1 : a0) + t2;
#pragma unroll
      for (int o = 4; o < RG; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      const int q_mine = (low1 ? 2 : 0) + (low2 ? 1 : 0);
      if (rg < 4 && col_first + q_mine < d) {
        const float vq = low1 ? (low2 ? v[3] : v[2]) : (low2 ? v[1] : v[0]);
        const float pq = low1 ? (low2 ? p[3] : p[2]) : (low2 ? p[1] : p[0]);
        out[((size_t)(first + base + i) * H + h) * d + col_first + q_mine] = fmaf(vq, rk, fmaf(-pq, ra, sum));
      }
    }
    __syncthreads();
  }
  if (owns_slot(slots, b)) {
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int q = 0; q < 4; ++q)
        if (row_first + r < d && col_first + q < d) S[(size_t)(row_first + r) * d + col_first + q] = s[r][q];
  }
}

// scratch: float32 [T, H, 6 d + 2].
extern "C" int sb_general_delta_scan(const void* pre, int pre_width, const void* low, int low_width, int dtype,
                                     const float* decay_bias, const float* removal_bias, float* state,
                                     const int* cu_q, const int* slots, int num_tokens, int num_seqs, int num_slots,
                                     int H, int d, int max_q_len, float* scratch, float* out, int* err,
                                     cudaStream_t stream) {
  if (num_seqs == 0 || num_tokens == 0) return 0;
  if (d <= 0 || d > 1024 || H <= 0) return -13;
  float* vecs = scratch;
  float* vals = vecs + (size_t)num_tokens * H * 5 * d;
  float* dots = vals + (size_t)num_tokens * H * d;
  const long long items = (long long)num_tokens * H;
  const unsigned in_blocks = (unsigned)((items + 7) / 8);
  if (dtype == SB_DTYPE_F32)
    sb_launch(general_delta_inputs_kernel<float>, in_blocks, 256, 0, stream, (const float*)pre, pre_width,
              (const float*)low, low_width, decay_bias, removal_bias, H, d, num_tokens, vecs, vals, dots);
  else
    sb_launch(general_delta_inputs_kernel<bf16>, in_blocks, 256, 0, stream, (const bf16*)pre, pre_width,
              (const bf16*)low, low_width, decay_bias, removal_bias, H, d, num_tokens, vecs, vals, dots);
  SB_LAUNCH_CHECK();
  const bool long_walk = max_q_len >= 64;
  if (long_walk && d >= 16 && d <= 128 && (d & 3) == 0) {
    int rg = 4;
    while (rg * 4 < d) rg <<= 1;
    const int chunk = 16, warps = d <= 64 ? 2 : 4, cols = warps * (32 / rg) * 4;
    const dim3 grid(H, num_seqs, (d + cols - 1) / cols);
    const size_t smem = (size_t)2 * chunk * (5 * rg * 4 + cols + 4) * sizeof(float);
#define SB_GD_PATCH(RG_)                                                                                        \
  do {                                                                                                          \
    if (smem > 48 * 1024)                                                                                       \
      cudaFuncSetAttribute(general_delta_patch_kernel<RG_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    sb_launch_plain(general_delta_patch_kernel<RG_>, grid, warps * 32, smem, stream, vecs, vals, dots, state, cu_q, \
                    slots, num_slots, H, d, chunk, out, err);                                                   \
  } while (0)
    switch (rg) {
      case 4: SB_GD_PATCH(4); break;
      case 8: SB_GD_PATCH(8); break;
      case 16: SB_GD_PATCH(16); break;
      default: SB_GD_PATCH(32); break;
    }
#undef SB_GD_PATCH
    SB_LAUNCH_CHECK();
    return 0;
  }
  const int rows = d <= 256 ? 8 : 32;
  int rs = 1;
  while (rs * rows < d) rs <<= 1;
  const int threads = long_walk ? 128 : 64;
  int chunk = 1;
  while (chunk < 16 && chunk < max_q_len) chunk <<= 1;
  if ((size_t)2 * chunk * (5 * d + 40) * sizeof(float) > 160 * 1024) chunk = chunk > 4 ? 4 : chunk;
  int cols = threads / rs;
  if (cols < 1) cols = 1;
  if (cols > d) cols = d;
  const int block = ((cols * rs + 31) / 32) * 32;
  const dim3 grid(H, num_seqs, (d + cols - 1) / cols);
  const size_t smem = (size_t)2 * chunk * (5 * d + ((cols + 3) & ~3) + 4) * sizeof(float);
  if (smem > 200 * 1024) return -13;
#define SB_GD_SCAN(RS_, ROWS_)                                                                                  \
  do {                                                                                                          \
    if (smem > 48 * 1024)                                                                                       \
      cudaFuncSetAttribute(general_delta_scan_kernel<RS_, ROWS_>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                           (int)smem);                                                                          \
    if (long_walk)                                                                                              \
      sb_launch_plain(general_delta_scan_kernel<RS_, ROWS_>, grid, block, smem, stream, vecs, vals, dots, state, \
                      cu_q, slots, num_slots, H, d, cols, chunk, out, err);                                     \
    else                                                                                                        \
      sb_launch(general_delta_scan_kernel<RS_, ROWS_>, grid, block, smem, stream, vecs, vals, dots, state,     \
                cu_q, slots, num_slots, H, d, cols, chunk, out, err);                                           \
  } while (0)
#define SB_GD(RS_)                               \
  do {                                           \
    if (rows == 8) SB_GD_SCAN(RS_, 8);           \
    else SB_GD_SCAN(RS_, 32);                    \
  } while (0)
  switch (rs) {
    case 1: SB_GD(1); break;
    case 2: SB_GD(2); break;
    case 4: SB_GD(4); break;
    case 8: SB_GD(8); break;
    case 16: SB_GD(16); break;
    default: SB_GD(32); break;
  }
#undef SB_GD
#undef SB_GD_SCAN
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// The state-space recurrence.  xbc [T, C] float32 = x (H dv) | B (G N) | C (G N) after the
// convolution and silu; steps [T, H, 2] = exp(neg_rate dt), dt with dt = softplus(pre + bias).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void state_space_steps_kernel(const T* __restrict__ pre, int pre_width, int offset,
                                         const float* __restrict__ step_bias, const float* __restrict__ neg_rate,
                                         int H, long long total, float* __restrict__ steps) {
  pdl_wait_block();
  pdl_launch_dependents();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / H;
  const int h = (int)(i - t * H);
  const float z = to_f32<T>(pre[t * pre_width + offset + h]) + step_bias[h];
  const float dt = z > 20.f ? z : log1pf(expf(z));
  steps[2 * i] = expf(neg_rate[h] * dt);
  steps[2 * i + 1] = dt;
}

template <int RS, int ROWS>
__global__ void __launch_bounds__(128)
state_space_scan_kernel(const float* __restrict__ xbc, int C, const float* __restrict__ steps,
                        const float* __restrict__ skip, float* __restrict__ state, const int* __restrict__ cu_q,
                        const int* __restrict__ slots, int num_slots, int H, int G, int N, int dv, int cols,
                        int chunk, float* __restrict__ out, int* err) {
  pdl_wait_block();
  pdl_launch_dependents();
  extern __shared__ __align__(16) float stage[];  // two buffers of chunk x (B: N | C: N | x: cols_pad | 4)
  const int h = blockIdx.x, b = blockIdx.y, col0 = blockIdx.z * cols;
  const int rs = threadIdx.x % RS, col_local = threadIdx.x / RS;
  const int col = col0 + col_local;
  const bool on = col_local < cols && col < dv;
  const int first = cu_q[b], n = cu_q[b + 1] - first;
  const int slot = slots[b];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(err, SB_ERR_BAD_SLOT);
    return;
  }
  const int g = h / (H / G);
  const int inner = H * dv;
  const int cols_pad = (cols + 3) & ~3;
  const int n_pad = (N + 3) & ~3;
  const int per_token = 2 * n_pad + cols_pad + 4;
  const bool wide = (N & 3) == 0 && (C & 3) == 0 && (inner & 3) == 0;
  const float d_skip = skip[h];

  auto issue = [&](int which, int base) {
    float* buf = stage + (size_t)which * chunk * per_token;
    const int count = min(chunk, n - base);
    for (int i = 0; i < count; ++i) {
      const float* row = xbc + (size_t)(first + base + i) * C;
      float* dst = buf + (size_t)i * per_token;
      stage_row(dst, row + inner + (size_t)g * N, N, wide);
      stage_row(dst + n_pad, row + inner + (size_t)(G + g) * N, N, wide);
      for (int c = threadIdx.x; c < cols; c += blockDim.x)
        stage4(dst + 2 * n_pad + c, row + (size_t)h * dv + min(col0 + c, dv - 1));
      if (threadIdx.x < 2)
        stage4(dst + 2 * n_pad + cols_pad + threadIdx.x, steps + ((size_t)(first + base + i) * H + h) * 2 + threadIdx.x);
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };

  if (n > 0) issue(0, 0);
  float* S = state + ((size_t)slot * H + h) * N * dv;
  float s[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int row = rs + RS * r;
    s[r] = (on && row < N) ? S[(size_t)row * dv + col] : 0.f;
  }
  int which = 0;
  for (int base = 0; base < n; base += chunk, which ^= 1) {
    const int count = min(chunk, n - base);
    if (base + chunk < n) {
      issue(which ^ 1, base + chunk);
      asm volatile("cp.async.wait_group 1;\n" ::);
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::);
    }
    __syncthreads();
    const float* buf = stage + (size_t)which * chunk * per_token;
    // (a token's update of the state does not wait for the sum that reads it: four tokens at a time let
    // the fetches, updates and sums over lanes of neighbouring tokens overlap)
#pragma unroll(ROWS <= 8 ? 4 : 1)
    for (int i = 0; i < count; ++i) {
      const float* bm = buf + (size_t)i * per_token;
      const float* cm = bm + n_pad;
      const float xj = bm[2 * n_pad + min(col_local, cols - 1)];
      const float decay = bm[2 * n_pad + cols_pad], dt = bm[2 * n_pad + cols_pad + 1];
      const float push = dt * xj;
      float y = 0.f;
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const int row = rs + RS * r;
        if (row < N) {
          s[r] = fmaf(push, bm[row], decay * s[r]);
          y = fmaf(s[r], cm[row], y);
        }
      }
#pragma unroll
      for (int o = 1; o < RS; o <<= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      if (on && rs == 0) out[((size_t)(first + base + i) * H + h) * dv + col] = fmaf(d_skip, xj, y);
    }
    __syncthreads();
  }
  if (on && owns_slot(slots, b)) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int row = rs + RS * r;
      if (row < N) S[(size_t)row * dv + col] = s[r];
    }
  }
}

// The same walk with a patch of the state per lane: 4 neighbouring rows x 4 neighbouring columns, so a
// fetched element of B, C or x serves four multiply-adds (the column-per-lanes layout above fetches one
// per multiply-add, and its instructions, not memory, bound a long walk).  RG lanes (a power of two, 4 to
// 32) stand side by side over the rows, 32 / RG groups of four columns per warp.  The four sums of a lane
// meet over the RG lanes in a butterfly that halves what is passed on in its first two steps.  State sizes
// 16 to 128; rows and columns beyond the state's stay zero (their B, C and x are zero in shared memory).
template <int RG>
__global__ void __launch_bounds__(128)
state_space_patch_kernel(const float* __restrict__ xbc, int C, const float* __restrict__ steps,
                         const float* __restrict__ skip, float* __restrict__ state, const int* __restrict__ cu_q,
                         const int* __restrict__ slots, int num_slots, int H, int G, int N, int dv, int chunk,
                         float* __restrict__ out, int* err) {
  pdl_wait_block();
  pdl_launch_dependents();
  constexpr int CG = 32 / RG, NP = RG * 4;       // column groups per warp; rows a warp spans
  extern __shared__ __align__(16) float stage[];  // two buffers of chunk x (B: NP | C: NP | x: cols | 4)
  const int warps = blockDim.x >> 5, cols = warps * CG * 4;
  const int h = blockIdx.x, b = blockIdx.y, col0 = blockIdx.z * cols;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rg = lane % RG, cg = warp * CG + lane / RG;
  const int row_first = rg * 4, col_local = cg * 4, col_first = col0 + col_local;
  const int first = cu_q[b], n = cu_q[b + 1] - first;
  const int slot = slots[b];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(err, SB_ERR_BAD_SLOT);
    return;
  }
  const int g = h / (H / G);
  const int inner = H * dv;
  const int per_token = 2 * NP + cols + 4;
  const bool wide = (N & 3) == 0 && (C & 3) == 0 && (inner & 3) == 0;
  const int cols_here = min(cols, dv - col0);
  const float d_skip = skip[h];
  // what no copy ever writes stays zero: rows from N on, columns from the head's last on
  for (int i = threadIdx.x; i < 2 * chunk * per_token; i += blockDim.x) stage[i] = 0.f;
  __syncthreads();

  // Staging a chunk: where every piece of a token fits one thread (16 bytes of B or C, one x, one step
  // value), a thread copies its piece of every token of the chunk, one copy and two additions per token;
  // otherwise the threads share out every token's rows in turn.
  const int nb = N >> 2;
  const bool piecewise = wide && 2 * nb + cols_here + 2 <= (int)blockDim.x;
  const float* piece_src = nullptr;
  size_t piece_stride = 0;
  int piece_dst = 0;
  bool piece16 = false;
  {
    const int k = threadIdx.x;
    if (k < nb) {
      piece_src = xbc + (size_t)first * C + inner + (size_t)g * N + 4 * k; piece_stride = C; piece_dst = 4 * k; piece16 = true;
    } else if (k < 2 * nb) {
      piece_src = xbc + (size_t)first * C + inner + (size_t)(G + g) * N + 4 * (k - nb); piece_stride = C;
      piece_dst = NP + 4 * (k - nb); piece16 = true;
    } else if (k < 2 * nb + cols_here) {
      piece_src = xbc + (size_t)first * C + (size_t)h * dv + col0 + (k - 2 * nb); piece_stride = C; piece_dst = 2 * NP + (k - 2 * nb);
    } else if (k < 2 * nb + cols_here + 2) {
      const int j = k - 2 * nb - cols_here;
      piece_src = steps + ((size_t)first * H + h) * 2 + j; piece_stride = (size_t)2 * H; piece_dst = 2 * NP + cols + j;
    }
  }
  auto issue = [&](int which, int base) {
    float* buf = stage + (size_t)which * chunk * per_token;
    const int count = min(chunk, n - base);
    if (piecewise) {
      if (piece_src != nullptr) {
        const float* src = piece_src + (size_t)base * piece_stride;
        float* dst = buf + piece_dst;
        for (int i = 0; i < count; ++i, src += piece_stride, dst += per_token) {
          if (piece16) stage16(dst, src);
          else stage4(dst, src);
        }
      }
      asm volatile("cp.async.commit_group;\n" ::);
      return;
    }
    for (int i = 0; i < count; ++i) {
      const float* row = xbc + (size_t)(first + base + i) * C;
      float* dst = buf + (size_t)i * per_token;
      stage_row(dst, row + inner + (size_t)g * N, N, wide);
      stage_row(dst + NP, row + inner + (size_t)(G + g) * N, N, wide);
      for (int c = threadIdx.x; c < cols_here; c += blockDim.x) stage4(dst + 2 * NP + c, row + (size_t)h * dv + col0 + c);
      if (threadIdx.x < 2)
        stage4(dst + 2 * NP + cols + threadIdx.x, steps + ((size_t)(first + base + i) * H + h) * 2 + threadIdx.x);
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };

  if (n > 0) issue(0, 0);
  float* S = state + ((size_t)slot * H + h) * N * dv;
  float s[4][4];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int q = 0; q < 4; ++q)
      s[r][q] = (row_first + r < N && col_first + q < dv) ? S[(size_t)(row_first + r) * dv + col_first + q] : 0.f;
  const bool low1 = rg & 1, low2 = rg & 2;
  int which = 0;
  for (int base = 0; base < n; base += chunk, which ^= 1) {
    const int count = min(chunk, n - base);
    if (base + chunk < n) {
      issue(which ^ 1, base + chunk);
      asm volatile("cp.async.wait_group 1;\n" ::);
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::);
    }
    __syncthreads();
    const float* buf = stage + (size_t)which * chunk * per_token;
#pragma unroll 2
    for (int i = 0; i < count; ++i) {
      const float* tok = buf + (size_t)i * per_token;
      const float4 bv = *reinterpret_cast<const float4*>(tok + row_first);
      const float4 cv = *reinterpret_cast<const float4*>(tok + NP + row_first);
      const float4 xv = *reinterpret_cast<const float4*>(tok + 2 * NP + col_local);
      const float decay = tok[2 * NP + cols], dt = tok[2 * NP + cols + 1];
      const float bm[4] = {bv.x, bv.y, bv.z, bv.w}, cm[4] = {cv.x, cv.y, cv.z, cv.w};
      const float x[4] = {xv.x, xv.y, xv.z, xv.w};
      float y[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float push = dt * x[q];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          s[r][q] = fmaf(push, bm[r], decay * s[r][q]);
          y[q] = fmaf(s[r][q], cm[r], y[q]);
        }
      }
      // lanes with an odd rg go on with columns 2, 3, the others with 0, 1; then one column each
      const float t0 = __shfl_xor_sync(0xffffffffu, low1 ? y[0] : y[2], 1);
      const float t1 = __shfl_xor_sync(0xffffffffu, low1 ? y[1] : y[3], 1);
      const float a0 = (low1 ? y[2] : y[0]) + t0, a1 = (low1 ? y[3] : y[1]) + t1;
      const float t2 = __shfl_xor_sync(0xffffffffu, low2 ? a0 : a1, 2);
      float v = (low2 ? a1 : a0) + t2;
#pragma unroll
      for (int o = 4; o < RG; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      const int q_mine = (low1 ? 2 : 0) + (low2 ? 1 : 0);
      if (rg < 4 && col_first + q_mine < dv) {
        const float xq = low1 ? (low2 ? x[3] : x[2]) : (low2 ? x[1] : x[0]);
        out[((size_t)(first + base + i) * H + h) * dv + col_first + q_mine] = fmaf(d_skip, xq, v);
      }
    }
    __syncthreads();
  }
  if (owns_slot(slots, b)) {
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int q = 0; q < 4; ++q)
        if (row_first + r < N && col_first + q < dv) S[(size_t)(row_first + r) * dv + col_first + q] = s[r][q];
  }
}

// scratch: float32 [T, H, 2].
extern "C" int sb_state_space_scan(const float* xbc, int C, const void* pre, int pre_width, int dtype,
                                   int step_offset, const float* step_bias, const float* neg_rate,
                                   const float* skip, float* state, const int* cu_q, const int* slots,
                                   int num_tokens, int num_seqs, int num_slots, int H, int G, int N, int dv,
                                   int max_q_len, float* scratch, float* out, int* err, cudaStream_t stream) {
  if (num_seqs == 0 || num_tokens == 0) return 0;
  if (N <= 0 || N > 1024 || dv <= 0 || H <= 0 || G <= 0 || H % G) return -13;
  const long long total = (long long)num_tokens * H;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == SB_DTYPE_F32)
    sb_launch(state_space_steps_kernel<float>, blocks, 256, 0, stream, (const float*)pre, pre_width, step_offset,
              step_bias, neg_rate, H, total, scratch);
  else
    sb_launch(state_space_steps_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)pre, pre_width, step_offset,
              step_bias, neg_rate, H, total, scratch);
  SB_LAUNCH_CHECK();
  const bool long_walk = max_q_len >= 64;
  if (long_walk && N >= 16 && N <= 128) {
    int rg = 4;
    while (rg * 4 < N) rg <<= 1;
    int chunk = 16;
    const int warps = 4, cols = warps * (32 / rg) * 4;
    const dim3 grid(H, num_seqs, (dv + cols - 1) / cols);
    const size_t smem = (size_t)2 * chunk * (2 * rg * 4 + cols + 4) * sizeof(float);
#define SB_SS_PATCH(RG_)                                                                                       \
  do {                                                                                                         \
    if (smem > 48 * 1024)                                                                                      \
      cudaFuncSetAttribute(state_space_patch_kernel<RG_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    sb_launch_plain(state_space_patch_kernel<RG_>, grid, warps * 32, smem, stream, xbc, C, scratch, skip, state, \
                    cu_q, slots, num_slots, H, G, N, dv, chunk, out, err);                                     \
  } while (0)
    switch (rg) {
      case 4: SB_SS_PATCH(4); break;
      case 8: SB_SS_PATCH(8); break;
      case 16: SB_SS_PATCH(16); break;
      default: SB_SS_PATCH(32); break;
    }
#undef SB_SS_PATCH
    SB_LAUNCH_CHECK();
    return 0;
  }
  const int rows = N <= 256 ? 8 : 32;
  int rs = 1;
  while (rs * rows < N) rs <<= 1;
  const int threads = long_walk ? 128 : 64;
  int chunk = 1;
  while (chunk < 16 && chunk < max_q_len) chunk <<= 1;
  int cols = threads / rs;
  if (cols < 1) cols = 1;
  if (cols > dv) cols = dv;
  const int block = ((cols * rs + 31) / 32) * 32;
  const dim3 grid(H, num_seqs, (dv + cols - 1) / cols);
  const size_t smem = (size_t)2 * chunk * (2 * ((N + 3) & ~3) + ((cols + 3) & ~3) + 4) * sizeof(float);
  if (smem > 200 * 1024) return -13;
#define SB_SS_SCAN(RS_, ROWS_)                                                                                 \
  do {                                                                                                         \
    if (smem > 48 * 1024)                                                                                      \
      cudaFuncSetAttribute(state_space_scan_kernel<RS_, ROWS_>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                           (int)smem);                                                                         \
    if (long_walk)                                                                                             \
      sb_launch_plain(state_space_scan_kernel<RS_, ROWS_>, grid, block, smem, stream, xbc, C, scratch, skip,   \
                      state, cu_q, slots, num_slots, H, G, N, dv, cols, chunk, out, err);                      \
    else                                                                                                       \
      sb_launch(state_space_scan_kernel<RS_, ROWS_>, grid, block, smem, stream, xbc, C, scratch, skip, state,  \
                cu_q, slots, num_slots, H, G, N, dv, cols, chunk, out, err);                                   \
  } while (0)
#define SB_SS(RS_)                               \
  do {                                           \
    if (rows == 8) SB_SS_SCAN(RS_, 8);           \
    else SB_SS_SCAN(RS_, 32);                    \
  } while (0)
  switch (rs) {
    case 1: SB_SS(1); break;
    case 2: SB_SS(2); break;
    case 4: SB_SS(4); break;
    case 8: SB_SS(8); break;
    case 16: SB_SS(16); break;
    default: SB_SS(32); break;
  }
#undef SB_SS
#undef SB_SS_SCAN
  SB_LAUNCH_CHECK();
  return 0;
}
