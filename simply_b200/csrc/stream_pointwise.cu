// Steps on the residual stream and on rows of activations that need no sum over a row.
//
//   scaled_residual_tanh   h += s1 * b1 + s2 * b2 (a learned factor per channel on each branch; a
//                          branch without factors is added as it is), then y = tanh(alpha h) w + b
//                          for the next reader: the counterpart of the fused residual + RMS norm
//                          kernel for a norm that computes no statistics.  With `rows`, row r of y
//                          comes from row rows[r] of h and h is left as it is.
//   pack_pair              out[t] = [a[t], b[t]] in the activation dtype, from two float32 rows
//   add_row                y[t] += row (float32)
//   xielu                  z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z/2,
//                          p and q read from the device, both softplus in float32
//   scale_values           x *= c (float32)
//
// The stream h is float32; T is the storage type of the branches and of y.
#include "common.cuh"

template <typename T>
__global__ void __launch_bounds__(256)
scaled_residual_tanh_kernel(float* __restrict__ h, const T* __restrict__ b1, const float* __restrict__ s1,
                            const T* __restrict__ b2, const float* __restrict__ s2,
                            const float* __restrict__ alpha, const float* __restrict__ w,
                            const float* __restrict__ bias, const int* __restrict__ rows, T* __restrict__ y,
                            int width, int num_rows_total, int* err) {
  // A thread owns one 16-byte vector of the branches' and the result's storage type: 4 channels
  // in float32, 8 in bfloat16 (two vectors of the stream).  The factors and the norm's vectors
  // are weights: fetched before the wait for the inputs.
  constexpr int N = Vec<T>::N;
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * N;
  const bool on = c0 < width;
  const bool vec = width % N == 0;
  float f1[N], f2[N], wv[N], bv[N];
#pragma unroll
  for (int k = 0; k < N; ++k) { f1[k] = f2[k] = 1.f; wv[k] = bv[k] = 0.f; }
  const float a = alpha != nullptr ? alpha[0] : 0.f;
  if (on) {
    if (vec) {
      if (b1 != nullptr && s1 != nullptr) load_scalars<N>(s1, 1, c0, f1);
      if (b2 != nullptr && s2 != nullptr) load_scalars<N>(s2, 1, c0, f2);
      if (y != nullptr) { load_scalars<N>(w, 1, c0, wv); load_scalars<N>(bias, 1, c0, bv); }
    } else {
#pragma unroll
      for (int k = 0; k < N; ++k) {
        if (c0 + k < width) {
          if (b1 != nullptr && s1 != nullptr) f1[k] = s1[c0 + k];
          if (b2 != nullptr && s2 != nullptr) f2[k] = s2[c0 + k];
          if (y != nullptr) { wv[k] = w[c0 + k]; bv[k] = bias[c0 + k]; }
        }
      }
    }
  }
  pdl_wait_block();
  pdl_launch_dependents();
  if (!on) return;
  const int r = blockIdx.y;
  int src = rows ? rows[r] : r;
  if (src < 0 || src >= num_rows_total) {
    if (threadIdx.x == 0) atomicOr(err, SB_ERR_BAD_ROW);
    src = 0;
  }
  const size_t at = (size_t)src * width + c0;
  float* hp = h + at;
  float v[N], x1[N], x2[N];
#pragma unroll
  for (int k = 0; k < N; ++k) v[k] = x1[k] = x2[k] = 0.f;
  // every load is issued before the first sum
  if (vec) {
#pragma unroll
    for (int k = 0; k < N; k += 4) Vec<float>::load(hp + k, v + k);
    if (b1 != nullptr) Vec<T>::load(b1 + at, x1);
    if (b2 != nullptr) Vec<T>::load(b2 + at, x2);
  } else {
#pragma unroll
    for (int k = 0; k < N; ++k) {
      if (c0 + k < width) {
        v[k] = hp[k];
        if (b1 != nullptr) x1[k] = to_f32<T>(b1[at + k]);
        if (b2 != nullptr) x2[k] = to_f32<T>(b2[at + k]);
      }
    }
  }
  const bool adds = b1 != nullptr || b2 != nullptr;
  if (adds) {
    // (the sum of the branches first, then the stream: one order whatever the step holds)
#pragma unroll
    for (int k = 0; k < N; ++k) v[k] += fmaf(f2[k], x2[k], f1[k] * x1[k]);
    if (rows == nullptr) {
      if (vec) {
#pragma unroll
        for (int k = 0; k < N; k += 4) Vec<float>::store(hp + k, v + k);
      } else {
#pragma unroll
        for (int k = 0; k < N; ++k)
          if (c0 + k < width) hp[k] = v[k];
      }
    }
  }
  if (y != nullptr) {
    T* yp = y + (size_t)r * width + c0;
    float out[N];
#pragma unroll
    for (int k = 0; k < N; ++k) out[k] = fmaf(tanhf(a * v[k]), wv[k], bv[k]);
    if (vec) {
      Vec<T>::store(yp, out);
    } else {
#pragma unroll
      for (int k = 0; k < N; ++k)
        if (c0 + k < width) yp[k] = from_f32<T>(out[k]);
    }
  }
}

extern "C" int sb_scaled_residual_tanh(float* h, const void* b1, const float* s1, const void* b2, const float* s2,
                                       int dtype, const float* alpha, const float* w, const float* bias,
                                       const int* rows, void* y, int num_rows, int width, int num_rows_total,
                                       int* err, cudaStream_t stream) {
  if (num_rows == 0 || width == 0) return 0;
  if (y != nullptr && (alpha == nullptr || w == nullptr || bias == nullptr)) return -13;
  const int per = dtype == SB_DTYPE_F32 ? 4 : 8;  // channels per thread: one 16-byte vector of T
  const int lanes = (width + per - 1) / per;
  const int threads = lanes >= 256 ? 256 : (lanes + 31) / 32 * 32;
  const unsigned gx = (unsigned)((lanes + threads - 1) / threads);
  for (int r0 = 0; r0 < num_rows; r0 += 65535) {
    const int n = min(65535, num_rows - r0);
    const dim3 grid(gx, (unsigned)n);
    // (a chunk beyond the first works on its own rows: without `rows` the pointers move on)
    const size_t off = rows ? 0 : (size_t)r0 * width;
    if (dtype == SB_DTYPE_F32)
      sb_launch(scaled_residual_tanh_kernel<float>, grid, threads, 0, stream, h + off,
                b1 ? (const float*)b1 + off : nullptr, s1, b2 ? (const float*)b2 + off : nullptr, s2, alpha, w, bias,
                rows ? rows + r0 : nullptr, y ? (float*)y + (size_t)r0 * width : nullptr, width,
                rows ? num_rows_total : n, err);
    else
      sb_launch(scaled_residual_tanh_kernel<bf16>, grid, threads, 0, stream, h + off,
                b1 ? (const bf16*)b1 + off : nullptr, s1, b2 ? (const bf16*)b2 + off : nullptr, s2, alpha, w, bias,
                rows ? rows + r0 : nullptr, y ? (bf16*)y + (size_t)r0 * width : nullptr, width,
                rows ? num_rows_total : n, err);
  }
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
pack_pair_kernel(const float* __restrict__ a, const float* __restrict__ b, T* __restrict__ out, int width) {
  pdl_wait_block();
  pdl_launch_dependents();
  const size_t t = blockIdx.y;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < 2 * width; c += gridDim.x * blockDim.x) {
    const float v = c < width ? a[t * width + c] : b[t * width + c - width];
    out[t * 2 * width + c] = from_f32<T>(v);
  }
}

extern "C" int sb_pack_pair(const float* a, const float* b, void* out, int dtype, int num_rows, int width,
                            cudaStream_t stream) {
  if (num_rows == 0 || width == 0) return 0;
  for (int r0 = 0; r0 < num_rows; r0 += 65535) {
    const dim3 grid((unsigned)min((2 * width + 255) / 256, 64), (unsigned)min(65535, num_rows - r0));
    const size_t off = (size_t)r0 * width;
    if (dtype == SB_DTYPE_F32)
      sb_launch(pack_pair_kernel<float>, grid, 256, 0, stream, a + off, b + off, (float*)out + 2 * off, width);
    else
      sb_launch(pack_pair_kernel<bf16>, grid, 256, 0, stream, a + off, b + off, (bf16*)out + 2 * off, width);
  }
  SB_LAUNCH_CHECK();
  return 0;
}

__global__ void __launch_bounds__(256)
add_row_kernel(float* __restrict__ y, const float* __restrict__ row, int width) {
  pdl_wait_block();
  pdl_launch_dependents();
  const size_t t = blockIdx.y;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < width; c += gridDim.x * blockDim.x)
    y[t * width + c] += row[c];
}

extern "C" int sb_add_row(float* y, const float* row, int num_rows, int width, cudaStream_t stream) {
  if (num_rows == 0 || width == 0) return 0;
  for (int r0 = 0; r0 < num_rows; r0 += 65535) {
    const dim3 grid((unsigned)min((width + 255) / 256, 64), (unsigned)min(65535, num_rows - r0));
    sb_launch(add_row_kernel, grid, 256, 0, stream, y + (size_t)r0 * width, row, width);
  }
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
__device__ __forceinline__ float softplus_f32(float z) { return log1pf(expf(-fabsf(z))) + fmaxf(z, 0.f); }

template <typename T>
__global__ void __launch_bounds__(256)
xielu_kernel(const T* __restrict__ z, const float* __restrict__ act, T* __restrict__ out, long long n) {
  const float ap = softplus_f32(act[0]), an = 0.5f + softplus_f32(act[1]);  // (weights: before the wait)
  pdl_wait_block();
  pdl_launch_dependents();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float x = to_f32<T>(z[i]);
    const float r = x > 0.f ? fmaf(ap * x, x, 0.5f * x) : fmaf(an, expm1f(x) - x, 0.5f * x);
    out[i] = from_f32<T>(r);
  }
}

extern "C" int sb_xielu(const void* z, const float* act, void* out, int dtype, long long n, cudaStream_t stream) {
  if (n == 0) return 0;
  const unsigned blocks = (unsigned)min((n + 255) / 256, (long long)148 * 16);
  if (dtype == SB_DTYPE_F32)
    sb_launch(xielu_kernel<float>, blocks, 256, 0, stream, (const float*)z, act, (float*)out, n);
  else
    sb_launch(xielu_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)z, act, (bf16*)out, n);
  SB_LAUNCH_CHECK();
  return 0;
}

__global__ void __launch_bounds__(256)
scale_values_kernel(float* __restrict__ x, float c, long long n) {
  pdl_wait_block();
  pdl_launch_dependents();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    x[i] *= c;
}

extern "C" int sb_scale_values(float* x, float c, long long n, cudaStream_t stream) {
  if (n == 0) return 0;
  const unsigned blocks = (unsigned)min((n + 255) / 256, (long long)148 * 16);
  sb_launch(scale_values_kernel, blocks, 256, 0, stream, x, c, n);
  SB_LAUNCH_CHECK();
  return 0;
}
