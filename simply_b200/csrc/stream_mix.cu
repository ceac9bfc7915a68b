// Kernels around a residual stream that is kept several times, and small per-token steps that
// several mixers share.  Everything computes in float32; T is the storage type of activations.
//
//   embedding with positions   out = table[id] * scale + positions[p]
//   streams step               x_t <- sum_s mix[s, t] x_s + out[t] y ;  u = sum_s in[s] x_s ;
//                              y' = u * rsqrt(mean(u^2) + eps) * w          one block per token
//   short convolution          y_c[t] = sum_j w[c, j] x_c[t - (K-1) + j] (+ b_c), inputs before the
//                              step's first token from the request's state; silu; x + y
//   group norm with a gate     per token, N numbers in equal groups, each divided by its root mean
//                              square, times w; a gate as silu before or as sigmoid after
//   tanh of a column range, experts by a table of token ids, a product per head
#include <type_traits>

#include "common.cuh"

#define SB_ERR_BAD_SLOT 16    // a state slot outside the state tensor
#define SB_ERR_BAD_EXPERT 32  // a table entry that names no expert
#define SB_MAX_STREAMS 8

__device__ __forceinline__ bool slot_written_by(const int* slots, int b) {
  // A decode graph pads its batch by repeating the last request: only the first row of a slot
  // writes the slot's state.
  const int slot = slots[b];
  for (int i = 0; i < b; ++i)
    if (slots[i] == slot) return false;
  return true;
}

// ---------------------------------------------------------------------------
template <typename T>
__global__ void embed_positions_kernel(const T* __restrict__ table, const T* __restrict__ pos_table,
                                       const int* __restrict__ ids, const int* __restrict__ positions, float scale,
                                       float* __restrict__ out, int width, int vocab, int max_positions, int* err) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(err, SB_ERR_BAD_TOKEN);
    id = 0;
  }
  int p = pos_table != nullptr ? positions[t] : 0;
  if (p < 0 || p >= max_positions) {
    if (threadIdx.x == 0 && pos_table != nullptr) atomicOr(err, SB_ERR_BAD_ROW);
    p = 0;
  }
  const T* row = table + (size_t)id * width;
  const T* prow = pos_table != nullptr ? pos_table + (size_t)p * width : nullptr;
  float* o = out + (size_t)t * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = to_f32<T>(row[i]) * scale;
    if (prow != nullptr) v += to_f32<T>(prow[i]);
    o[i] = v;
  }
}

extern "C" int sb_embed_positions(const void* table, const void* pos_table, int dtype, const int* ids,
                                  const int* positions, float scale, float* out, int num_tokens, int width,
                                  int vocab, int max_positions, int* err, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (dtype == SB_DTYPE_F32)
    sb_launch(embed_positions_kernel<float>, num_tokens, 256, 0, stream, (const float*)table,
              (const float*)pos_table, ids, positions, scale, out, width, vocab, max_positions, err);
  else
    sb_launch(embed_positions_kernel<bf16>, num_tokens, 256, 0, stream, (const bf16*)table, (const bf16*)pos_table,
              ids, positions, scale, out, width, vocab, max_positions, err);
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// lanes [T, S, W] float32 from h [T, W]
__global__ void spread_streams_kernel(const float* __restrict__ h, float* __restrict__ lanes, int copies, int width) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = h[(size_t)t * width + i];
    for (int s = 0; s < copies; ++s) lanes[((size_t)t * copies + s) * width + i] = v;
  }
}

extern "C" int sb_spread_streams(const float* h, float* lanes, int num_tokens, int copies, int width,
                                 cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  sb_launch(spread_streams_kernel, num_tokens, 256, 0, stream, h, lanes, copies, width);
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// One block per row.  With `rows`, block r works on row rows[r], writes y[r] and leaves the lanes.
// S_: the number of copies where the launch knows it at compile time (1 to 4), else 0.
template <typename T, int S_>
__global__ void streams_step_kernel(float* __restrict__ lanes, const T* __restrict__ branch,
                                    const float* __restrict__ mix, const float* __restrict__ out_w,
                                    const float* __restrict__ in_w, const void* __restrict__ norm_w, int norm_f32,
                                    float eps, int plus_one, const int* __restrict__ rows, T* __restrict__ y,
                                    float* __restrict__ y_sum, int copies, int width, int num_rows_total, int* err) {
  extern __shared__ float row[];  // width floats + 33 scratch
  float* scratch = row + width;
  __shared__ float s_mix[SB_MAX_STREAMS * SB_MAX_STREAMS], s_out[SB_MAX_STREAMS], s_in[SB_MAX_STREAMS];
  // the small matrices are weights: fetched before the wait for the kernel before
  if (threadIdx.x < copies * copies && branch != nullptr) s_mix[threadIdx.x] = mix[threadIdx.x];
  if (threadIdx.x < copies) {
    s_out[threadIdx.x] = branch != nullptr ? out_w[threadIdx.x] : 0.f;
    s_in[threadIdx.x] = in_w != nullptr ? in_w[threadIdx.x] : 0.f;
  }
  pdl_wait_block();
  pdl_launch_dependents();
  constexpr int MAXS = S_ > 0 ? S_ : SB_MAX_STREAMS;
  if (S_ > 0) copies = S_;
  int r = blockIdx.x;
  if (rows != nullptr) {
    r = rows[blockIdx.x];
    if (r < 0 || r >= num_rows_total) {
      if (threadIdx.x == 0) atomicOr(err, SB_ERR_BAD_ROW);
      r = 0;
    }
  }
  float* x = lanes + (size_t)r * copies * width;
  float sq = 0.f;
  // V neighbouring columns per thread and turn, every copy's V values fetched at once (16 bytes when
  // the width allows) before anything is written: a row's columns are a few turns of independent
  // fetches, not a chain of fetch, compute, store per column.
  auto columns = [&](auto vtag, int c) {
    constexpr int V = decltype(vtag)::value;
    float old[MAXS][V], now[MAXS][V], b[V];
#pragma unroll
    for (int s = 0; s < MAXS; ++s) {
      if (s < copies) {
        if constexpr (V == 4) {
          const float4 v = *reinterpret_cast<const float4*>(x + (size_t)s * width + c);
          old[s][0] = v.x; old[s][1] = v.y; old[s][2] = v.z; old[s][3] = v.w;
        } else {
          old[s][0] = x[(size_t)s * width + c];
        }
      } else {
#pragma unroll
        for (int e = 0; e < V; ++e) old[s][e] = 0.f;
      }
    }
    if (branch != nullptr) {
#pragma unroll
      for (int e = 0; e < V; ++e) b[e] = to_f32<T>(branch[(size_t)r * width + c + e]);
#pragma unroll
      for (int t = 0; t < MAXS; ++t) {
        if (t < copies) {
#pragma unroll
          for (int e = 0; e < V; ++e) {
            float acc = 0.f;
#pragma unroll
            for (int s = 0; s < MAXS; ++s)
              if (s < copies) acc = fmaf(s_mix[s * copies + t], old[s][e], acc);
            now[t][e] = fmaf(s_out[t], b[e], acc);
          }
          if (rows == nullptr) {
            if constexpr (V == 4)
              *reinterpret_cast<float4*>(x + (size_t)t * width + c) = make_float4(now[t][0], now[t][1], now[t][2], now[t][3]);
            else
              x[(size_t)t * width + c] = now[t][0];
          }
        }
      }
    } else {
#pragma unroll
      for (int s = 0; s < MAXS; ++s)
#pragma unroll
        for (int e = 0; e < V; ++e) now[s][e] = old[s][e];
    }
    if (in_w != nullptr) {
#pragma unroll
      for (int e = 0; e < V; ++e) {
        float u = 0.f;
#pragma unroll
        for (int s = 0; s < MAXS; ++s)
          if (s < copies) u = fmaf(s_in[s], now[s][e], u);
        row[c + e] = u;
        sq = fmaf(u, u, sq);
      }
    }
  };
  if (S_ > 0 && (width & 3) == 0) {
    for (int c = threadIdx.x * 4; c < width; c += blockDim.x * 4) columns(std::integral_constant<int, 4>{}, c);
  } else {
    for (int c = threadIdx.x; c < width; c += blockDim.x) columns(std::integral_constant<int, 1>{}, c);
  }
  if (in_w == nullptr) return;
  if (norm_w == nullptr) {
    __syncthreads();
    for (int c = threadIdx.x; c < width; c += blockDim.x) y_sum[(size_t)blockIdx.x * width + c] = row[c];
    return;
  }
  const float total = block_sum(sq, scratch);
  const float inv = rsqrtf(total / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float w = load_scalar(norm_w, norm_f32, c) + (plus_one ? 1.0f : 0.f);
    y[(size_t)blockIdx.x * width + c] = from_f32<T>(row[c] * inv * w);
  }
}

extern "C" int sb_streams_step(float* lanes, const void* branch, int dtype, const float* mix, const float* out_w,
                               const float* in_w, const void* norm_w, int norm_f32, float eps, int plus_one,
                               const int* rows, int num_rows, void* y, float* y_sum, int copies, int width,
                               int num_rows_total, int* err, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  if (copies < 1 || copies > SB_MAX_STREAMS) return -13;
  const size_t smem = ((size_t)width + 33) * sizeof(float);
  if (smem > 200 * 1024) return -13;
  const int threads = width >= 1024 ? 256 : 128;
#define SB_STREAMS(T_, S__)                                                                                           \
  do {                                                                                                           \
    if (smem > 48 * 1024)                                                                                        \
      cudaFuncSetAttribute(streams_step_kernel<T_, S__>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
    sb_launch(streams_step_kernel<T_, S__>, num_rows, threads, smem, stream, lanes, (const T_*)branch, mix, out_w, \
              in_w, norm_w, norm_f32, eps, plus_one, rows, (T_*)y, y_sum, copies, width, num_rows_total, err);   \
  } while (0)
#define SB_STREAMS_OF(S__)                       \
  do {                                           \
    if (dtype == SB_DTYPE_F32) SB_STREAMS(float, S__); \
    else SB_STREAMS(bf16, S__);                  \
  } while (0)
  switch (copies) {
    case 1: SB_STREAMS_OF(1); break;
    case 2: SB_STREAMS_OF(2); break;
    case 3: SB_STREAMS_OF(3); break;
    case 4: SB_STREAMS_OF(4); break;
    default: SB_STREAMS_OF(0); break;
  }
#undef SB_STREAMS_OF
#undef SB_STREAMS
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// Short causal convolution.  x [T, x_width] (columns offset .. offset + C), weight [C, K] float32,
// state [slots, K - 1, C] float32 (the last K - 1 inputs of every request), out [T, C].
// Grid (token, channel tiles).
template <typename T>
__global__ void __launch_bounds__(256)
short_conv_kernel(const T* __restrict__ x, int x_width, int offset, const float* __restrict__ weight,
                  const float* __restrict__ bias, const float* __restrict__ state, const int* __restrict__ token_seq,
                  const int* __restrict__ cu_q, const int* __restrict__ slots, int num_slots, int taps, int channels,
                  int act, int residual, int out_f32, void* __restrict__ out, int* err) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int b = token_seq[t];
  const int i = t - cu_q[b];  // place among the step's tokens of this request
  const int slot = slots[b];
  if (taps > 1 && (slot < 0 || slot >= num_slots)) {
    if (threadIdx.x == 0) atomicOr(err, SB_ERR_BAD_SLOT);
    return;
  }
  const float* st = taps > 1 ? state + (size_t)slot * (taps - 1) * channels : nullptr;
  float acc = bias != nullptr ? bias[c] : 0.f;
  const float* w = weight + (size_t)c * taps;
  for (int j = 0; j < taps; ++j) {
    const int at = i - (taps - 1) + j;  // relative to the step's first token
    const float v = at >= 0 ? to_f32<T>(x[(size_t)(t - i + at) * x_width + offset + c])
                            : st[(size_t)(taps - 1 + at) * channels + c];
    acc = fmaf(w[j], v, acc);
  }
  if (act == 1) acc = acc / (1.0f + expf(-acc));
  if (residual) acc += to_f32<T>(x[(size_t)t * x_width + offset + c]);
  if (out_f32) reinterpret_cast<float*>(out)[(size_t)t * channels + c] = acc;
  else reinterpret_cast<T*>(out)[(size_t)t * channels + c] = from_f32<T>(acc);
}

// The state after the step: the last K - 1 rows of (state, the step's inputs).  One thread per
// (sequence, channel), rows ascending, so that it reads only what it has not yet written.
template <typename T>
__global__ void short_conv_state_kernel(const T* __restrict__ x, int x_width, int offset, float* __restrict__ state,
                                        const int* __restrict__ cu_q, const int* __restrict__ slots, int num_slots,
                                        int taps, int channels) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int b = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int slot = slots[b];
  if (slot < 0 || slot >= num_slots || !slot_written_by(slots, b)) return;
  const int first = cu_q[b], n = cu_q[b + 1] - first;
  float* st = state + (size_t)slot * (taps - 1) * channels;
  for (int r = 0; r < taps - 1; ++r) {
    const int at = n + r;  // row of (state, inputs)
    st[(size_t)r * channels + c] = at < taps - 1 ? st[(size_t)at * channels + c]
                                                 : to_f32<T>(x[(size_t)(first + at - (taps - 1)) * x_width + offset + c]);
  }
}

extern "C" int sb_short_conv(const void* x, int x_width, int offset, int dtype, const float* weight,
                             const float* bias, float* state, const int* token_seq, const int* cu_q,
                             const int* slots, int num_tokens, int num_seqs, int num_slots, int taps, int channels,
                             int act, int residual, int out_f32, void* out, int* err, cudaStream_t stream) {
  if (num_tokens == 0 || channels == 0) return 0;
  if (taps < 1 || (taps > 1 && state == nullptr)) return -13;
  const int threads = channels >= 256 ? 256 : ((channels + 31) / 32) * 32;
  const unsigned tiles = (unsigned)((channels + threads - 1) / threads);
  if (tiles > 65535) return -13;
#define SB_CONV(T_)                                                                                                \
  do {                                                                                                             \
    sb_launch(short_conv_kernel<T_>, dim3((unsigned)num_tokens, tiles), threads, 0, stream, (const T_*)x, x_width, \
              offset, weight, bias, (const float*)state, token_seq, cu_q, slots, num_slots, taps, channels, act,   \
              residual, out_f32, out, err);                                                                        \
    if (taps > 1)                                                                                                  \
      sb_launch(short_conv_state_kernel<T_>, dim3((unsigned)num_seqs, tiles), threads, 0, stream, (const T_*)x,    \
                x_width, offset, state, cu_q, slots, num_slots, taps, channels);                                   \
  } while (0)
  if (dtype == SB_DTYPE_F32) SB_CONV(float);
  else SB_CONV(bf16);
#undef SB_CONV
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// Group norm with a gate.  o [T, N] float32; gate [T, gate_width] of T at gate_offset (null: none).
// gate_kind 1: sigmoid after the norm; 2: silu before it.  Grid (token, group).
template <typename T>
__global__ void __launch_bounds__(256)
group_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ gate, int gate_width, int gate_offset,
                       int gate_kind, const float* __restrict__ weight, float eps, int n, int groups,
                       T* __restrict__ out) {
  __shared__ float scratch[33];
  pdl_wait_block();
  pdl_launch_dependents();
  const int t = blockIdx.x, g = blockIdx.y;
  const int size = n / groups, c0 = g * size;
  const float* row = o + (size_t)t * n + c0;
  const T* grow = gate != nullptr ? gate + (size_t)t * gate_width + gate_offset + c0 : nullptr;
  float sq = 0.f;
  for (int c = threadIdx.x; c < size; c += blockDim.x) {
    float v = row[c];
    if (gate_kind == 2) {
      const float z = to_f32<T>(grow[c]);
      v *= z / (1.0f + expf(-z));
    }
    sq = fmaf(v, v, sq);
  }
  const float inv = rsqrtf(block_sum(sq, scratch) / (float)size + eps);
  for (int c = threadIdx.x; c < size; c += blockDim.x) {
    float v = row[c];
    if (gate_kind == 2) {
      const float z = to_f32<T>(grow[c]);
      v *= z / (1.0f + expf(-z));
    }
    v = v * inv * weight[c0 + c];
    if (gate_kind == 1) v /= 1.0f + expf(-to_f32<T>(grow[c]));
    out[(size_t)t * n + c0 + c] = from_f32<T>(v);
  }
}

extern "C" int sb_group_norm_gate(const float* o, const void* gate, int gate_width, int gate_offset, int gate_kind,
                                  int dtype, const float* weight, float eps, int num_tokens, int n, int groups,
                                  void* out, cudaStream_t stream) {
  if (num_tokens == 0 || n == 0) return 0;
  if (groups < 1 || n % groups || groups > 65535 || (gate_kind != 0 && gate == nullptr)) return -13;
  const int size = n / groups;
  const int threads = size >= 256 ? 256 : ((size + 31) / 32) * 32;
  const dim3 grid((unsigned)num_tokens, (unsigned)groups);
  if (dtype == SB_DTYPE_F32)
    sb_launch(group_norm_gate_kernel<float>, grid, threads, 0, stream, o, (const float*)gate, gate_width,
              gate_offset, gate_kind, weight, eps, n, groups, (float*)out);
  else
    sb_launch(group_norm_gate_kernel<bf16>, grid, threads, 0, stream, o, (const bf16*)gate, gate_width, gate_offset,
              gate_kind, weight, eps, n, groups, (bf16*)out);
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
template <typename T>
__global__ void tanh_columns_kernel(const T* __restrict__ x, int x_width, int offset, int n, T* __restrict__ out,
                                    long long total) {
  pdl_wait_block();
  pdl_launch_dependents();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / n;
    const int c = (int)(i - t * n);
    out[i] = from_f32<T>(tanhf(to_f32<T>(x[t * x_width + offset + c])));
  }
}

extern "C" int sb_tanh_columns(const void* x, int x_width, int offset, int n, int dtype, void* out, int num_tokens,
                               cudaStream_t stream) {
  const long long total = (long long)num_tokens * n;
  if (total == 0) return 0;
  const int blocks = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
  if (dtype == SB_DTYPE_F32)
    sb_launch(tanh_columns_kernel<float>, blocks, 256, 0, stream, (const float*)x, x_width, offset, n, (float*)out, total);
  else
    sb_launch(tanh_columns_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)x, x_width, offset, n, (bf16*)out, total);
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// Experts by a table of token ids: chosen[t, j] = table[id_t, j], weight 1 / top.
__global__ void table_route_kernel(const int* __restrict__ ids, const int* __restrict__ table, int vocab, int top,
                                   int num_experts, int* __restrict__ chosen, float* __restrict__ weight, int pairs,
                                   int* err) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= pairs) return;
  const int t = p / top, j = p - t * top;
  int id = ids[t];
  if (id < 0 || id >= vocab) {
    atomicOr(err, SB_ERR_BAD_TOKEN);
    id = 0;
  }
  int e = table[(size_t)id * top + j];
  if (e < 0 || e >= num_experts) {
    atomicOr(err, SB_ERR_BAD_EXPERT);
    e = 0;
  }
  chosen[p] = e;
  weight[p] = 1.0f / (float)top;
}

extern "C" int sb_table_route(const int* ids, const int* table, int vocab, int top, int num_experts, int* chosen,
                              float* weight, int num_tokens, int* err, cudaStream_t stream) {
  const int pairs = num_tokens * top;
  if (pairs == 0) return 0;
  sb_launch(table_route_kernel, (pairs + 255) / 256, 256, 0, stream, ids, table, vocab, top, num_experts, chosen,
            weight, pairs, err);
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// A product per head: out[t, h, :] = alpha * w[h] x[t, h, :], w [H, Dout, Din], x rows of
// x_stride numbers with head h at h * x_head + x_offset, out rows of out_stride numbers with head h
// at h * out_head.  Tiles of 32 tokens x 32 outputs, k in steps of 32 in a fixed order, so a
// token's result does not depend on the step's other tokens.
#define HL_TM 32
#define HL_TN 32
#define HL_TK 32
template <typename T>
__global__ void __launch_bounds__(256)
head_linear_kernel(const T* __restrict__ x, int x_stride, int x_head, int x_offset, const T* __restrict__ w,
                   int d_in, int d_out, T* __restrict__ out, int out_stride, int out_head, float alpha,
                   int num_tokens) {
  __shared__ float xs[HL_TM][HL_TK + 1], ws[HL_TN][HL_TK + 1];
  pdl_wait_block();
  pdl_launch_dependents();
  const int h = blockIdx.y, t0 = blockIdx.x * HL_TM, n0 = blockIdx.z * HL_TN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // outputs tx, tx + 16; tokens ty, ty + 16
  const T* wh = w + (size_t)h * d_out * d_in;
  float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  for (int k0 = 0; k0 < d_in; k0 += HL_TK) {
    for (int idx = threadIdx.x; idx < HL_TM * HL_TK; idx += 256) {
      const int r = idx / HL_TK, c = idx - r * HL_TK;
      const int t = t0 + r, k = k0 + c;
      xs[r][c] = (t < num_tokens && k < d_in) ? to_f32<T>(x[(size_t)t * x_stride + (size_t)h * x_head + x_offset + k]) : 0.f;
      const int n = n0 + r;
      ws[r][c] = (n < d_out && k < d_in) ? to_f32<T>(wh[(size_t)n * d_in + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < HL_TK; ++c) {
      const float a0 = xs[ty][c], a1 = xs[ty + 16][c], b0 = ws[tx][c], b1 = ws[tx + 16][c];
      acc[0][0] = fmaf(a0, b0, acc[0][0]);
      acc[0][1] = fmaf(a0, b1, acc[0][1]);
      acc[1][0] = fmaf(a1, b0, acc[1][0]);
      acc[1][1] = fmaf(a1, b1, acc[1][1]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int t = t0 + ty + 16 * i, n = n0 + tx + 16 * j;
      if (t < num_tokens && n < d_out)
        out[(size_t)t * out_stride + (size_t)h * out_head + n] = from_f32<T>(alpha * acc[i][j]);
    }
}

extern "C" int sb_head_linear(const void* x, int x_stride, int x_head, int x_offset, const void* w, int dtype,
                              int num_heads, int d_in, int d_out, void* out, int out_stride, int out_head,
                              float alpha, int num_tokens, cudaStream_t stream) {
  if (num_tokens == 0 || num_heads == 0 || d_out == 0) return 0;
  if (num_heads > 65535 || (d_out + HL_TN - 1) / HL_TN > 65535) return -13;
  const dim3 grid((unsigned)((num_tokens + HL_TM - 1) / HL_TM), (unsigned)num_heads, (unsigned)((d_out + HL_TN - 1) / HL_TN));
  if (dtype == SB_DTYPE_F32)
    sb_launch(head_linear_kernel<float>, grid, 256, 0, stream, (const float*)x, x_stride, x_head, x_offset,
              (const float*)w, d_in, d_out, (float*)out, out_stride, out_head, alpha, num_tokens);
  else
    sb_launch(head_linear_kernel<bf16>, grid, 256, 0, stream, (const bf16*)x, x_stride, x_head, x_offset,
              (const bf16*)w, d_in, d_out, (bf16*)out, out_stride, out_head, alpha, num_tokens);
  SB_LAUNCH_CHECK();
  return 0;
}
