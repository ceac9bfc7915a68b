// Attention over latents: what happens between the projections and the attention kernel.
//
//   prepare   down [T, down_width] = c_q (Rq) | c (Rkv) | k_r (Dr) | ... as projected.
//             c_q' = c_q * rsqrt(mean c_q^2 + eps) * n_q          -> cq [T, Rq] (storage type)
//             c'   = c * rsqrt(mean c^2 + eps) * n_kv,  k_r' = turn(k_r, position)
//             the token's row [c' | k_r'] -> its place in the paged cache (one row per token)
//   queries   the rotated part of every head's query, turned and scaled, into its place behind
//             the head's vector over the latent:  asked[t, h, Rkv + i] = scale * turn(q[t, h, D + i])
//
// turn(x, p): dims i and i + n of the first 2 n dims become (a cos - b sin, b cos + a sin) with the
// angle p * freq[i], in float32 with sincosf; the other dims pass.  One block per token.
#include "common.cuh"

template <typename T>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const T* __restrict__ down, int down_width, const float* __restrict__ q_norm,
                      const float* __restrict__ kv_norm, float eps, const float* __restrict__ freq, int half,
                      int q_rank, int kv_rank, int rot_dim, const int* __restrict__ positions,
                      const int* __restrict__ token_seq, const int* __restrict__ block_table, int max_pages,
                      int page_size, int num_pages, T* __restrict__ cache, T* __restrict__ cq, int* err) {
  __shared__ float scratch[33];
  pdl_wait_block();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const T* row = down + (size_t)t * down_width;
  float sq = 0.f;
  for (int c = threadIdx.x; c < q_rank; c += blockDim.x) {
    const float v = to_f32<T>(row[c]);
    sq = fmaf(v, v, sq);
  }
  const float inv_q = rsqrtf(block_sum(sq, scratch) / (float)q_rank + eps);
  for (int c = threadIdx.x; c < q_rank; c += blockDim.x)
    cq[(size_t)t * q_rank + c] = from_f32<T>(to_f32<T>(row[c]) * inv_q * q_norm[c]);
  if (cache == nullptr) return;
  sq = 0.f;
  for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) {
    const float v = to_f32<T>(row[q_rank + c]);
    sq = fmaf(v, v, sq);
  }
  const float inv_kv = rsqrtf(block_sum(sq, scratch) / (float)kv_rank + eps);
  const int pos = positions[t], b = token_seq[t];
  const long long page = block_table[(size_t)b * max_pages + pos / page_size];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(err, SB_ERR_BAD_PAGE);
    return;
  }
  const int row_dim = kv_rank + rot_dim;
  T* dst = cache + ((size_t)page * page_size + pos % page_size) * row_dim;
  for (int c = threadIdx.x; c < kv_rank; c += blockDim.x)
    dst[c] = from_f32<T>(to_f32<T>(row[q_rank + c]) * inv_kv * kv_norm[c]);
  const T* kr = row + q_rank + kv_rank;
  for (int i = threadIdx.x; i < rot_dim; i += blockDim.x) {
    float v = to_f32<T>(kr[i]);
    if (i < 2 * half) {
      const int j = i < half ? i : i - half;
      float sn, cs;
      sincosf((float)pos * freq[j], &sn, &cs);
      const float a = to_f32<T>(kr[j]), bb = to_f32<T>(kr[j + half]);
      v = i < half ? a * cs - bb * sn : bb * cs + a * sn;
    }
    dst[kv_rank + i] = from_f32<T>(v);
  }
}

extern "C" int sb_latent_prepare(const void* down, int down_width, int dtype, const float* q_norm,
                                 const float* kv_norm, float eps, const float* freq, int half, int q_rank,
                                 int kv_rank, int rot_dim, const int* positions, const int* token_seq,
                                 const int* block_table, int max_pages, int page_size, int num_pages, void* cache,
                                 void* cq, int num_tokens, int* err, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (2 * half > rot_dim || q_rank <= 0 || kv_rank <= 0) return -13;
  if (dtype == SB_DTYPE_F32)
    sb_launch(latent_prepare_kernel<float>, num_tokens, 256, 0, stream, (const float*)down, down_width, q_norm,
              kv_norm, eps, freq, half, q_rank, kv_rank, rot_dim, positions, token_seq, block_table, max_pages,
              page_size, num_pages, (float*)cache, (float*)cq, err);
  else
    sb_launch(latent_prepare_kernel<bf16>, num_tokens, 256, 0, stream, (const bf16*)down, down_width, q_norm,
              kv_norm, eps, freq, half, q_rank, kv_rank, rot_dim, positions, token_seq, block_table, max_pages,
              page_size, num_pages, (bf16*)cache, (bf16*)cq, err);
  SB_LAUNCH_CHECK();
  return 0;
}

// q [T, H, in_head] with the rotated part at in_offset; out [T, H, out_head] with it at out_offset.
template <typename T>
__global__ void __launch_bounds__(256)
turn_query_part_kernel(const T* __restrict__ q, int in_head, int in_offset, T* __restrict__ out, int out_head,
                       int out_offset, const float* __restrict__ freq, int half, int rot_dim, float scale,
                       const int* __restrict__ positions, int num_heads) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const float pos = (float)positions[t];
  for (int idx = threadIdx.x; idx < num_heads * rot_dim; idx += blockDim.x) {
    const int h = idx / rot_dim, i = idx - h * rot_dim;
    const T* src = q + ((size_t)t * num_heads + h) * in_head + in_offset;
    float v = to_f32<T>(src[i]);
    if (i < 2 * half) {
      const int j = i < half ? i : i - half;
      float sn, cs;
      sincosf(pos * freq[j], &sn, &cs);
      const float a = to_f32<T>(src[j]), b = to_f32<T>(src[j + half]);
      v = i < half ? a * cs - b * sn : b * cs + a * sn;
    }
    out[((size_t)t * num_heads + h) * out_head + out_offset + i] = from_f32<T>(v * scale);
  }
}

extern "C" int sb_turn_query_part(const void* q, int in_head, int in_offset, void* out, int out_head, int out_offset,
                                  int dtype, const float* freq, int half, int rot_dim, float scale,
                                  const int* positions, int num_tokens, int num_heads, cudaStream_t stream) {
  if (num_tokens == 0 || rot_dim == 0) return 0;
  if (2 * half > rot_dim) return -13;
  if (dtype == SB_DTYPE_F32)
    sb_launch(turn_query_part_kernel<float>, num_tokens, 256, 0, stream, (const float*)q, in_head, in_offset,
              (float*)out, out_head, out_offset, freq, half, rot_dim, scale, positions, num_heads);
  else
    sb_launch(turn_query_part_kernel<bf16>, num_tokens, 256, 0, stream, (const bf16*)q, in_head, in_offset,
              (bf16*)out, out_head, out_offset, freq, half, rot_dim, scale, positions, num_heads);
  SB_LAUNCH_CHECK();
  return 0;
}
