// Latent attention keeps, per token, one row [c | k_rot]: a normed latent c of `rank` values from
// which every head's keys and values are linear maps, and `rd` rotated key values shared by all heads.
// With the key map folded into the query (q_lat = W_uk^T q_plain) the score of head h against a cached
// row is q_eff . row with q_eff = [q_lat | q_rot], and the head's output is W_uv applied to the
// softmax-weighted sum of the c parts: one cached row serves all heads, as keys and as values.
//
// This file holds the kernel that makes the cached row and the rotated query part from a token's
// projections; the attention over the rows is zi_paged_attention_v (attention_generic.cu) with one
// kv head whose values are the first `rank` columns of its keys.
#include "api.h"
#include "common.cuh"

namespace {
// One block per token.  src row: [q heads, each (dim plain | rd rotated)] [rank latent | rd key part].
// Rotary: of the rd values the first rot_dims are rotated (pairs (i, i + rot_dims/2)), the rest pass.
template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const T* __restrict__ src, int ld, int heads, int dim, int rd, int rank, int rot_dims,
                      const float* __restrict__ cw, float eps, const float* __restrict__ cos_t,
                      const float* __restrict__ sin_t, int n_table_pos, const int* __restrict__ positions,
                      T* __restrict__ q_eff, T* __restrict__ cache, const int* __restrict__ slots, int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const T* row = src + (size_t)t * ld;
  const int D = rank + rd, half = rot_dims / 2;
  int pos = positions[t];
  pos = pos < 0 ? 0 : (pos >= n_table_pos ? n_table_pos - 1 : pos);   // callers keep positions inside the table
  const float* cs = cos_t + (size_t)pos * half;
  const float* sn = sin_t + (size_t)pos * half;
  // the rotated part of every query head -> q_eff[t, h, rank ..]
  for (int e = threadIdx.x; e < heads * rd; e += blockDim.x) {
    const int h = e / rd, i = e - h * rd;
    const T* qr = row + (size_t)h * (dim + rd) + dim;
    float v = to_f32(qr[i]);
    if (i < half) {
      float x = v, y = to_f32(qr[i + half]);
      rotate_pair(x, y, cs[i], sn[i]);
      v = x;
    } else if (i < rot_dims) {
      float x = to_f32(qr[i - half]), y = v;
      rotate_pair(x, y, cs[i - half], sn[i - half]);
      v = y;
    }
    q_eff[((size_t)t * heads + h) * D + rank + i] = from_f32<T>(v);
  }
  if (!write_cache) return;
  const int slot = slots[t];
  if (slot < 0) return;      // a row that pads a captured batch
  const T* kv = row + (size_t)heads * (dim + rd);
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = to_f32(kv[i]);
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)rank + eps);
  T* out = cache + (size_t)slot * D;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) out[i] = from_f32<T>(norm_scale(to_f32(kv[i]), cw[i], inv));
  for (int i = threadIdx.x; i < rd; i += blockDim.x) {
    float v = to_f32(kv[rank + i]);
    if (i < half) {
      float x = v, y = to_f32(kv[rank + i + half]);
      rotate_pair(x, y, cs[i], sn[i]);
      v = x;
    } else if (i < rot_dims) {
      float x = to_f32(kv[rank + i - half]), y = v;
      rotate_pair(x, y, cs[i - half], sn[i - half]);
      v = y;
    }
    out[rank + i] = from_f32<T>(v);
  }
}
}  // namespace

extern "C" int zi_latent_prepare(const void* src, int ld, int dtype, int T, int heads, int dim, int rd, int rank,
                                 int rot_dims, const float* cw, float eps, const float* cos_t, const float* sin_t,
                                 int n_table_pos, const int* positions, void* q_eff, void* cache, const int* slots,
                                 int write_cache, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rot_dims < 0 || rot_dims % 2 || rot_dims > rd) return zi_refuse("latent_prepare: %d rotated dimensions of %d", rot_dims, rd);
  if (n_table_pos <= 0 && rot_dims > 0) return zi_refuse("latent_prepare: the rotary table is empty");
  ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(latent_prepare_kernel<TT>, dim3(T), dim3(128), 0, stream, (const TT*)src, ld, heads,
                                         dim, rd, rank, rot_dims, cw, eps, cos_t, sin_t, n_table_pos, positions,
                                         (TT*)q_eff, (TT*)cache, slots, write_cache));
  return zi_check_launch("latent_prepare");
}

ZI_TRACE_SETTER(latent_attention)
