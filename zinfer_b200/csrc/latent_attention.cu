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

// A request's cached rows, gathered from its pages for the tensor-core products of a prompt's portion:
// keys[j, :] = row j (all D columns; rows kv_len .. kv_pad-1 are zero) and values_t[r, j] = row j's
// column r for r < rank (the latent part, transposed: the second product's weight-side operand).
// One block takes 32 keys.
template <typename T>
__global__ void __launch_bounds__(256)
latent_gather_kernel(T* __restrict__ keys, T* __restrict__ values_t, const T* __restrict__ cache,
                     const int* __restrict__ block_table, int page_size, int kv_len, int kv_pad, int D, int rank) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ unsigned char raw[];
  T* tile = reinterpret_cast<T*>(raw);           // [32][D + 2]
  const int j0 = blockIdx.x * 32, pitch = D + 2;
  for (int e = threadIdx.x; e < 32 * D; e += blockDim.x) {
    const int kk = e / D, c = e - kk * D, j = j0 + kk;
    T v = from_f32<T>(0.f);
    if (j < kv_len) {
      const int page = block_table[j / page_size];
      if (page >= 0) v = cache[((size_t)page * page_size + (j % page_size)) * D + c];
    }
    tile[kk * pitch + c] = v;
    if (j < kv_pad) keys[(size_t)j * D + c] = v;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < 32 * rank; e += blockDim.x) {
    const int r = e / 32, kk = e - r * 32, j = j0 + kk;
    if (j < kv_pad) values_t[(size_t)r * kv_pad + j] = tile[kk * pitch + r];
  }
}

// Causal softmax over a portion's scores: row (t, h) of S [rows, kv_pad] (32-bit) belongs to the query at
// position ctx + t and sees keys 0 .. ctx + t; P[row, j] = exp(scale * (S - max)) / sum there, 0 beyond
// (also in the padding columns), written in the activations' type for the second product.
template <typename T>
__global__ void __launch_bounds__(256)
causal_softmax_kernel(T* __restrict__ P, const float* __restrict__ S, int heads, int ctx, int kv_pad, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  __shared__ float red[8];
  const size_t row = blockIdx.x;
  const int visible = ctx + (int)(row / heads) + 1;
  const float* s = S + row * kv_pad;
  T* p = P + row * kv_pad;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float m = -INFINITY;
  for (int j = threadIdx.x; j < visible; j += blockDim.x) m = fmaxf(m, s[j]);
  m = warp_max(m);
  if (lane == 0) red[warp] = m;
  __syncthreads();
  m = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
  float sum = 0.f;
  for (int j = threadIdx.x; j < visible; j += blockDim.x) sum += expf(scale * (s[j] - m));
  const float inv = 1.0f / block_sum(sum, scratch);
  for (int j = threadIdx.x; j < kv_pad; j += blockDim.x)
    p[j] = from_f32<T>(j < visible ? expf(scale * (s[j] - m)) * inv : 0.f);
}
}  // namespace

extern "C" int zi_latent_gather(void* keys, void* values_t, const void* cache, int dtype, const int* block_table,
                                int page_size, int kv_len, int kv_pad, int D, int rank, cudaStream_t stream) {
  if (kv_pad <= 0) return 0;
  if (rank > D || kv_len > kv_pad) return zi_refuse("latent_gather: rank %d of %d columns, %d of %d keys", rank, D, kv_len, kv_pad);
  const size_t smem = (size_t)32 * (D + 2) * (dtype == ZI_F32 ? 4 : 2);
  ZI_DISPATCH_DTYPE(dtype, TT, {
    auto kern = latent_gather_kernel<TT>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return zi_refuse("latent_gather: cannot get %zu bytes of shared memory", smem);
    zi_launch(kern, dim3((kv_pad + 31) / 32), dim3(256), smem, stream, (TT*)keys, (TT*)values_t, (const TT*)cache,
              block_table, page_size, kv_len, kv_pad, D, rank);
  });
  return zi_check_launch("latent_gather");
}

extern "C" int zi_causal_softmax(void* P, const float* S, int dtype, long long rows, int heads, int ctx, int kv_pad,
                                 float scale, cudaStream_t stream) {
  if (rows <= 0 || kv_pad <= 0) return 0;
  if (rows > 0x7fffffffLL) return zi_refuse("causal_softmax: too many rows");
  ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(causal_softmax_kernel<TT>, dim3((unsigned)rows), dim3(256), 0, stream, (TT*)P, S,
                                         heads, ctx, kv_pad, scale));
  return zi_check_launch("causal_softmax");
}

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
