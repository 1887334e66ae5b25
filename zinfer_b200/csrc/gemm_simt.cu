// out[M,N] = x[M,K] * w[N,K]^T on the CUDA cores with 32-bit multiply-adds: the
// true 32-bit matrix product (no tensor-core mode of reduced precision), also
// usable with bfloat16 operands as the plain stand-in of the tensor-core kernel.
// Every output element is one chain of fused multiply-adds over k = 0..K-1 in
// order, so a row's result does not depend on which other rows are in the batch.
#include "api.h"
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256) gemm_simt_kernel(TO* __restrict__ out, const TX* __restrict__ x,
                                                        const TW* __restrict__ w, int M, int N, int K, int ldx,
                                                        int ldw, int ldo) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // each thread loads 4 elements of each tile: row = e / BK, k = e % BK
#pragma unroll
    for (int e = tid; e < BM * BK; e += 256) {
      const int r = e / BK, kk = e % BK;
      const int m = m0 + r, k = k0 + kk;
      xs[kk][r] = (m < M && k < K) ? to_f32(x[(size_t)m * ldx + k]) : 0.f;
    }
#pragma unroll
    for (int e = tid; e < BN * BK; e += 256) {
      const int r = e / BK, kk = e % BK;
      const int n = n0 + r, k = k0 + kk;
      ws[kk][r] = (n < N && k < K) ? to_f32(w[(size_t)n * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = xs[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n < N) out[(size_t)m * ldo + n] = from_f32<TO>(acc[i][j]);
    }
  }
}

template <typename TX, typename TW, typename TO>
int launch(void* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldw, int ldo,
           cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  zi_launch(gemm_simt_kernel<TX, TW, TO>, dim3(grid), dim3(256), 0, stream, (TO*)out, (const TX*)x, (const TW*)w, M, N, K, ldx, ldw, ldo);
  return zi_check_launch("gemm_simt");
}

// ------------------------------------------------------------------ batched and grouped forms
// The same product with three additions, for block-diagonal gates, per-head projections and the
// experts of a mixture:
//   batch    blockIdx.z picks one of `batch` independent products whose operands lie sx, sw, so
//            (and sb for the bias) elements apart;
//   groups   every tile of TM*16 output rows names the weight group (expert) it multiplies with in
//            tile_group[], groups lie group_stride elements apart, the x row of an output row comes
//            from row_src[] (a gather; -1: no row, nothing is stored), and tiles at or beyond
//            *n_tiles_dev do nothing: the sizes are known on the device only;
//   epilogue an optional bias per output column, then ZI_EPI_NONE or ZI_EPI_RELU2 (the square of relu).
// Every output is still one chain of fused multiply-adds over k in order.
template <typename TX, typename TW, typename TO, int TM_>
__global__ void __launch_bounds__(256)
gemm_simt_general_kernel(TO* __restrict__ out, const TX* __restrict__ x, const TW* __restrict__ w, int M, int N, int K,
                         int ldx, int ldw, int ldo, long long sx, long long sw, long long so,
                         const float* __restrict__ bias, long long sb, const int* __restrict__ row_src,
                         const int* __restrict__ tile_group, const int* __restrict__ n_tiles_dev,
                         long long group_stride, int epilogue) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int BM_ = 16 * TM_;
  __shared__ float xs[BK][BM_ + 4];
  __shared__ float ws[BK][BN + 4];
  __shared__ int src_rows[BM_];
  if (n_tiles_dev && (int)blockIdx.y >= *n_tiles_dev) return;
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * BM_, n0 = blockIdx.x * BN;
  x += (size_t)blockIdx.z * sx;
  w += (size_t)blockIdx.z * sw;
  out += (size_t)blockIdx.z * so;
  if (bias) bias += (size_t)blockIdx.z * sb;
  if (tile_group) {
    const int e = tile_group[blockIdx.y];
    w += (size_t)e * group_stride;
    if (bias) bias += (size_t)e * N;
  }
  if (tid < BM_) {
    const int m = m0 + tid;
    src_rows[tid] = m < M ? (row_src ? row_src[m] : m) : -1;
  }
  __syncthreads();
  float acc[TM_][TN];
#pragma unroll
  for (int i = 0; i < TM_; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int e = tid; e < BM_ * BK; e += 256) {
      const int r = e / BK, kk = e % BK;
      const int src = src_rows[r], k = k0 + kk;
      xs[kk][r] = (src >= 0 && k < K) ? to_f32(x[(size_t)src * ldx + k]) : 0.f;
    }
#pragma unroll
    for (int e = tid; e < BN * BK; e += 256) {
      const int r = e / BK, kk = e % BK;
      const int n = n0 + r, k = k0 + kk;
      ws[kk][r] = (n < N && k < K) ? to_f32(w[(size_t)n * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM_], b[TN];
#pragma unroll
      for (int i = 0; i < TM_; ++i) a[i] = xs[kk][ty * TM_ + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM_; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM_; ++i) {
    const int m = m0 + ty * TM_ + i;
    if (m >= M || src_rows[ty * TM_ + i] < 0) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      if (epilogue == ZI_EPI_RELU2) {
        v = fmaxf(v, 0.f);
        v *= v;
      }
      out[(size_t)m * ldo + n] = from_f32<TO>(v);
    }
  }
}

template <typename TX, typename TW, typename TO>
int launch_general(void* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldw, int ldo, int batch,
                   long long sx, long long sw, long long so, const float* bias, long long sb, const int* row_src,
                   const int* tile_group, const int* n_tiles_dev, long long group_stride, int epilogue, int small_tiles,
                   cudaStream_t stream) {
  const int bm = small_tiles ? 16 : 64;
  dim3 grid((N + BN - 1) / BN, (M + bm - 1) / bm, batch);
  if (small_tiles)
    zi_launch(gemm_simt_general_kernel<TX, TW, TO, 1>, dim3(grid), dim3(256), 0, stream, (TO*)out, (const TX*)x, (const TW*)w,
              M, N, K, ldx, ldw, ldo, sx, sw, so, bias, sb, row_src, tile_group, n_tiles_dev, group_stride, epilogue);
  else
    zi_launch(gemm_simt_general_kernel<TX, TW, TO, 4>, dim3(grid), dim3(256), 0, stream, (TO*)out, (const TX*)x, (const TW*)w,
              M, N, K, ldx, ldw, ldo, sx, sw, so, bias, sb, row_src, tile_group, n_tiles_dev, group_stride, epilogue);
  return zi_check_launch("gemm_simt (batched or grouped)");
}
}  // namespace

extern "C" int zi_gemm_simt_general(void* out, int out_dtype, const void* x, int x_dtype, const void* w, int w_dtype,
                                    int M, int N, int K, int ldx, int ldw, int ldo, int batch, long long sx,
                                    long long sw, long long so, const float* bias, long long sb, const int* row_src,
                                    const int* tile_group, const int* n_tiles_dev, long long group_stride,
                                    int epilogue, int tile_rows, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || batch <= 0) return 0;
  if (K <= 0) return zi_refuse("gemm: K must be positive, got %d", K);
  if (tile_rows != 16 && tile_rows != 64) return zi_refuse("gemm: tiles have 16 or 64 rows, not %d", tile_rows);
  if (batch > 65535) return zi_refuse("gemm: at most 65535 products in a batch, got %d", batch);
  if (epilogue != ZI_EPI_NONE && epilogue != ZI_EPI_RELU2) return zi_refuse("gemm: unknown epilogue %d", epilogue);
  using bf = __nv_bfloat16;
  const int small = tile_rows == 16;
#define ZI_GENERAL(TX, TW, TO)                                                                                     \
  return launch_general<TX, TW, TO>(out, x, w, M, N, K, ldx, ldw, ldo, batch, sx, sw, so, bias, sb, row_src, tile_group, \
                                    n_tiles_dev, group_stride, epilogue, small, stream)
  const int key = x_dtype * 4 + w_dtype * 2 + out_dtype;
  switch (key) {
    case 0: ZI_GENERAL(float, float, float);
    case 1: ZI_GENERAL(float, float, bf);
    case 2: ZI_GENERAL(float, bf, float);
    case 3: ZI_GENERAL(float, bf, bf);
    case 4: ZI_GENERAL(bf, float, float);
    case 5: ZI_GENERAL(bf, float, bf);
    case 6: ZI_GENERAL(bf, bf, float);
    case 7: ZI_GENERAL(bf, bf, bf);
  }
#undef ZI_GENERAL
  return zi_refuse("gemm: unknown dtype tags x=%d w=%d out=%d", x_dtype, w_dtype, out_dtype);
}

namespace {
}  // namespace

extern "C" int zi_gemm_simt(void* out, int out_dtype, const void* x, int x_dtype, const void* w, int w_dtype, int M,
                            int N, int K, int ldx, int ldw, int ldo, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return zi_refuse("gemm: K must be positive, got %d", K);
  using bf = __nv_bfloat16;
  const int key = x_dtype * 4 + w_dtype * 2 + out_dtype;
  switch (key) {
    case 0: return launch<float, float, float>(out, x, w, M, N, K, ldx, ldw, ldo, stream);
    case 1: return launch<float, float, bf>(out, x, w, M, N, K, ldx, ldw, ldo, stream);
    case 2: return launch<float, bf, float>(out, x, w, M, N, K, ldx, ldw, ldo, stream);
    case 3: return launch<float, bf, bf>(out, x, w, M, N, K, ldx, ldw, ldo, stream);
    case 4: return launch<bf, float, float>(out, x, w, M, N, K, ldx, ldw, ldo, stream);
    case 5: return launch<bf, float, bf>(out, x, w, M, N, K, ldx, ldw, ldo, stream);
    case 6: return launch<bf, bf, float>(out, x, w, M, N, K, ldx, ldw, ldo, stream);
    case 7: return launch<bf, bf, bf>(out, x, w, M, N, K, ldx, ldw, ldo, stream);
  }
  return zi_refuse("gemm: unknown dtype tags x=%d w=%d out=%d", x_dtype, w_dtype, out_dtype);
}

ZI_TRACE_SETTER(gemm_simt)
