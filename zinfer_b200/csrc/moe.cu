// Routing of a mixture of experts: scores and choice per token, the layout of the chosen
// (token, expert) pairs for the grouped products, and the weighted sum of the experts' outputs.
// The grouped products themselves are zi_gemm_simt_general (gemm_simt.cu).  All arithmetic is 32-bit.
//
// A router has NR outputs: the first E are experts with weights, the last NR - E stand for
// "identity experts" whose output is their input.  Scores are a softmax over all NR outputs; the
// choice adds a correction per output to the score, the weight of a chosen expert is its score
// without the correction, optionally divided by the sum of the chosen scores.
#include "api.h"
#include "common.cuh"

namespace {
constexpr int ROUTE_WARPS = 4;

// One warp per token.  Sums run over a fixed order of lanes, so a token's choice does not depend on
// the batch.  Ties go to the lower index.
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(int* __restrict__ chosen, float* __restrict__ weight, const float* __restrict__ logits,
                 const float* __restrict__ correction, int T, int NR, int top, int renormalize) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= T) return;
  float* score = sm + (size_t)warp * 2 * NR;   // softmax scores
  float* pick = score + NR;                    // scores plus correction; -inf once chosen
  const float* z = logits + (size_t)t * NR;
  float m = -INFINITY;
  for (int j = lane; j < NR; j += 32) m = fmaxf(m, z[j]);
  m = warp_max(m);
  float sum = 0.f;
  for (int j = lane; j < NR; j += 32) {
    const float e = expf(z[j] - m);
    score[j] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  const float inv = 1.0f / sum;
  for (int j = lane; j < NR; j += 32) {
    const float s = score[j] * inv;
    score[j] = s;
    pick[j] = s + (correction ? correction[j] : 0.f);
  }
  __syncwarp();
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int j = lane; j < NR; j += 32) {
      const float v = pick[j];
      if (v > best) {      // ascending j: the first of equal values stays
        best = v;
        arg = j;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) {
        best = ob;
        arg = oa;
      }
    }
    if (arg == 0x7fffffff) arg = 0;    // every remaining value is -inf or NaN
    const float s = score[arg];
    total += s;
    if (lane == 0) {
      chosen[(size_t)t * top + k] = arg;
      weight[(size_t)t * top + k] = s;
      pick[arg] = -INFINITY;
    }
    __syncwarp();
  }
  if (renormalize && lane == 0) {
    const float r = 1.0f / total;
    for (int k = 0; k < top; ++k) weight[(size_t)t * top + k] *= r;
  }
}

// One block lays the P = T * top pairs out by expert.  Pairs of expert e take the rows
// off[e] .. off[e] + count[e] - 1, and off[e+1] - off[e] is count[e] rounded up to whole tiles of
// `tile_rows`, so that every tile of the grouped product has one expert.  Pairs that chose an
// identity expert (index >= E) take no row.
//   row_token[r]  token whose input row r multiplies (-1: padding)
//   row_self[r]   r where the row is in use, else -1
//   pair_row[p]   row of pair p (-1: an identity expert)
//   tile_expert[i], *n_tiles     the arrays have cap_tiles tiles (at least P / tile_rows + E); rows and tiles
//                                beyond the ones in use are marked -1 and expert 0
__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ chosen, int P, int top, int E, int tile_rows, int cap_tiles,
                 int* __restrict__ row_token,
                 int* __restrict__ row_self, int* __restrict__ pair_row, int* __restrict__ tile_expert,
                 int* __restrict__ n_tiles) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ int si[];
  int* count = si;            // [E]
  int* off = si + E;          // [E + 1]
  int* cursor = off + E + 1;  // [E]
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = cursor[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = chosen[p];
    if (e >= 0 && e < E) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = o;
      const int nt = (count[e] + tile_rows - 1) / tile_rows;
      for (int i = 0; i < nt; ++i) tile_expert[tiles + i] = e;
      tiles += nt;
      o += nt * tile_rows;
    }
    off[E] = o;
    *n_tiles = tiles;
    for (int i = tiles; i < cap_tiles; ++i) tile_expert[i] = 0;   // tiles not in use still name a group that exists
  }
  __syncthreads();
  const int rows = cap_tiles * tile_rows;      // all rows the arrays have: a product may walk every tile
  for (int r = threadIdx.x; r < rows; r += blockDim.x) row_token[r] = row_self[r] = -1;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = chosen[p];
    int r = -1;
    if (e >= 0 && e < E) {
      r = off[e] + atomicAdd(&cursor[e], 1);
      row_token[r] = p / top;
      row_self[r] = r;
    }
    pair_row[p] = r;
  }
}

// out[r] = x[row_src[r]], or zeros where row_src[r] is -1: the tokens' rows in the order of the pairs.
template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* __restrict__ x, const int* __restrict__ row_src,
                                   int width, int ldx) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, src = row_src[r];
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    out[(size_t)r * width + c] = src >= 0 ? x[(size_t)src * ldx + c] : from_f32<T>(0.f);
}

// out[t] = sum_k weight[t,k] * (expert output of pair (t,k), or x[t] for an identity expert), k ascending.
template <typename T>
__global__ void moe_combine_kernel(T* __restrict__ out, const float* __restrict__ y, const T* __restrict__ x,
                                   const int* __restrict__ chosen, const float* __restrict__ weight,
                                   const int* __restrict__ pair_row, int top, int E, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float acc = 0.f;
  for (int k = 0; k < top; ++k) {
    const size_t p = (size_t)t * top + k;
    const int e = chosen[p];
    const float v = e < E ? y[(size_t)pair_row[p] * H + c] : to_f32(x[(size_t)t * H + c]);
    acc = fmaf(weight[p], v, acc);
  }
  out[(size_t)t * H + c] = from_f32<T>(acc);
}
}  // namespace

extern "C" int zi_moe_route(int* chosen, float* weight, const float* logits, const float* correction, int T, int NR,
                            int top, int renormalize, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (top <= 0 || top > NR) return zi_refuse("moe_route: %d of %d outputs cannot be chosen", top, NR);
  const size_t smem = (size_t)ROUTE_WARPS * 2 * NR * sizeof(float);
  if (smem > 48 * 1024) return zi_refuse("moe_route: %d router outputs are more than this kernel holds", NR);
  zi_launch(moe_route_kernel, dim3((T + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), smem, stream, chosen,
            weight, logits, correction, T, NR, top, renormalize);
  return zi_check_launch("moe_route");
}

extern "C" int zi_moe_align(const int* chosen, int P, int top, int E, int tile_rows, int cap_tiles, int* row_token,
                            int* row_self, int* pair_row, int* tile_expert, int* n_tiles, cudaStream_t stream) {
  if (P <= 0) return 0;
  if (cap_tiles < (P + tile_rows - 1) / tile_rows + E) return zi_refuse("moe_align: %d tiles cannot hold %d pairs of %d experts", cap_tiles, P, E);
  const size_t smem = (size_t)(3 * E + 1) * sizeof(int);
  if (smem > 48 * 1024) return zi_refuse("moe_align: %d experts are more than this kernel holds", E);
  zi_launch(moe_align_kernel, dim3(1), dim3(1024), smem, stream, chosen, P, top, E, tile_rows, cap_tiles, row_token,
            row_self, pair_row, tile_expert, n_tiles);
  return zi_check_launch("moe_align");
}

extern "C" int zi_gather_rows(void* out, const void* x, int dtype, const int* row_src, int rows, int width, int ldx,
                              cudaStream_t stream) {
  if (rows <= 0 || width <= 0) return 0;
  ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(gather_rows_kernel<TT>, dim3(rows), dim3(256), 0, stream, (TT*)out, (const TT*)x,
                                         row_src, width, ldx));
  return zi_check_launch("gather_rows");
}

extern "C" int zi_moe_combine(void* out, const float* y, const void* x, int dtype, const int* chosen,
                              const float* weight, const int* pair_row, int T, int top, int E, int H,
                              cudaStream_t stream) {
  if (T <= 0) return 0;
  dim3 grid((H + 255) / 256, T);
  ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(moe_combine_kernel<TT>, dim3(grid), dim3(256), 0, stream, (TT*)out, y, (const TT*)x,
                                         chosen, weight, pair_row, top, E, H));
  return zi_check_launch("moe_combine");
}

ZI_TRACE_SETTER(moe)
