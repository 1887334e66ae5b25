// Kernels of recurrent mixers: a short causal convolution per channel whose last inputs are carried
// from step to step, and the real-gated linear recurrence
//     a_t = exp(-c * r_t * softplus(lam)),  S_t = a_t S_(t-1) + sqrt(1 - a_t^2) * i_t * u_t
// with its state carried per request.  Everything here is 32-bit arithmetic; only the branch inputs
// (x and y, the outputs of matrix products) and the result may be bfloat16.
//
// The per-request state is one 32-bit array [slots][taps][C]: rows 0 .. taps-2 hold the last taps-1
// inputs of the convolution (oldest first), row taps-1 holds S.  A request's tokens of this step are
// rows cu_q[s] .. cu_q[s+1]-1 of the flat batch; they continue the request from the state in slot
// state_slots[s].  A row is never touched by two blocks, and each channel's tokens are visited in
// order, so a result does not depend on how the request was cut into steps or on the batch.
#include "api.h"
#include "common.cuh"

namespace {

__device__ __forceinline__ float softplus_f32(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f32(float x) { return 1.0f / (1.0f + expf(-x)); }

// Input of the convolution `back` tokens before token t of request s (back >= 0): from this step's
// rows if it lies in them, else from the carried rows, else (before the request's start: the carried
// rows are zero then) zero.
template <typename T>
__device__ __forceinline__ float conv_input(const T* __restrict__ x, int ldx, const float* __restrict__ xb,
                                            const float* __restrict__ st, int C, int taps, int t_local, int tok0,
                                            int back, int c) {
  const int src = t_local - back;
  if (src >= 0) return to_f32(x[(size_t)(tok0 + src) * ldx + c]) + xb[c];
  const int row = taps - 1 + src;        // src = -1 is the newest carried input: row taps-2
  return row >= 0 ? st[(size_t)row * C + c] : 0.f;
}

// u[t, c] = cb[c] + sum_j k[c, j] * input(t - (taps-1-j)), one thread per (token, channel).
template <typename T>
__global__ void causal_conv_kernel(float* __restrict__ u, const T* __restrict__ x, int ldx,
                                   const float* __restrict__ xb, const float* __restrict__ kern,
                                   const float* __restrict__ cb, const float* __restrict__ state, int C, int taps,
                                   const int* __restrict__ cu_q, const int* __restrict__ state_slots, int n_seqs) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  int s = 0, hi = n_seqs - 1;          // the request whose rows hold token t: cu_q[s] <= t < cu_q[s+1]
  while (s < hi) {
    const int mid = (s + hi + 1) >> 1;
    if (cu_q[mid] <= t) s = mid; else hi = mid - 1;
  }
  const int tok0 = cu_q[s];
  const float* st = state + (size_t)state_slots[s] * taps * C;
  float acc = cb[c];
  for (int j = 0; j < taps; ++j)
    acc = fmaf(kern[(size_t)c * taps + j], conv_input(x, ldx, xb, st, C, taps, t - tok0, tok0, taps - 1 - j, c), acc);
  u[(size_t)t * C + c] = acc;
}

// The recurrence over a request's tokens of this step, one thread per (request, channel).
// gates [T, blocks, 2, bw] (the products of the block-diagonal gate matrices: recurrence gate, then
// input gate, per block), rb and ib their biases [C], lam [C], y the gated branch before its bias
// and gelu.  Writes out[t, c] = S_t * gelu_tanh(y + yb), the new S and the new carried inputs.
template <typename T>
__global__ void rglru_scan_kernel(T* __restrict__ out, int ldo, const float* __restrict__ u,
                                  const float* __restrict__ gates, int bw, const float* __restrict__ rb,
                                  const float* __restrict__ ib, const float* __restrict__ lam, float decay_scale,
                                  const T* __restrict__ y, int ldy, const float* __restrict__ yb,
                                  const T* __restrict__ x, int ldx, const float* __restrict__ xb,
                                  float* __restrict__ state, int C, int taps, const int* __restrict__ cu_q,
                                  const int* __restrict__ state_slots) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int tok0 = cu_q[s], n = cu_q[s + 1] - tok0;
  if (n <= 0) return;
  float* st = state + (size_t)state_slots[s] * taps * C;
  const int b = c / bw, o = c - b * bw;
  const size_t gcol = (size_t)b * 2 * bw + o;       // recurrence gate; the input gate lies bw further
  const float rate = -decay_scale * softplus_f32(lam[c]);
  const float rbias = rb[c], ibias = ib[c], ybias = yb[c];
  float S = st[(size_t)(taps - 1) * C + c];
  for (int t = 0; t < n; ++t) {
    const size_t row = (size_t)(tok0 + t);
    const float r = sigmoid_f32(gates[row * 2 * C + gcol] + rbias);
    const float i = sigmoid_f32(gates[row * 2 * C + gcol + bw] + ibias);
    const float log_a = rate * r;
    const float a = expf(log_a);
    const float mult = sqrtf(-expm1f(2.0f * log_a));      // sqrt(1 - a^2) without cancellation near a = 1
    S = fmaf(a, S, mult * (i * u[row * C + c]));
    const float yv = gelu_tanh_f32(to_f32(y[row * ldy + c]) + ybias);
    out[row * ldo + c] = from_f32<T>(S * yv);
  }
  st[(size_t)(taps - 1) * C + c] = S;
  // the last taps-1 inputs of the convolution, oldest first (read before any is overwritten)
  float keep[8];
  for (int j = 0; j < taps - 1; ++j) keep[j] = conv_input(x, ldx, xb, st, C, taps, n, tok0, taps - 1 - j, c);
  for (int j = 0; j < taps - 1; ++j) st[(size_t)j * C + c] = keep[j];
}

// ------------------------------------------------------------- the recurrence in chunks (prompts)
// One thread per channel walking a prompt's tokens one after the other leaves most of the GPU idle.  The
// recurrence S_t = a_t S_(t-1) + b_t is linear, so the flat batch is cut into chunks of `chunk` tokens:
//   1. every chunk alone: A = product of its a_t, B = its final state from zero   (blocks: channels x chunks)
//   2. the chunks' incoming states, one after the other: S_in[k+1] = A[k] S_in[k] + B[k]   (blocks: channels)
//   3. every chunk again from its S_in, writing the outputs                         (blocks: channels x chunks)
//   4. per request: the new state and the convolution's carried inputs              (blocks: channels x requests)
// A request's first token of the step takes the request's carried state as S_(t-1): in the flat recurrence
// that is a_t = 0 with b_t = a_t * carried + b_t, so chunks may span requests.  The sums are associated
// differently than in the token-by-token walk (rounding only); the 32-bit path keeps the walk.
struct GateTerms {
  float a, b;
};

__device__ __forceinline__ GateTerms gate_terms(const float* __restrict__ gates, const float* __restrict__ u, size_t row,
                                                int C, size_t gcol, int bw, float rbias, float ibias, float rate, int c) {
  const float r = sigmoid_f32(gates[row * 2 * C + gcol] + rbias);
  const float i = sigmoid_f32(gates[row * 2 * C + gcol + bw] + ibias);
  const float log_a = rate * r;
  GateTerms t;
  t.a = expf(log_a);
  t.b = sqrtf(-expm1f(2.0f * log_a)) * (i * u[row * C + c]);
  return t;
}

// request whose rows hold flat token t
__device__ __forceinline__ int seq_of_token(const int* __restrict__ cu_q, int n_seqs, int t) {
  int s = 0, hi = n_seqs - 1;
  while (s < hi) {
    const int mid = (s + hi + 1) >> 1;
    if (cu_q[mid] <= t) s = mid; else hi = mid - 1;
  }
  return s;
}

// passes 1 (WRITE false: A and B of the chunk into ab[chunk][2][C]) and 3 (WRITE true: outputs from s_in[chunk][C],
// and each request's last state into last[request][C])
template <typename T, bool WRITE>
__global__ void rglru_chunk_kernel(T* __restrict__ out, int ldo, float* __restrict__ ab, const float* __restrict__ s_in,
                                   float* __restrict__ last, const float* __restrict__ u,
                                   const float* __restrict__ gates, int bw, const float* __restrict__ rb,
                                   const float* __restrict__ ib, const float* __restrict__ lam, float decay_scale,
                                   const T* __restrict__ y, int ldy, const float* __restrict__ yb,
                                   const float* __restrict__ state, int C, int taps, const int* __restrict__ cu_q,
                                   const int* __restrict__ state_slots, int n_seqs, int T_total, int chunk) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int k = blockIdx.y, t0 = k * chunk, t1 = min(T_total, t0 + chunk);
  const int b = c / bw, o = c - b * bw;
  const size_t gcol = (size_t)b * 2 * bw + o;
  const float rate = -decay_scale * softplus_f32(lam[c]);
  const float rbias = rb[c], ibias = ib[c], ybias = WRITE ? yb[c] : 0.f;
  int s = seq_of_token(cu_q, n_seqs, t0);
  int next_start = cu_q[s + 1];
  float A = 1.f, S = WRITE ? s_in[(size_t)k * C + c] : 0.f;
  for (int t = t0; t < t1; ++t) {
    while (t >= next_start) {        // requests that bring no token have no rows
      ++s;
      next_start = cu_q[s + 1];
    }
    if (t == cu_q[s]) {              // the request's first token of this step: from its carried state
      S = state[((size_t)state_slots[s] * taps + (taps - 1)) * C + c];
      A = 0.f;
    }
    const GateTerms g = gate_terms(gates, u, (size_t)t, C, gcol, bw, rbias, ibias, rate, c);
    S = fmaf(g.a, S, g.b);
    A *= g.a;
    if (WRITE) {
      out[(size_t)t * ldo + c] = from_f32<T>(S * gelu_tanh_f32(to_f32(y[(size_t)t * ldy + c]) + ybias));
      if (t == next_start - 1) last[(size_t)s * C + c] = S;
    }
  }
  if (!WRITE) {
    ab[((size_t)k * 2) * C + c] = A;
    ab[((size_t)k * 2 + 1) * C + c] = S;
  }
}

// pass 2: s_in[k] for every chunk.  A chunk that begins with a request's first token has A = 0 there, so
// what flows in does not matter; chunk 0 always does.
__global__ void rglru_carry_kernel(float* __restrict__ s_in, const float* __restrict__ ab, int C, int n_chunks) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float S = 0.f;
  for (int k = 0; k < n_chunks; ++k) {
    s_in[(size_t)k * C + c] = S;
    S = fmaf(ab[((size_t)k * 2) * C + c], S, ab[((size_t)k * 2 + 1) * C + c]);
  }
}

// pass 4: the requests' new states and carried inputs
template <typename T>
__global__ void rglru_finish_kernel(float* __restrict__ state, const float* __restrict__ last, const T* __restrict__ x,
                                    int ldx, const float* __restrict__ xb, int C, int taps, const int* __restrict__ cu_q,
                                    const int* __restrict__ state_slots) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int tok0 = cu_q[s], n = cu_q[s + 1] - tok0;
  if (n <= 0) return;
  float* st = state + (size_t)state_slots[s] * taps * C;
  st[(size_t)(taps - 1) * C + c] = last[(size_t)s * C + c];
  float keep[8];
  for (int j = 0; j < taps - 1; ++j) keep[j] = conv_input(x, ldx, xb, st, C, taps, n, tok0, taps - 1 - j, c);
  for (int j = 0; j < taps - 1; ++j) st[(size_t)j * C + c] = keep[j];
}

// A step in which every request brings one token: convolution, both gates, the recurrence and the gated
// output in one kernel.  Block (channel block b, request s); a warp takes gate rows in turn, its lanes
// stride over the block's inputs and the partial sums meet in a fixed order.
//   wg [blocks][2 bw][bw]: per block the recurrence gate's matrix above the input gate's.
template <typename T, typename TW>
__global__ void __launch_bounds__(256)
rglru_decode_kernel(T* __restrict__ out, int ldo, const T* __restrict__ yx, int ld, const float* __restrict__ yb,
                    const float* __restrict__ xb, const float* __restrict__ kern, const float* __restrict__ cb,
                    const TW* __restrict__ wg, int bw, const float* __restrict__ rb, const float* __restrict__ ib,
                    const float* __restrict__ lam, float decay_scale, float* __restrict__ state, int C, int taps,
                    const int* __restrict__ state_slots) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sh[];
  float* u = sh;               // [bw]
  float* gate = sh + bw;       // [2 bw]
  const int b = blockIdx.x, s = blockIdx.y, c0 = b * bw;
  float* st = state + (size_t)state_slots[s] * taps * C;
  const T* y = yx + (size_t)s * ld;          // this request's row: y branch, then x branch
  const T* x = y + C;
  for (int o = threadIdx.x; o < bw; o += blockDim.x) {
    const int c = c0 + o;
    const float xin = to_f32(x[c]) + xb[c];
    float acc = cb[c];
    for (int j = 0; j < taps - 1; ++j) acc = fmaf(kern[(size_t)c * taps + j], st[(size_t)j * C + c], acc);
    u[o] = fmaf(kern[(size_t)c * taps + taps - 1], xin, acc);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const TW* w = wg + (size_t)b * 2 * bw * bw;
  for (int row = warp; row < 2 * bw; row += nwarp) {
    float acc = 0.f;
    for (int i = lane; i < bw; i += 32) acc = fmaf(to_f32(w[(size_t)row * bw + i]), u[i], acc);
    acc = warp_sum(acc);
    if (lane == 0) gate[row] = acc;
  }
  __syncthreads();
  for (int o = threadIdx.x; o < bw; o += blockDim.x) {
    const int c = c0 + o;
    const float r = sigmoid_f32(gate[o] + rb[c]);
    const float i = sigmoid_f32(gate[bw + o] + ib[c]);
    const float log_a = -decay_scale * softplus_f32(lam[c]) * r;
    const float a = expf(log_a);
    const float mult = sqrtf(-expm1f(2.0f * log_a));
    const float S = fmaf(a, st[(size_t)(taps - 1) * C + c], mult * (i * u[o]));
    st[(size_t)(taps - 1) * C + c] = S;
    out[(size_t)s * ldo + c] = from_f32<T>(S * gelu_tanh_f32(to_f32(y[c]) + yb[c]));
    // the carried inputs move up by one; the newest is this token's
    for (int j = 0; j + 1 < taps - 1; ++j) st[(size_t)j * C + c] = st[(size_t)(j + 1) * C + c];
    if (taps > 1) st[(size_t)(taps - 2) * C + c] = to_f32(x[c]) + xb[c];
  }
}
}  // namespace

extern "C" int zi_rglru_decode(void* out, int ldo, const void* yx, int ld, int dtype, const float* yb, const float* xb,
                               const float* kern, const float* cb, const void* wg, int wg_dtype, int block_width,
                               const float* rb, const float* ib, const float* lam, float decay_scale, float* state,
                               int C, int taps, const int* state_slots, int n_seqs, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (taps < 1 || taps > 9) return zi_refuse("rglru_decode: 1 to 9 taps, got %d", taps);
  if (block_width <= 0 || C % block_width) return zi_refuse("rglru_decode: %d channels do not divide into blocks of %d", C, block_width);
  const size_t smem = (size_t)3 * block_width * sizeof(float);
  if (smem > 48 * 1024) return zi_refuse("rglru_decode: blocks of %d channels are more than this kernel holds", block_width);
  dim3 grid(C / block_width, n_seqs);
  using bf = __nv_bfloat16;
#define ZI_RGLRU_DECODE(TT, TW)                                                                                      \
  zi_launch(rglru_decode_kernel<TT, TW>, dim3(grid), dim3(256), smem, stream, (TT*)out, ldo, (const TT*)yx, ld, yb, xb, \
            kern, cb, (const TW*)wg, block_width, rb, ib, lam, decay_scale, state, C, taps, state_slots)
  if (dtype == ZI_F32 && wg_dtype == ZI_F32) ZI_RGLRU_DECODE(float, float);
  else if (dtype == ZI_F32 && wg_dtype == ZI_BF16) ZI_RGLRU_DECODE(float, bf);
  else if (dtype == ZI_BF16 && wg_dtype == ZI_F32) ZI_RGLRU_DECODE(bf, float);
  else if (dtype == ZI_BF16 && wg_dtype == ZI_BF16) ZI_RGLRU_DECODE(bf, bf);
  else return zi_refuse("rglru_decode: unknown dtype tags %d, %d", dtype, wg_dtype);
#undef ZI_RGLRU_DECODE
  return zi_check_launch("rglru_decode");
}

extern "C" long long zi_rglru_chunked_workspace_floats(int T, int C, int n_seqs, int chunk) {
  const long long n_chunks = (T + chunk - 1) / chunk;
  return 3 * n_chunks * C + (long long)n_seqs * C;
}

extern "C" int zi_rglru_scan_chunked(void* out, int ldo, float* work, const float* u, const float* gates, int block_width,
                                     const float* rb, const float* ib, const float* lam, float decay_scale, const void* y,
                                     int ldy, const float* yb, const void* x, int ldx, const float* xb, int dtype,
                                     float* state, int C, int taps, const int* cu_q, const int* state_slots, int n_seqs,
                                     int T, int chunk, cudaStream_t stream) {
  if (n_seqs <= 0 || T <= 0) return 0;
  if (taps < 1 || taps > 9) return zi_refuse("rglru_scan: 1 to 9 taps, got %d", taps);
  if (chunk < 1) return zi_refuse("rglru_scan: chunks of %d tokens", chunk);
  if (block_width <= 0 || C % block_width) return zi_refuse("rglru_scan: %d channels do not divide into blocks of %d", C, block_width);
  const int n_chunks = (T + chunk - 1) / chunk;
  float* ab = work;                                   // [n_chunks][2][C]
  float* s_in = work + (size_t)2 * n_chunks * C;      // [n_chunks][C]
  float* last = s_in + (size_t)n_chunks * C;          // [n_seqs][C]
  dim3 grid((C + 127) / 128, n_chunks);
  ZI_DISPATCH_DTYPE(dtype, TT, {
    zi_launch(rglru_chunk_kernel<TT, false>, dim3(grid), dim3(128), 0, stream, (TT*)out, ldo, ab, (const float*)s_in, last, u,
              gates, block_width, rb, ib, lam, decay_scale, (const TT*)y, ldy, yb, (const float*)state, C, taps, cu_q,
              state_slots, n_seqs, T, chunk);
    zi_launch(rglru_carry_kernel, dim3((C + 127) / 128), dim3(128), 0, stream, s_in, (const float*)ab, C, n_chunks);
    zi_launch(rglru_chunk_kernel<TT, true>, dim3(grid), dim3(128), 0, stream, (TT*)out, ldo, ab, (const float*)s_in, last, u,
              gates, block_width, rb, ib, lam, decay_scale, (const TT*)y, ldy, yb, (const float*)state, C, taps, cu_q,
              state_slots, n_seqs, T, chunk);
    zi_launch(rglru_finish_kernel<TT>, dim3((C + 127) / 128, n_seqs), dim3(128), 0, stream, state, (const float*)last,
              (const TT*)x, ldx, xb, C, taps, cu_q, state_slots);
  });
  return zi_check_launch("rglru_scan_chunked");
}

extern "C" int zi_causal_conv(float* u, const void* x, int ldx, int dtype, const float* xb, const float* kern,
                              const float* cb, const float* state, int C, int taps, const int* cu_q,
                              const int* state_slots, int n_seqs, int T, cudaStream_t stream) {
  if (T <= 0 || n_seqs <= 0) return 0;
  if (taps < 1 || taps > 9) return zi_refuse("causal_conv: 1 to 9 taps, got %d", taps);
  dim3 grid((C + 127) / 128, T);
  ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(causal_conv_kernel<TT>, dim3(grid), dim3(128), 0, stream, u, (const TT*)x, ldx, xb,
                                         kern, cb, state, C, taps, cu_q, state_slots, n_seqs));
  return zi_check_launch("causal_conv");
}

extern "C" int zi_rglru_scan(void* out, int ldo, const float* u, const float* gates, int block_width, const float* rb,
                             const float* ib, const float* lam, float decay_scale, const void* y, int ldy,
                             const float* yb, const void* x, int ldx, const float* xb, int dtype, float* state, int C,
                             int taps, const int* cu_q, const int* state_slots, int n_seqs, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (taps < 1 || taps > 9) return zi_refuse("rglru_scan: 1 to 9 taps, got %d", taps);
  if (block_width <= 0 || C % block_width) return zi_refuse("rglru_scan: %d channels do not divide into blocks of %d", C, block_width);
  dim3 grid((C + 127) / 128, n_seqs);
  ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(rglru_scan_kernel<TT>, dim3(grid), dim3(128), 0, stream, (TT*)out, ldo, u, gates,
                                         block_width, rb, ib, lam, decay_scale, (const TT*)y, ldy, yb, (const TT*)x, ldx,
                                         xb, state, C, taps, cu_q, state_slots));
  return zi_check_launch("rglru_scan");
}

ZI_TRACE_SETTER(recurrent)
