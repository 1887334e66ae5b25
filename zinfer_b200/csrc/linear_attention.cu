// Kernels of mixers that keep a matrix-valued state per head instead of keys (linear attention
// with a decay per key channel, with or without the delta rule), and of the short convolutions and
// the gated per-head norm around them.
//
// The recurrence, per head, with S [D key channels, V value channels] carried per request:
//     S <- diag(g_t) S                      the decay acts on the rows that belong to key channels
//     u_t = v_t                             plain form
//     u_t = beta_t (v_t - S^T k_t)          delta rule
//     S <- S + k_t u_t^T ;  o_t = S^T (q_scale q_t)
// Everything here is 32-bit arithmetic.  A request's tokens of this step are rows cu_q[s] ..
// cu_q[s+1]-1 of the flat batch and continue the request from slot state_slots[s].  Each column of S
// is visited by one group of lanes, token after token, in an order that depends on D alone, so a
// result depends neither on how the request was cut into steps nor on the batch.
#include "api.h"
#include "common.cuh"

namespace {

__device__ __forceinline__ float softplus_f32(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f32(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float log_sigmoid_f32(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

__device__ __forceinline__ int seq_of_token(const int* __restrict__ cu_q, int n_seqs, int t) {
  int s = 0, hi = n_seqs - 1;          // cu_q[s] <= t < cu_q[s+1]
  while (s < hi) {
    const int mid = (s + hi + 1) >> 1;
    if (cu_q[mid] <= t) s = mid; else hi = mid - 1;
  }
  return s;
}

// ------------------------------------------------------------------ short causal convolution
// y[t, c] = act(sum_j kern[c, j] * x[t - (taps-1-j), c]), inputs before the step's first token from the
// carried rows tail[slot][taps-1][C] (oldest first), one thread per (token, channel).
template <typename T>
__global__ void short_conv_kernel(float* __restrict__ y, int ldy, const T* __restrict__ x, int ldx,
                                  const float* __restrict__ kern, const float* __restrict__ tail,
                                  long long slot_stride, int C, int taps, int act, const int* __restrict__ cu_q,
                                  const int* __restrict__ state_slots, int n_seqs) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int s = seq_of_token(cu_q, n_seqs, t);
  const int tok0 = cu_q[s], tl = t - tok0;
  const float* st = tail + (size_t)state_slots[s] * slot_stride;
  float acc = 0.f;
  for (int j = 0; j < taps; ++j) {
    const int src = tl - (taps - 1 - j);
    float v;
    if (src >= 0) v = to_f32(x[(size_t)(tok0 + src) * ldx + c]);
    else v = st[(size_t)(taps - 1 + src) * C + c];      // src = -1: the newest carried input, row taps-2
    acc = fmaf(kern[(size_t)c * taps + j], v, acc);
  }
  if (act == 1) acc = acc * sigmoid_f32(acc);
  y[(size_t)t * ldy + c] = acc;
}

// The carried rows after the step: the last taps-1 inputs of each request, one thread per (request, channel).
// Row r takes an index above r, so ascending r may overwrite in place.
template <typename T>
__global__ void short_conv_carry_kernel(float* __restrict__ tail, long long slot_stride, const T* __restrict__ x, int ldx,
                                        int C, int taps, const int* __restrict__ cu_q,
                                        const int* __restrict__ state_slots, int n_seqs) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C || s >= n_seqs) return;
  const int tok0 = cu_q[s], qlen = cu_q[s + 1] - tok0;
  if (qlen <= 0) return;
  float* st = tail + (size_t)state_slots[s] * slot_stride;
  for (int r = 0; r < taps - 1; ++r) {
    const int src = qlen - (taps - 1) + r;
    st[(size_t)r * C + c] = src >= 0 ? to_f32(x[(size_t)(tok0 + src) * ldx + c]) : st[(size_t)(r + qlen) * C + c];
  }
}

// ------------------------------------------------------------------------------- decays
// mode 0: g = sigmoid(z + bias)^(inv_tau) = exp(log_sigmoid(z + bias) * inv_tau)
// mode 1: g = exp(-exp(a_log[head]) * softplus(z + bias)), head = column / D
__global__ void decay_kernel(float* __restrict__ z, size_t total, int N, int D, const float* __restrict__ bias,
                             const float* __restrict__ a_log, float inv_tau, int mode) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int c = (int)(idx % N);
  const float x = z[idx] + (bias ? bias[c] : 0.f);
  z[idx] = mode == 0 ? expf(log_sigmoid_f32(x) * inv_tau) : expf(-expf(a_log[c / D]) * softplus_f32(x));
}

// x[t, head, :] <- scale * x / sqrt(sum(x^2) + eps), one warp per (token, head), in place
__global__ void unit_norm_kernel(float* __restrict__ x, int ld, int T, int heads, int d, float eps, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (w >= T * heads) return;
  float* p = x + (size_t)(w / heads) * ld + (size_t)(w % heads) * d;
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) ss = fmaf(p[i], p[i], ss);
  ss = warp_sum(ss);
  const float r = scale / sqrtf(ss + eps);
  for (int i = lane; i < d; i += 32) p[i] *= r;
}

template <typename T>
__global__ void sigmoid_rows_kernel(float* __restrict__ out, int ldo, const T* __restrict__ x, int ldx, int rows, int W) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)rows * W) return;
  const int r = (int)(idx / W), c = (int)(idx % W);
  out[(size_t)r * ldo + c] = sigmoid_f32(to_f32(x[(size_t)r * ldx + c]));
}

// --------------------------------------------------------------------------- the recurrence
// Block: one request, one head, CB neighbouring value channels; 8 warps.  A column of S (D key channels of one
// value channel) belongs to P neighbouring lanes of one warp, R = 8 (or 16) rows each, in registers, and every
// lane works on NC = 2 columns at once (two independent chains of arithmetic per lane); the sums over a column's
// rows meet by a butterfly of shuffles over those P lanes (a fixed order), so nothing in the loop over tokens
// waits for another warp.  q, k and the decays of TB tokens at a time are staged in shared memory for the whole
// block, laid out so that the lanes' 16-byte reads fall into different banks; the next TB tokens are fetched
// into registers while these are worked on and stored afterwards (one barrier per TB tokens).
constexpr int LR_WARPS = 8, LR_THREADS = LR_WARPS * 32, TB = 16, NC = 2;

template <typename TQ, typename TV, int R, bool DELTA>
__global__ void __launch_bounds__(LR_THREADS)
linear_recurrence_kernel(float* __restrict__ out, int ldo, const TQ* __restrict__ q, int ldq, const TQ* __restrict__ k,
                         int ldk, const TV* __restrict__ v, int ldv, const float* __restrict__ decay, int ldg,
                         const float* __restrict__ beta, int ldb, float q_scale, float* __restrict__ state,
                         long long slot_stride, int H, int G, int D, int V, int P, const int* __restrict__ cu_q,
                         const int* __restrict__ state_slots) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float sm[];
  const int DP = P * R;                           // key channels rounded up to whole parts
  const int CW = (32 / P) * NC, CB = LR_WARPS * CW;   // columns per warp and per block
  const int BUF = 3 * TB * DP + TB * CB + TB;     // one staging buffer: q, k, g [TB][DP], v [TB][CB], beta [TB]
  const int s = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * CB;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int p = lane % P, cw = lane / P;
  const int cb = warp * CW + cw * NC, col = j0 + cb;   // this lane's first column within the block, and of the head
  const int kvh = h / (H / G);
  const int tok0 = cu_q[s], qlen = cu_q[s + 1] - tok0;
  if (qlen <= 0) return;
  float* S = state + (size_t)state_slots[s] * slot_stride + (size_t)h * D * V;
  float Sr[NC][R];
#pragma unroll
  for (int c = 0; c < NC; ++c)
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int i = p * R + r;
      Sr[c][r] = (i < D && col + c < V) ? S[(size_t)i * V + col + c] : 0.f;
    }
  // DP and CB are powers of two: shifts instead of divisions
  const int lgDP = 31 - __clz(DP), lgCB = 31 - __clz(CB), lgP = 31 - __clz(P);
  // Key channel i = p R + 4 r4 + x lies at ((r4 P + p) 4 + x) of its token's row: for one r4 the P lanes of a column
  // read neighbouring 16-byte pieces.
  constexpr int LGR = R == 8 ? 3 : 4;
  auto place = [&](int i) { return ((((i >> 2) & (R / 4 - 1)) << lgP) + (i >> LGR)) * 4 + (i & 3); };
  // Staging in two halves: fetch() takes the first NPF elements per thread of q, k and the decays (all of them
  // while DP <= 128) and the first two of v into registers as they are stored; put() widens and stores them, and
  // fetches and stores whatever is left beyond them.
  constexpr int NPF = 8, NPV = 2;
  TQ fq[NPF], fk[NPF];
  TV fv[NPV];
  float fg[NPF], fb = 1.f;
  auto fetch = [&](int t0, int nt) {
    const int total = nt << lgDP;
#pragma unroll
    for (int u = 0; u < NPF; ++u) {
      const int e = tid + u * LR_THREADS;
      const int tt = e >> lgDP, i = e & (DP - 1);
      if (e < total && i < D) {
        const size_t row = (size_t)(tok0 + t0 + tt);
        fq[u] = q[row * ldq + (size_t)kvh * D + i];
        fk[u] = k[row * ldk + (size_t)kvh * D + i];
        fg[u] = decay[row * ldg + (size_t)h * D + i];
      } else {
        fq[u] = from_f32<TQ>(0.f);
        fk[u] = from_f32<TQ>(0.f);
        fg[u] = 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < NPV; ++u) {
      const int e = tid + u * LR_THREADS;
      const int c = j0 + (e & (CB - 1));
      fv[u] = (e < (nt << lgCB) && c < V) ? v[(size_t)(tok0 + t0 + (e >> lgCB)) * ldv + (size_t)h * V + c] : from_f32<TV>(0.f);
    }
    if (DELTA && tid < nt) fb = beta[(size_t)(tok0 + t0 + tid) * ldb + h];
  };
  auto put = [&](int t0, int nt, float* buf) {
    const int total = nt << lgDP;
#pragma unroll
    for (int u = 0; u < NPF; ++u) {
      const int e = tid + u * LR_THREADS;
      if (e < total) {
        const int at = (e & ~(DP - 1)) + place(e & (DP - 1));
        buf[at] = to_f32(fq[u]) * q_scale;
        buf[TB * DP + at] = to_f32(fk[u]);
        buf[2 * TB * DP + at] = fg[u];
      }
    }
    for (int e = tid + NPF * LR_THREADS; e < total; e += LR_THREADS) {      // beyond the registers (DP > 128)
      const int tt = e >> lgDP, i = e & (DP - 1);
      const size_t row = (size_t)(tok0 + t0 + tt);
      const bool in = i < D;
      const int at = (e & ~(DP - 1)) + place(i);
      buf[at] = in ? to_f32(q[row * ldq + (size_t)kvh * D + i]) * q_scale : 0.f;
      buf[TB * DP + at] = in ? to_f32(k[row * ldk + (size_t)kvh * D + i]) : 0.f;
      buf[2 * TB * DP + at] = in ? decay[row * ldg + (size_t)h * D + i] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < NPV; ++u) {
      const int e = tid + u * LR_THREADS;
      if (e < (nt << lgCB)) buf[3 * TB * DP + e] = to_f32(fv[u]);
    }
    for (int e = tid + NPV * LR_THREADS; e < (nt << lgCB); e += LR_THREADS) {
      const int c = j0 + (e & (CB - 1));
      buf[3 * TB * DP + e] = c < V ? to_f32(v[(size_t)(tok0 + t0 + (e >> lgCB)) * ldv + (size_t)h * V + c]) : 0.f;
    }
    if (tid < nt) buf[3 * TB * DP + TB * CB + tid] = fb;
  };
  fetch(0, min(TB, qlen));
  put(0, min(TB, qlen), sm);
  __syncthreads();
  int cur = 0;
  for (int t0 = 0; t0 < qlen; t0 += TB) {
    const int nt = min(TB, qlen - t0);
    const float* buf = sm + cur * BUF;
    // the next batch's loads go out now and land in the other buffer after this batch's work; nobody reads that
    // buffer before the barrier at the end of this iteration
    const bool more = t0 + TB < qlen;
    if (more) fetch(t0 + TB, min(TB, qlen - t0 - TB));
    const float* vs = buf + 3 * TB * DP;
    const float* bs = vs + TB * CB;
    for (int tt = 0; tt < nt; ++tt) {
      const float4* qt = reinterpret_cast<const float4*>(buf + tt * DP) + p;
      const float4* kt = reinterpret_cast<const float4*>(buf + TB * DP + tt * DP) + p;
      const float4* gt = reinterpret_cast<const float4*>(buf + 2 * TB * DP + tt * DP) + p;
      float a[NC], b[NC], kq = 0.f;      // (g S)^T k and (g S)^T q per column, k . q, over this lane's rows
#pragma unroll
      for (int c = 0; c < NC; ++c) a[c] = b[c] = 0.f;
      float kr[R];
#pragma unroll
      for (int r4 = 0; r4 < R / 4; ++r4) {
        const float4 g4 = gt[r4 << lgP], k4 = kt[r4 << lgP], q4 = qt[r4 << lgP];
        kr[4 * r4] = k4.x; kr[4 * r4 + 1] = k4.y; kr[4 * r4 + 2] = k4.z; kr[4 * r4 + 3] = k4.w;
        kq = fmaf(k4.x, q4.x, fmaf(k4.y, q4.y, fmaf(k4.z, q4.z, fmaf(k4.w, q4.w, kq))));
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          float* sr = Sr[c] + 4 * r4;
          sr[0] *= g4.x; sr[1] *= g4.y; sr[2] *= g4.z; sr[3] *= g4.w;
          if (DELTA) a[c] = fmaf(sr[0], k4.x, fmaf(sr[1], k4.y, fmaf(sr[2], k4.z, fmaf(sr[3], k4.w, a[c]))));
          b[c] = fmaf(sr[0], q4.x, fmaf(sr[1], q4.y, fmaf(sr[2], q4.z, fmaf(sr[3], q4.w, b[c]))));
        }
      }
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {       // the column's P lanes are neighbours: every lane ends with the sums
        if (o < P) {
#pragma unroll
          for (int c = 0; c < NC; ++c) {
            if (DELTA) a[c] += __shfl_xor_sync(0xffffffffu, a[c], o);
            b[c] += __shfl_xor_sync(0xffffffffu, b[c], o);
          }
          kq += __shfl_xor_sync(0xffffffffu, kq, o);
        }
      }
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const float vj = vs[tt * CB + cb + c];
        const float u = DELTA ? bs[tt] * (vj - a[c]) : vj;
#pragma unroll
        for (int r = 0; r < R; ++r) Sr[c][r] = fmaf(kr[r], u, Sr[c][r]);
        if (p == 0 && col + c < V) out[(size_t)(tok0 + t0 + tt) * ldo + (size_t)h * V + col + c] = fmaf(u, kq, b[c]);
      }
    }
    if (more) put(t0 + TB, min(TB, qlen - t0 - TB), sm + (cur ^ 1) * BUF);
    __syncthreads();     // the other buffer is filled, and this one is free for the batch after it
    cur ^= 1;
  }
#pragma unroll
  for (int c = 0; c < NC; ++c)
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int i = p * R + r;
      if (i < D && col + c < V) S[(size_t)i * V + col + c] = Sr[c][r];
    }
}

// ----------------------------------------------------------------------- gated per-head norm
// out[t, head, :] = o / sqrt(mean(o^2) + eps) * w * act(gate[t, head, :]); act: 0 silu, 1 sigmoid.
// One warp per (token, head).
template <typename TG, typename TO>
__global__ void head_norm_gate_kernel(TO* __restrict__ out, int ldo, const float* __restrict__ o, int ldi,
                                      const float* __restrict__ w, float eps, const TG* __restrict__ gate, int ldgate,
                                      int act, int T, int heads, int V) {
  pdl_launch_dependents();
  pdl_wait();
  const int wi = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (wi >= T * heads) return;
  const int t = wi / heads, h = wi % heads;
  const float* p = o + (size_t)t * ldi + (size_t)h * V;
  float ss = 0.f;
  for (int i = lane; i < V; i += 32) ss = fmaf(p[i], p[i], ss);
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)V + eps);
  for (int i = lane; i < V; i += 32) {
    const float g = to_f32(gate[(size_t)t * ldgate + (size_t)h * V + i]);
    const float a = act == 0 ? g * sigmoid_f32(g) : sigmoid_f32(g);
    out[(size_t)t * ldo + (size_t)h * V + i] = from_f32<TO>(p[i] * inv * w[i] * a);
  }
}
}  // namespace

extern "C" int zi_short_conv(float* y, int ldy, const void* x, int ldx, int dtype, const float* kern, const float* tail,
                             long long slot_stride, int C, int taps, int act, const int* cu_q, const int* state_slots,
                             int n_seqs, int T, cudaStream_t stream) {
  if (T <= 0 || C <= 0) return 0;
  if (taps < 1 || taps > 64) return zi_refuse("short_conv: %d taps", taps);
  dim3 grid((C + 127) / 128, T);
  ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(short_conv_kernel<TT>, dim3(grid), dim3(128), 0, stream, y, ldy, (const TT*)x, ldx,
                                         kern, tail, slot_stride, C, taps, act, cu_q, state_slots, n_seqs));
  return zi_check_launch("short_conv");
}

extern "C" int zi_short_conv_carry(float* tail, long long slot_stride, const void* x, int ldx, int dtype, int C, int taps,
                                   const int* cu_q, const int* state_slots, int n_seqs, cudaStream_t stream) {
  if (n_seqs <= 0 || C <= 0 || taps <= 1) return 0;
  dim3 grid((C + 127) / 128, n_seqs);
  ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(short_conv_carry_kernel<TT>, dim3(grid), dim3(128), 0, stream, tail, slot_stride,
                                         (const TT*)x, ldx, C, taps, cu_q, state_slots, n_seqs));
  return zi_check_launch("short_conv_carry");
}

extern "C" int zi_decay(float* z, long long rows, int N, int D, const float* bias, const float* a_log, float inv_tau,
                        int mode, cudaStream_t stream) {
  const size_t total = (size_t)rows * N;
  if (total == 0) return 0;
  if (mode != 0 && mode != 1) return zi_refuse("decay: unknown mode %d", mode);
  if (mode == 1 && (!a_log || D <= 0 || N % D)) return zi_refuse("decay: the per-head form needs a_log and whole heads");
  zi_launch(decay_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, z, total, N, D, bias, a_log, inv_tau, mode);
  return zi_check_launch("decay");
}

extern "C" int zi_unit_norm(float* x, int ld, int T, int heads, int d, float eps, float scale, cudaStream_t stream) {
  if (T <= 0 || heads <= 0) return 0;
  const int warps = 4;
  zi_launch(unit_norm_kernel, dim3((unsigned)((T * heads + warps - 1) / warps)), dim3(warps * 32), 0, stream, x, ld, T, heads, d,
            eps, scale);
  return zi_check_launch("unit_norm");
}

extern "C" int zi_sigmoid_rows(float* out, int ldo, const void* x, int ldx, int dtype, int rows, int W, cudaStream_t stream) {
  const size_t total = (size_t)rows * W;
  if (total == 0) return 0;
  ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(sigmoid_rows_kernel<TT>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream,
                                         out, ldo, (const TT*)x, ldx, rows, W));
  return zi_check_launch("sigmoid_rows");
}

extern "C" int zi_linear_recurrence(float* out, int ldo, const void* q, int ldq, const void* k, int ldk, int qk_dtype,
                                    const void* v, int ldv, int v_dtype, const float* decay, int ldg, const float* beta,
                                    int ldb, float q_scale, float* state, long long slot_stride, int H, int G, int D,
                                    int V, int delta, const int* cu_q, const int* state_slots, int n_seqs,
                                    cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G) return zi_refuse("linear_recurrence: %d heads do not divide into %d key heads", H, G);
  if (D <= 0 || D > 512 || V <= 0) return zi_refuse("linear_recurrence: %d key channels (1..512), %d value channels", D, V);
  if (delta && !beta) return zi_refuse("linear_recurrence: the delta rule needs beta");
  // R rows of a column per lane, P lanes per column (a power of two: the sums meet by a butterfly of shuffles)
  const int R = D <= 256 ? 8 : 16;
  int P = 1;
  while (P * R < D) P <<= 1;
  const int CB = LR_WARPS * (32 / P) * NC;
  const size_t smem = (size_t)2 * (3 * TB * P * R + TB * CB + TB) * sizeof(float);
  dim3 grid(n_seqs, H, (V + CB - 1) / CB), block(LR_THREADS);
#define ZI_LR(TQ, TV, RR, DD)                                                                                          \
  do {                                                                                                                 \
    auto kern = linear_recurrence_kernel<TQ, TV, RR, DD>;                                                              \
    if (smem > 48 * 1024) {                                                                                            \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)           \
        return zi_refuse("linear_recurrence: cannot get %zu bytes of shared memory", smem);                            \
    }                                                                                                                  \
    zi_launch(kern, dim3(grid), dim3(block), smem, stream, out, ldo, (const TQ*)q, ldq, (const TQ*)k, ldk, (const TV*)v, \
              ldv, decay, ldg, beta, ldb, q_scale, state, slot_stride, H, G, D, V, P, cu_q, state_slots);              \
  } while (0)
#define ZI_LR_R(TQ, TV)                                          \
  do {                                                           \
    if (R == 8) { if (delta) ZI_LR(TQ, TV, 8, true); else ZI_LR(TQ, TV, 8, false); } \
    else { if (delta) ZI_LR(TQ, TV, 16, true); else ZI_LR(TQ, TV, 16, false); }         \
  } while (0)
  if (qk_dtype == ZI_F32 && v_dtype == ZI_F32) ZI_LR_R(float, float);
  else if (qk_dtype == ZI_BF16 && v_dtype == ZI_BF16) ZI_LR_R(__nv_bfloat16, __nv_bfloat16);
  else if (qk_dtype == ZI_F32 && v_dtype == ZI_BF16) ZI_LR_R(float, __nv_bfloat16);
  else return zi_refuse("linear_recurrence: operand types %d and %d", qk_dtype, v_dtype);
#undef ZI_LR_R
#undef ZI_LR
  return zi_check_launch("linear_recurrence");
}

extern "C" int zi_head_norm_gate(void* out, int out_dtype, int ldo, const float* o, int ldi, const float* w, float eps,
                                 const void* gate, int gate_dtype, int ldgate, int act, int T, int heads, int V,
                                 cudaStream_t stream) {
  if (T <= 0 || heads <= 0) return 0;
  if (act != 0 && act != 1) return zi_refuse("head_norm_gate: unknown gate %d", act);
  const int warps = 4;
  dim3 grid((unsigned)(((size_t)T * heads + warps - 1) / warps));
  ZI_DISPATCH_DTYPE(gate_dtype, TG, ZI_DISPATCH_DTYPE(out_dtype, TO,
      zi_launch(head_norm_gate_kernel<TG, TO>, dim3(grid), dim3(warps * 32), 0, stream, (TO*)out, ldo, o, ldi, w, eps,
                (const TG*)gate, ldgate, act, T, heads, V)));
  return zi_check_launch("head_norm_gate");
}

ZI_TRACE_SETTER(linear_attention)
