// Recurrent mixers with a matrix state per (request, head): the state S [d x dv] lives in a
// slot of 32-bit floats, is loaded once per step into registers, advanced token by token over
// the request's new tokens, and stored back. Prompt portions and single decoded tokens are the
// same kernel; what a request brings is read from cu_q on the device.
//
// Work split: a CTA owns (request, head, block of 32 value columns); warp j owns the key rows
// j, j + W, j + 2W, ... (W warps, 32 rows each), lane c the column c of the block, so a thread
// keeps 32 elements of S in registers. A read-out sum over the key rows is a sum over the
// thread's registers plus one exchange between the warps through shared memory. The next
// token's operands are fetched while the current one is computed (two buffers), so a token
// costs one block barrier (two for the delta rule, whose write depends on a read).
//
//  * mLSTM: m' = max(f + m, i); S <- e^(f + m - m') S + e^(i - m') k v^T; n likewise with k;
//    o = S^T q / (max(|n.q|, e^(-m')) + 1e-6), with log gates i = cap tanh(a_i / cap) and
//    f = logsigmoid(cap tanh(a_f / cap)). The normaliser n is kept one row per lane.
//  * gated delta rule with a decay per key channel: S <- diag(g) S; u = beta (v - S^T k);
//    S <- S + k u^T; o = S^T q, with q and k scaled to unit length (q also by q_scale) and
//    g = exp(-exp(A_log) softplus(a + dt_bias)). The unit scalings are applied to the sums,
//    not to the vectors: S^T (k/|k|) = (S^T k)/|k|.
//  * the short causal convolution with SiLU in front of it, whose last taps-1 inputs are state too.
#define TS_PDL_CLASS PDL_OTHER
#include "common.cuh"

namespace ts {

constexpr int SCAN_MAX_TAPS = 8;
constexpr int SCAN_MAX_KEY_DIM = 256;   // 8 warps of 32 key rows: what the register file holds of S per CTA

__device__ __forceinline__ float softplusf(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float logsigmoidf(float z) { return z < 0.f ? z - log1pf(expf(z)) : -log1pf(expf(-z)); }

// ------------------------------------------------------------------------ mLSTM
template <typename T>
__global__ void mlstm_scan_kernel(const T* __restrict__ qkv, int stride, int q_off, int k_off, int v_off,
                                  const float* __restrict__ gates, const float* __restrict__ gate_bias, float cap,
                                  float q_scale, float* __restrict__ state, int state_stride,
                                  const int* __restrict__ cu_q, const int* __restrict__ state_slots, int H, int d,
                                  int dv, float* __restrict__ out) {
  extern __shared__ float sm[];
  const int W = blockDim.x >> 5, dpad = W * 32;
  float* qs = sm;                    // [2][dpad]
  float* ks = qs + 2 * dpad;         // [2][dpad]
  float* vs = ks + 2 * dpad;         // [2][32]
  float* part = vs + 64;             // [2][W][32]
  float* nqp = part + 2 * W * 32;    // [2][W]
  const int b = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * 32;
  const int tid = threadIdx.x, lane = tid & 31, j = tid >> 5;
  pdl_trigger();
  pdl_wait();
  const int start = cu_q[b], end = cu_q[b + 1];
  if (end <= start) return;
  const int slot = state_slots[b];
  const int col = c0 + lane;
  const bool col_ok = col < dv;
  // per head: S [d][dv], then one copy of (n [d], m) per column block, so that the CTAs of a
  // head share nothing that one of them writes
  float* S = state + (size_t)slot * state_stride + (size_t)h * ((size_t)d * dv + (size_t)gridDim.z * (d + 1));
  float* nvec = S + (size_t)d * dv + (size_t)blockIdx.z * (d + 1);
  float* mptr = nvec + d;
  float s[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int r = j + W * i;
    s[i] = (r < d && col_ok) ? S[(size_t)r * dv + col] : 0.f;
  }
  const int rn = j + W * lane;       // the row of n this lane keeps
  float n = rn < d ? nvec[rn] : 0.f;
  float m = *mptr;
  float fq, fk, fv = 0.f;
  auto fetch = [&](int t) {
    const T* row = qkv + (size_t)t * stride;
    fq = tid < d ? to_float(row[q_off + h * d + tid]) * q_scale : 0.f;
    fk = tid < d ? to_float(row[k_off + h * d + tid]) : 0.f;
    if (tid < 32) fv = (c0 + tid < dv) ? to_float(row[v_off + h * dv + c0 + tid]) : 0.f;
  };
  fetch(start);
  qs[tid] = fq;
  ks[tid] = fk;
  if (tid < 32) vs[tid] = fv;
  __syncthreads();
  for (int t = start; t < end; ++t) {
    const int cur = (t - start) & 1, nxt = cur ^ 1;
    if (t + 1 < end) fetch(t + 1);
    const float ai = gates[(size_t)t * 2 * H + h] + gate_bias[h];
    const float af = gates[(size_t)t * 2 * H + H + h] + gate_bias[H + h];
    const float li = cap * tanhf(ai / cap);
    const float lf = logsigmoidf(cap * tanhf(af / cap));
    const float m_new = fmaxf(lf + m, li);
    const float keep = expf(lf + m - m_new), take = expf(li - m_new);
    m = m_new;
    const float* q_ = qs + cur * dpad;
    const float* k_ = ks + cur * dpad;
    const float tv = take * vs[cur * 32 + lane];
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int r = j + W * i;
      s[i] = fmaf(keep, s[i], k_[r] * tv);
      acc = fmaf(s[i], q_[r], acc);
    }
    n = fmaf(keep, n, take * k_[rn]);
    const float nq = warp_sum(n * q_[rn]);
    part[(cur * W + j) * 32 + lane] = acc;
    if (lane == 0) nqp[cur * W + j] = nq;
    if (t + 1 < end) {
      qs[nxt * dpad + tid] = fq;
      ks[nxt * dpad + tid] = fk;
      if (tid < 32) vs[nxt * 32 + tid] = fv;
    }
    __syncthreads();
    if (j == 0 && col_ok) {
      float num = 0.f, nqs = 0.f;
      for (int w = 0; w < W; ++w) {
        num += part[(cur * W + w) * 32 + lane];
        nqs += nqp[cur * W + w];
      }
      out[((size_t)t * H + h) * dv + col] = num / (fmaxf(fabsf(nqs), expf(-m)) + 1e-6f);
    }
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int r = j + W * i;
    if (r < d && col_ok) S[(size_t)r * dv + col] = s[i];
  }
  if (rn < d) nvec[rn] = n;
  if (tid == 0) *mptr = m;
}

// ------------------------------------------------------------------- delta rule
__global__ void delta_scan_kernel(const float* __restrict__ qkv, int stride, int q_off, int k_off, int v_off,
                                  const float* __restrict__ a, const float* __restrict__ dt_bias,
                                  const float* __restrict__ a_log, const float* __restrict__ beta_pre,
                                  float q_scale, float* __restrict__ state, int state_stride,
                                  const int* __restrict__ cu_q, const int* __restrict__ state_slots, int H, int G,
                                  int d, int dv, float* __restrict__ out) {
  extern __shared__ float sm[];
  const int W = blockDim.x >> 5, dpad = W * 32;
  float* qs = sm;                    // [2][dpad]
  float* ks = qs + 2 * dpad;
  float* gs = ks + 2 * dpad;
  float* vs = gs + 2 * dpad;         // [2][32]
  float* p1 = vs + 64;               // [2][W][32]
  float* p2 = p1 + 2 * W * 32;
  float* ksq = p2 + 2 * W * 32;      // [2][W]
  float* qsq = ksq + 2 * W;
  const int b = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * 32;
  const int g = h / (H / G);
  const int tid = threadIdx.x, lane = tid & 31, j = tid >> 5;
  pdl_trigger();
  pdl_wait();
  const int start = cu_q[b], end = cu_q[b + 1];
  if (end <= start) return;
  const int slot = state_slots[b];
  const int col = c0 + lane;
  const bool col_ok = col < dv;
  float* S = state + (size_t)slot * state_stride + (size_t)h * d * dv;
  float s[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int r = j + W * i;
    s[i] = (r < d && col_ok) ? S[(size_t)r * dv + col] : 0.f;
  }
  const int rn = j + W * lane;
  const float A = expf(a_log[h]);
  const float bias = tid < d ? dt_bias[h * d + tid] : 0.f;
  float fq, fk, fg, fv = 0.f;
  auto fetch = [&](int t) {
    const float* row = qkv + (size_t)t * stride;
    fq = tid < d ? row[q_off + g * d + tid] : 0.f;
    fk = tid < d ? row[k_off + g * d + tid] : 0.f;
    fg = tid < d ? expf(-A * softplusf(a[((size_t)t * H + h) * d + tid] + bias)) : 1.f;
    if (tid < 32) fv = (c0 + tid < dv) ? row[v_off + h * dv + c0 + tid] : 0.f;
  };
  fetch(start);
  qs[tid] = fq;
  ks[tid] = fk;
  gs[tid] = fg;
  if (tid < 32) vs[tid] = fv;
  __syncthreads();
  for (int t = start; t < end; ++t) {
    const int cur = (t - start) & 1, nxt = cur ^ 1;
    if (t + 1 < end) fetch(t + 1);
    const float z = beta_pre[(size_t)t * H + h];
    const float beta = 1.f / (1.f + expf(-z));
    const float* q_ = qs + cur * dpad;
    const float* k_ = ks + cur * dpad;
    const float* g_ = gs + cur * dpad;
    float p = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int r = j + W * i;
      s[i] *= g_[r];
      p = fmaf(s[i], k_[r], p);
    }
    const float kk = warp_sum(k_[rn] * k_[rn]);
    const float qq = warp_sum(q_[rn] * q_[rn]);
    p1[(cur * W + j) * 32 + lane] = p;
    if (lane == 0) {
      ksq[cur * W + j] = kk;
      qsq[cur * W + j] = qq;
    }
    __syncthreads();
    float pred = 0.f, ksum = 0.f;
    for (int w = 0; w < W; ++w) {
      pred += p1[(cur * W + w) * 32 + lane];
      ksum += ksq[cur * W + w];
    }
    const float rk = rsqrtf(ksum + 1e-6f);
    const float wu = beta * (vs[cur * 32 + lane] - pred * rk) * rk;
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int r = j + W * i;
      s[i] = fmaf(k_[r], wu, s[i]);
      o = fmaf(s[i], q_[r], o);
    }
    p2[(cur * W + j) * 32 + lane] = o;
    if (t + 1 < end) {
      qs[nxt * dpad + tid] = fq;
      ks[nxt * dpad + tid] = fk;
      gs[nxt * dpad + tid] = fg;
      if (tid < 32) vs[nxt * 32 + tid] = fv;
    }
    __syncthreads();
    if (j == 0 && col_ok) {
      float osum = 0.f, qsum = 0.f;
      for (int w = 0; w < W; ++w) {
        osum += p2[(cur * W + w) * 32 + lane];
        qsum += qsq[cur * W + w];
      }
      out[((size_t)t * H + h) * dv + col] = osum * rsqrtf(qsum + 1e-6f) * q_scale;
    }
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int r = j + W * i;
    if (r < d && col_ok) S[(size_t)r * dv + col] = s[i];
  }
}

// ------------------------------------------------- short causal convolution + SiLU
// Input of token tau of request b, channel c: x[tau][c] for tokens of this step, the state's
// row (K - 1) + (tau - start) for the K - 1 tokens before it (zero at a request's start).
template <typename T>
__device__ __forceinline__ float conv_input(const T* x, int x_stride, const float* st, int C, int K, int start,
                                            int tau, int c) {
  return tau >= start ? to_float(x[(size_t)tau * x_stride + c]) : st[(size_t)(K - 1 + tau - start) * C + c];
}

template <typename T>
__global__ void causal_conv_silu_kernel(const T* __restrict__ x, int x_stride, const T* __restrict__ taps,
                                        const float* __restrict__ state, int state_stride,
                                        const int* __restrict__ cu_q, const int* __restrict__ state_slots, int num_seqs,
                                        int num_tokens, int C, int K, float* __restrict__ y) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  // the request of token t: the last b with cu_q[b] <= t
  int lo = 0, hi = num_seqs - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_q[mid] <= t) lo = mid; else hi = mid - 1;
  }
  const int start = cu_q[lo];
  const float* st = state + (size_t)state_slots[lo] * state_stride;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < K; ++k)
      acc = fmaf(to_float(taps[(size_t)c * K + k]), conv_input(x, x_stride, st, C, K, start, t - (K - 1 - k), c), acc);
    y[(size_t)t * C + c] = acc / (1.f + expf(-acc));
  }
}

template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ x, int x_stride, float* __restrict__ state,
                                         int state_stride, const int* __restrict__ cu_q,
                                         const int* __restrict__ state_slots, int C, int K) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x;
  const int start = cu_q[b], end = cu_q[b + 1];
  if (end <= start) return;
  float* st = state + (size_t)state_slots[b] * state_stride;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    float keep[SCAN_MAX_TAPS];
    for (int i = 0; i < K - 1; ++i) keep[i] = conv_input(x, x_stride, st, C, K, start, end - (K - 1) + i, c);
    for (int i = 0; i < K - 1; ++i) st[(size_t)i * C + c] = keep[i];
  }
}

}  // namespace ts

using namespace ts;

static int scan_warps(int d) { return (d + 31) / 32; }

extern "C" int ts_mlstm_scan(const void* qkv, int stride, int q_off, int k_off, int v_off, const float* gates,
                             const float* gate_bias, float cap, float q_scale, float* state, int state_stride,
                             const int* cu_q, const int* state_slots, int num_seqs, int heads, int d, int dv, float* out, int dtype,
                             cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (d <= 0 || dv <= 0 || d > SCAN_MAX_KEY_DIM || !(cap > 0.f)) return TS_ERR_UNSUPPORTED;
  const int W = scan_warps(d);
  const size_t smem = sizeof(float) * (4 * (size_t)W * 32 + 64 + 2 * (size_t)W * 32 + 2 * W);
  dim3 grid(num_seqs, heads, (dv + 31) / 32);
  if (dtype == TS_DTYPE_F32)
    return launch(mlstm_scan_kernel<float>, grid, W * 32, smem, stream, (const float*)qkv, stride, q_off, k_off, v_off,
                  gates, gate_bias, cap, q_scale, state, state_stride, cu_q, state_slots, heads, d, dv, out);
  if (dtype == TS_DTYPE_BF16)
    return launch(mlstm_scan_kernel<bf16>, grid, W * 32, smem, stream, (const bf16*)qkv, stride, q_off, k_off, v_off,
                  gates, gate_bias, cap, q_scale, state, state_stride, cu_q, state_slots, heads, d, dv, out);
  return TS_ERR_BAD_ARGUMENT;
}

extern "C" int ts_delta_scan(const float* qkv, int stride, int q_off, int k_off, int v_off, const float* a,
                             const float* dt_bias, const float* a_log, const float* beta_pre, float q_scale,
                             float* state, int state_stride, const int* cu_q, const int* state_slots, int num_seqs,
                             int heads, int kv_heads, int d, int dv, float* out, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (d <= 0 || dv <= 0 || d > SCAN_MAX_KEY_DIM) return TS_ERR_UNSUPPORTED;
  if (kv_heads <= 0 || heads % kv_heads) return TS_ERR_BAD_ARGUMENT;
  const int W = scan_warps(d);
  const size_t smem = sizeof(float) * (6 * (size_t)W * 32 + 64 + 4 * (size_t)W * 32 + 4 * W);
  dim3 grid(num_seqs, heads, (dv + 31) / 32);
  return launch(delta_scan_kernel, grid, W * 32, smem, stream, qkv, stride, q_off, k_off, v_off, a, dt_bias, a_log,
                beta_pre, q_scale, state, state_stride, cu_q, state_slots, heads, kv_heads, d, dv, out);
}

extern "C" int ts_causal_conv_silu(const void* x, int x_stride, const void* taps, float* state, int state_stride, const int* cu_q,
                                   const int* state_slots, int num_seqs, int num_tokens, int channels, int num_taps,
                                   float* y, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0 || num_seqs <= 0) return 0;
  if (num_taps < 1 || num_taps > SCAN_MAX_TAPS) return TS_ERR_UNSUPPORTED;
  const int threads = 128;
  int by = (channels + threads - 1) / threads;
  if (by > 64) by = 64;
  dim3 grid(num_tokens, by), sgrid(num_seqs, by);
  int st;
  if (dtype == TS_DTYPE_F32) {
    st = launch(causal_conv_silu_kernel<float>, grid, threads, 0, stream, (const float*)x, x_stride, (const float*)taps,
                (const float*)state, state_stride, cu_q, state_slots, num_seqs, num_tokens, channels, num_taps, y);
    if (st != 0 || num_taps == 1) return st;
    return launch(conv_state_update_kernel<float>, sgrid, threads, 0, stream, (const float*)x, x_stride, state, state_stride, cu_q,
                  state_slots, channels, num_taps);
  }
  if (dtype == TS_DTYPE_BF16) {
    st = launch(causal_conv_silu_kernel<bf16>, grid, threads, 0, stream, (const bf16*)x, x_stride, (const bf16*)taps,
                (const float*)state, state_stride, cu_q, state_slots, num_seqs, num_tokens, channels, num_taps, y);
    if (st != 0 || num_taps == 1) return st;
    return launch(conv_state_update_kernel<bf16>, sgrid, threads, 0, stream, (const bf16*)x, x_stride, state, state_stride, cu_q,
                  state_slots, channels, num_taps);
  }
  return TS_ERR_BAD_ARGUMENT;
}
