// Attention over a cache of latent vectors: every token keeps ONE row of R + P elements, a normed
// latent vector c (R elements) from which all heads' keys and values derive, and a rotated key
// part (P elements) shared by the heads. With the keys' up-projection folded into the queries
// (q'_h = W_uk,h^T q_h) and the values' up-projection applied after the weighted sum, every head
// scores against the same row, score = q'_h . c + q_rot,h . k_rot, and sums the same c: the layer is
// attention with one shared key/value head whose values are the first R elements of its keys.
//
//  * ts_latent_prepare: per token, RMSNorm of the latent part (plain weight), rotation of the shared
//    key part, both written to the cache row of the token's slot; and the full query rows
//    [T, H, R + P] assembled from the folded queries [H, T, R] and the rotated query parts.
//  * ts_latent_attention: causal (optionally windowed) softmax attention of those query rows over
//    the cached rows, on CUDA cores in 32-bit, for float and bf16 storage. A CTA takes a few
//    tokens of one request and a few heads; every key tile it stages is shared by all its rows.
//    A warp owns a row at a time: each lane scores one key of the tile, then each lane owns
//    output columns. Rows of other requests or beyond a request's positions are never loaded.
#define TS_PDL_CLASS PDL_ATTENTION
#include "common.cuh"

namespace ts {

// ------------------------------------------------------------------------ prepare
struct LatentPrepArgs {
  const void* q_in;      // [T, q_stride]: per head `nope` unrotated then P rotated elements
  long long q_stride;
  const void* q_folded;  // [H, T, R]
  const void* ckr;       // [T, ckr_stride]: R latent elements, then P elements of the shared key part
  long long ckr_stride;
  const void* norm_weight;  // [R]
  float eps;
  const float* cos_t;    // [T, rotary_dim / 2]
  const float* sin_t;
  int rotary_dim, interleaved;
  const int* slots;      // [T] cache row of each token (null: nothing is written)
  void* cache;           // [rows, R + P]
  void* q_out;           // [T, H, R + P]
  int num_tokens, heads, nope, rank, rot;
};

// Rotation of element i of a vector of `rot` elements whose first `rotary_dim` turn.
template <typename T>
__device__ __forceinline__ float rotated(const T* v, int i, const float* c, const float* s, int rotary_dim, int interleaved) {
  if (i >= rotary_dim) return to_float(v[i]);
  const int half = rotary_dim >> 1;
  if (interleaved) {
    const int p = i >> 1;
    const float a = to_float(v[2 * p]), b = to_float(v[2 * p + 1]);
    return (i & 1) ? b * c[p] + a * s[p] : a * c[p] - b * s[p];
  }
  if (i < half) return to_float(v[i]) * c[i] - to_float(v[i + half]) * s[i];
  return to_float(v[i]) * c[i - half] + to_float(v[i - half]) * s[i - half];
}

template <typename T>
__global__ void latent_prepare_kernel(LatentPrepArgs a) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int D = a.rank + a.rot;
  const float* c = a.cos_t ? a.cos_t + (size_t)t * (a.rotary_dim >> 1) : nullptr;
  const float* s = a.sin_t ? a.sin_t + (size_t)t * (a.rotary_dim >> 1) : nullptr;
  const int rdim = c ? a.rotary_dim : 0;
  if (a.slots) {
    const T* row = (const T*)a.ckr + (size_t)t * a.ckr_stride;
    T* dst = (T*)a.cache + (size_t)a.slots[t] * D;
    float ss = 0.f;
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) {
      const float v = to_float(row[i]);
      ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float rstd = rsqrtf(ss / (float)a.rank + a.eps);
    const T* w = (const T*)a.norm_weight;
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) dst[i] = from_float<T>(to_float(row[i]) * rstd * to_float(w[i]));
    for (int i = threadIdx.x; i < a.rot; i += blockDim.x)
      dst[a.rank + i] = from_float<T>(rotated(row + a.rank, i, c, s, rdim, a.interleaved));
  }
  const T* qf = (const T*)a.q_folded;
  T* qo = (T*)a.q_out + (size_t)t * a.heads * D;
  for (int idx = threadIdx.x; idx < a.heads * a.rank; idx += blockDim.x) {
    const int h = idx / a.rank, i = idx - h * a.rank;
    qo[(size_t)h * D + i] = qf[((size_t)h * a.num_tokens + t) * a.rank + i];
  }
  const T* qi = (const T*)a.q_in + (size_t)t * a.q_stride;
  for (int idx = threadIdx.x; idx < a.heads * a.rot; idx += blockDim.x) {
    const int h = idx / a.rot, i = idx - h * a.rot;
    qo[(size_t)h * D + a.rank + i] =
        from_float<T>(rotated(qi + (size_t)h * (a.nope + a.rot) + a.nope, i, c, s, rdim, a.interleaved));
  }
}

// ---------------------------------------------------------------------- attention
struct LatentAttnArgs {
  const void* q;           // [T, H, D]
  void* out;               // [T, H, R]
  const void* cache;       // [pages * page_size, D]
  const int* block_tables; // [B, table_width]
  const int* cu_q;         // [B + 1]
  const int* ctx_lens;     // [B]
  int table_width, num_seqs, heads, rank, rot, page_size;
  float scale_log2;
  int window;              // 0: every earlier position
  int tokens_per_cta, heads_per_cta;
};

constexpr int LA_WARPS = 8, LA_THREADS = LA_WARPS * 32, LA_TK = 32;
constexpr int LA_RPW = 4;          // rows a warp works on together

// RJ: output columns per lane (rank <= 32 * RJ).
template <typename T, int RJ>
__global__ void __launch_bounds__(LA_THREADS) latent_attention_kernel(LatentAttnArgs a) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int R = a.rank, D = a.rank + a.rot, DS = D + 1;
  const int rows_cta = a.tokens_per_cta * a.heads_per_cta;
  float* Qs = smem;                         // [rows_cta][D]  pre-scaled
  float* Ks = Qs + (size_t)rows_cta * D;    // [LA_TK][DS]
  const int seq = blockIdx.y;
  const int row0 = a.cu_q[seq];
  const int n = a.cu_q[seq + 1] - row0;
  const int t0 = blockIdx.x * a.tokens_per_cta;
  if (t0 >= n) return;
  const int nt = min(a.tokens_per_cta, n - t0);
  const int h0 = blockIdx.z * a.heads_per_cta;
  const int nh = min(a.heads_per_cta, a.heads - h0);
  const int ctx = a.ctx_lens[seq];
  const int first_pos = ctx - n;
  const int* table = a.block_tables + (size_t)seq * a.table_width;
  const T* q = (const T*)a.q;
  const T* cache = (const T*)a.cache;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nrows = nt * nh;                // row r -> token r / nh, head r % nh

  for (int idx = tid; idx < nrows * D; idx += LA_THREADS) {
    const int r = idx / D, d = idx - r * D;
    const int tt = r / nh, hh = r - tt * nh;
    Qs[(size_t)r * D + d] = to_float(q[((size_t)(row0 + t0 + tt) * a.heads + h0 + hh) * D + d]) * a.scale_log2;
  }
  const int qpos_first = first_pos + t0, qpos_last = first_pos + t0 + nt - 1;
  const int k_lo = a.window > 0 ? max(0, qpos_first - a.window + 1) : 0;
  const int k_begin = (k_lo / LA_TK) * LA_TK;

  // a warp's rows: warp, warp + LA_WARPS, ...  (at most LA_RPW of them a pass)
  for (int pass0 = 0; pass0 < nrows; pass0 += LA_WARPS * LA_RPW) {
    float m[LA_RPW], l[LA_RPW], acc[LA_RPW][RJ];
    int qpos[LA_RPW];
    bool live[LA_RPW];
#pragma unroll
    for (int i = 0; i < LA_RPW; ++i) {
      const int r = pass0 + warp + i * LA_WARPS;
      live[i] = r < nrows;
      qpos[i] = live[i] ? first_pos + t0 + r / nh : -1;
      m[i] = -INFINITY;
      l[i] = 0.f;
#pragma unroll
      for (int j = 0; j < RJ; ++j) acc[i][j] = 0.f;
    }
    for (int k0 = k_begin; k0 <= qpos_last; k0 += LA_TK) {
      __syncthreads();       // the tile before is consumed (and Qs is written)
      for (int idx = tid; idx < LA_TK * D; idx += LA_THREADS) {
        const int kk = idx / D, d = idx - kk * D;
        const int kpos = k0 + kk;
        float v = 0.f;
        if (kpos >= k_lo && kpos <= qpos_last) {
          const int pg = kpos / a.page_size;
          const size_t crow = (size_t)table[pg] * a.page_size + (kpos - pg * a.page_size);
          v = to_float(cache[crow * D + d]);
        }
        Ks[kk * DS + d] = v;
      }
      __syncthreads();
      // ---- scores: lane = key of the tile
      float s[LA_RPW];
#pragma unroll
      for (int i = 0; i < LA_RPW; ++i) s[i] = 0.f;
      const float* krow = Ks + lane * DS;
      for (int d = 0; d < D; ++d) {
        const float kv = krow[d];
#pragma unroll
        for (int i = 0; i < LA_RPW; ++i)
          if (live[i]) s[i] = fmaf(Qs[(size_t)(pass0 + warp + i * LA_WARPS) * D + d], kv, s[i]);
      }
      const int kpos = k0 + lane;
#pragma unroll
      for (int i = 0; i < LA_RPW; ++i) {
        if (!live[i]) continue;                       // warp-uniform
        bool ok = kpos <= qpos[i];
        if (a.window > 0) ok = ok && (kpos > qpos[i] - a.window);
        const float sv = ok ? s[i] : -INFINITY;
        const float mx = warp_max(sv);
        if (mx == -INFINITY) continue;                // no key of this tile is visible to the row
        const float m_new = fmaxf(m[i], mx);
        const float corr = exp2f(m[i] - m_new);       // m = -inf gives 0
        const float p = ok ? exp2f(sv - m_new) : 0.f;
        l[i] = l[i] * corr + warp_sum(p);
        m[i] = m_new;
#pragma unroll
        for (int j = 0; j < RJ; ++j) acc[i][j] *= corr;
        // ---- values: lane = output column (+ 32 j); the values are the first R elements of the keys
        for (int kk = 0; kk < LA_TK; ++kk) {
          const float pk = __shfl_sync(0xffffffffu, p, kk);
          if (pk == 0.f) continue;                    // warp-uniform
          const float* vrow = Ks + kk * DS;
#pragma unroll
          for (int j = 0; j < RJ; ++j) {
            const int col = lane + 32 * j;
            if (col < R) acc[i][j] = fmaf(pk, vrow[col], acc[i][j]);
          }
        }
      }
    }
    T* out = (T*)a.out;
#pragma unroll
    for (int i = 0; i < LA_RPW; ++i) {
      if (!live[i]) continue;
      const int r = pass0 + warp + i * LA_WARPS;
      const int tt = r / nh, hh = r - tt * nh;
      const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
#pragma unroll
      for (int j = 0; j < RJ; ++j) {
        const int col = lane + 32 * j;
        if (col < R) out[((size_t)(row0 + t0 + tt) * a.heads + h0 + hh) * R + col] = from_float<T>(acc[i][j] * inv);
      }
    }
  }
}

template <typename T, int RJ>
static int launch_latent(const LatentAttnArgs& a, int max_query_len, cudaStream_t stream) {
  const int D = a.rank + a.rot;
  const size_t smem = sizeof(float) * ((size_t)a.tokens_per_cta * a.heads_per_cta * D + (size_t)LA_TK * (D + 1));
  auto kern = latent_attention_kernel<T, RJ>;
  if (smem > 200 * 1024) return TS_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((max_query_len + a.tokens_per_cta - 1) / a.tokens_per_cta, a.num_seqs,
            (a.heads + a.heads_per_cta - 1) / a.heads_per_cta);
  return launch(kern, grid, LA_THREADS, smem, stream, a);
}

}  // namespace ts

using namespace ts;

extern "C" int ts_latent_prepare(const void* q_in, long long q_stride, const void* q_folded, const void* ckr,
                                 long long ckr_stride, const void* norm_weight, float eps, const float* cos_t,
                                 const float* sin_t, int rotary_dim, int interleaved, const int* slots, void* cache,
                                 void* q_out, int num_tokens, int heads, int nope, int rank, int rot, int dtype,
                                 cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (heads <= 0 || nope < 0 || rank <= 0 || rot < 0 || rotary_dim < 0 || rotary_dim > rot || (rotary_dim & 1))
    return TS_ERR_BAD_ARGUMENT;
  if (rotary_dim && (!cos_t || !sin_t)) return TS_ERR_BAD_ARGUMENT;
  if (slots && (!cache || !ckr || !norm_weight)) return TS_ERR_BAD_ARGUMENT;
  LatentPrepArgs a;
  a.q_in = q_in; a.q_stride = q_stride; a.q_folded = q_folded; a.ckr = ckr; a.ckr_stride = ckr_stride;
  a.norm_weight = norm_weight; a.eps = eps; a.cos_t = rotary_dim ? cos_t : nullptr; a.sin_t = rotary_dim ? sin_t : nullptr;
  a.rotary_dim = rotary_dim; a.interleaved = interleaved; a.slots = slots; a.cache = cache; a.q_out = q_out;
  a.num_tokens = num_tokens; a.heads = heads; a.nope = nope; a.rank = rank; a.rot = rot;
  if (dtype == TS_DTYPE_F32) return launch(latent_prepare_kernel<float>, num_tokens, 256, 0, stream, a);
  if (dtype == TS_DTYPE_BF16) return launch(latent_prepare_kernel<bf16>, num_tokens, 256, 0, stream, a);
  return TS_ERR_BAD_ARGUMENT;
}

// Largest latent size the kernel takes (32 output columns per lane and step, 16 steps).
extern "C" int ts_latent_attention_max_rank() { return 512; }

extern "C" int ts_latent_attention(const void* q, void* out, const void* cache, const int* block_tables, int table_width,
                                   const int* cu_q, const int* ctx_lens, int num_seqs, int max_query_len, int heads,
                                   int rank, int rot, int page_size, float scale, int window, int dtype,
                                   cudaStream_t stream) {
  if (num_seqs <= 0 || max_query_len <= 0) return 0;
  if (heads <= 0 || rank <= 0 || rank > 512 || rot < 0 || page_size <= 0 || window < 0) return TS_ERR_BAD_ARGUMENT;
  LatentAttnArgs a;
  a.q = q; a.out = out; a.cache = cache; a.block_tables = block_tables; a.table_width = table_width;
  a.cu_q = cu_q; a.ctx_lens = ctx_lens; a.num_seqs = num_seqs; a.heads = heads; a.rank = rank; a.rot = rot;
  a.page_size = page_size; a.scale_log2 = scale * 1.4426950408889634f; a.window = window;
  // 32 rows a CTA where the step has them: 8 heads of 4 tokens (a single token: 8 heads)
  a.heads_per_cta = heads < 8 ? heads : 8;
  a.tokens_per_cta = max_query_len == 1 ? 1 : (32 / a.heads_per_cta);
  const int rj = (rank + 31) / 32;
#define TS_LA_CASE(T_)                                                        \
  do {                                                                        \
    if (rj <= 4) return launch_latent<T_, 4>(a, max_query_len, stream);       \
    if (rj <= 8) return launch_latent<T_, 8>(a, max_query_len, stream);       \
    return launch_latent<T_, 16>(a, max_query_len, stream);                   \
  } while (0)
  if (dtype == TS_DTYPE_F32) TS_LA_CASE(float);
  if (dtype == TS_DTYPE_BF16) TS_LA_CASE(bf16);
#undef TS_LA_CASE
  return TS_ERR_BAD_ARGUMENT;
}
