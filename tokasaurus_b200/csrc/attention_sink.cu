// Grouped-query attention over the paged cache with a soft cap on the scores and a per-head sink in the softmax, for
// heads whose keys and values have different sizes:
//
//     s_ij = cap * tanh(scale * q_i . k_j / cap)   (cap <= 0: s_ij = scale * q_i . k_j),
//     o_i  = sum_j exp(s_ij) v_j / (exp(sink_h) + sum_j exp(s_ij)),      j over max(0, i - window + 1) .. i
//
// The sink takes part in the denominator only: it has no key and no value.  sink == null: an ordinary softmax.
// A cached row holds one token's key and value of one key/value head side by side: [k (QK values) | v (VD values)],
// rows [page][kv head][slot in page][QK + VD].
//
// Two kernels.  sink_attn_prep: one block a token; adds the projections' biases, divides every q head and every k
// head by its root mean square (float32, no weight) if asked, writes q in the activation type and the token's
// [k | v] rows into its page.  attn_sink_simt: one warp a (token, query head) on the FP32 pipes, any mix of prompt
// portions and single tokens; lane j scores key base + j, probabilities are passed round by shuffle while lane d
// sums output elements d, d + 32, ...  Scores, weights and sums are float32.
//
// Compile with -DTKB_QK=<query/key size> -DTKB_VD=<value size>.
#include "common.cuh"
#include <float.h>

#if !defined(TKB_QK) || !defined(TKB_VD)
#error "compile with -DTKB_QK=<query/key size> -DTKB_VD=<value size>"
#endif
static_assert(TKB_QK >= 1 && TKB_QK <= 512 && TKB_VD >= 1 && TKB_VD <= 512, "head sizes up to 512");

using namespace tkb;

namespace {

constexpr int QK = TKB_QK;
constexpr int VD = TKB_VD;
constexpr int ROW = QK + VD;
constexpr int WARPS = 4;
constexpr int DPL = (VD + 31) / 32;

template <typename T>
__device__ __forceinline__ float dot_key(const T* __restrict__ k, const float* __restrict__ q) {
  float acc = 0.f;
  if constexpr (sizeof(T) == 4 && QK % 4 == 0 && ROW % 4 == 0) {
    const float4* k4 = reinterpret_cast<const float4*>(k);
#pragma unroll 8
    for (int i = 0; i < QK / 4; i++) {
      const float4 v = k4[i];
      acc = fmaf(v.x, q[4 * i + 0], acc);
      acc = fmaf(v.y, q[4 * i + 1], acc);
      acc = fmaf(v.z, q[4 * i + 2], acc);
      acc = fmaf(v.w, q[4 * i + 3], acc);
    }
  } else if constexpr (sizeof(T) == 2 && QK % 8 == 0 && ROW % 8 == 0) {
    const uint4* k8 = reinterpret_cast<const uint4*>(k);
#pragma unroll 4
    for (int i = 0; i < QK / 8; i++) {
      const uint4 v = k8[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const float2 f = __bfloat1622float2(h[u]);
        acc = fmaf(f.x, q[8 * i + 2 * u + 0], acc);
        acc = fmaf(f.y, q[8 * i + 2 * u + 1], acc);
      }
    }
  } else {
#pragma unroll 8
    for (int i = 0; i < QK; i++) acc = fmaf(to_float(k[i]), q[i], acc);
  }
  return acc;
}

// qkv: float32 [T, stride] = [q (nh * QK) | k (nkv * QK) | v (nkv * VD)]
template <typename T>
__global__ void __launch_bounds__(256)
sink_attn_prep_kernel(const float* __restrict__ qkv, int stride, const float* __restrict__ bias, int unit_norm,
                      float eps, T* __restrict__ q_out, T* __restrict__ cache, const int* __restrict__ positions,
                      const int* __restrict__ token_seq, const int* __restrict__ page_indptr,
                      const int* __restrict__ page_ids, int nh, int nkv, int page_size, int num_pages, int write_cache,
                      int* __restrict__ status) {
  trigger_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int s = token_seq[t];
  if (s < 0) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const float* row = qkv + (size_t)t * stride;
  const int p = positions[t];
  int page = -1;
  if (write_cache) page = checked_page(page_ids[page_indptr[s] + p / page_size], num_pages, status);
  const int slot = p % page_size;
  // q heads and k heads: one warp a head
  for (int hh = warp; hh < nh + nkv; hh += nwarps) {
    const int off = hh * QK;  // k heads follow the q heads in the row
    float ss = 0.f;
    for (int d = lane; d < QK; d += 32) {
      const float v = row[off + d] + (bias ? bias[off + d] : 0.f);
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float r = unit_norm ? rsqrtf(ss / (float)QK + eps) : 1.f;
    T* dst = nullptr;
    if (hh < nh) dst = q_out + (size_t)t * nh * QK + off;
    else if (page >= 0) dst = cache + (((size_t)page * nkv + (hh - nh)) * page_size + slot) * ROW;
    if (dst != nullptr)
      for (int d = lane; d < QK; d += 32) dst[d] = from_float<T>((row[off + d] + (bias ? bias[off + d] : 0.f)) * r);
  }
  if (page >= 0) {
    const int voff = (nh + nkv) * QK;
    for (int idx = threadIdx.x; idx < nkv * VD; idx += blockDim.x) {
      const int g = idx / VD, d = idx - g * VD;
      cache[(((size_t)page * nkv + g) * page_size + slot) * ROW + QK + d] =
          from_float<T>(row[voff + idx] + (bias ? bias[voff + idx] : 0.f));
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attn_sink_simt_kernel(const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ cache,
                      const int* __restrict__ token_seq, const int* __restrict__ positions,
                      const int* __restrict__ page_indptr, const int* __restrict__ page_ids,
                      const int* __restrict__ rows, const float* __restrict__ sinks, int nh, int nkv, int page_size,
                      float scale, float softcap, int window, int num_pages, int* __restrict__ status) {
  __shared__ float qs[WARPS][QK];
  trigger_dependents();
  grid_dependency_wait();
  const int t = rows ? rows[blockIdx.x] : blockIdx.x;
  const int kvh = blockIdx.y;
  const int s = token_seq[t];
  if (s < 0) return;
  const int p = positions[t];
  const int group = nh / nkv;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int* table = page_ids + page_indptr[s];
  int lo = 0;
  if (window > 0 && p - window + 1 > 0) lo = p - window + 1;
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;

  for (int gq = warp; gq < group; gq += WARPS) {
    const int h = kvh * group + gq;
    const T* qrow = q + ((size_t)t * nh + h) * QK;
    for (int d = lane; d < QK; d += 32) qs[warp][d] = to_float(qrow[d]);
    __syncwarp();

    // the sink opens the running softmax: maximum sink, sum exp(sink - sink) = 1, nothing accumulated
    float m = sinks ? sinks[h] : -FLT_MAX;
    float l = sinks ? 1.f : 0.f;
    float acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; i++) acc[i] = 0.f;

    for (int base = lo; base <= p; base += 32) {
      const int j = base + lane;
      const bool live = j <= p;
      long long rowoff = 0;
      float sc = -FLT_MAX;
      bool counted = false;
      if (live) {
        const int page = checked_page(table[j / page_size], num_pages, status);
        if (page >= 0) {  // else: an id beyond the pool (the status flag is set); the key counts for nothing
          rowoff = (((long long)page * nkv + kvh) * page_size + (j % page_size)) * ROW;
          sc = dot_key<T>(cache + rowoff, qs[warp]) * scale;
          if (softcap > 0.f) sc = softcap * tanhf(sc * inv_cap);
          counted = true;
        }
      }
      const float bm = warp_max(sc);
      const float m_new = fmaxf(m, bm);
      const float alpha = expf(m - m_new);
      const float pj = counted ? expf(sc - m_new) : 0.f;
      l = l * alpha + warp_sum(pj);
      m = m_new;
#pragma unroll
      for (int i = 0; i < DPL; i++) acc[i] *= alpha;
      const int nlive = (p - base + 1) < 32 ? (p - base + 1) : 32;
      for (int jj = 0; jj < nlive; jj++) {
        const float pv = __shfl_sync(0xffffffffu, pj, jj);
        const long long ro = __shfl_sync(0xffffffffu, rowoff, jj);
        const T* vrow = cache + ro + QK;
#pragma unroll
        for (int i = 0; i < DPL; i++) {
          const int d = lane + 32 * i;
          if (d < VD) acc[i] = fmaf(pv, to_float(vrow[d]), acc[i]);
        }
      }
    }
    const float inv_l = l > 0.f ? 1.f / l : 0.f;
    T* orow = out + ((size_t)blockIdx.x * nh + h) * VD;
#pragma unroll
    for (int i = 0; i < DPL; i++) {
      const int d = lane + 32 * i;
      if (d < VD) orow[d] = from_float<T>(acc[i] * inv_l);
    }
    __syncwarp();
  }
}

template <typename T>
int prep_launch(const float* qkv, int stride, const float* bias, int unit_norm, float eps, void* q_out, void* cache,
                const int* positions, const int* token_seq, const int* page_indptr, const int* page_ids, int n_tokens,
                int nh, int nkv, int page_size, int num_pages, int write_cache, int* status, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  if (nkv <= 0 || nh <= 0 || nh % nkv != 0 || page_size <= 0) return -2;
  return launch_pdl(sink_attn_prep_kernel<T>, dim3(n_tokens), dim3(256), 0, st, qkv, stride, bias, unit_norm, eps,
                    (T*)q_out, (T*)cache, positions, token_seq, page_indptr, page_ids, nh, nkv, page_size, num_pages,
                    write_cache, status);
}

template <typename T>
int attn_launch(const void* q, void* out, const void* cache, const int* token_seq, const int* positions,
                const int* page_indptr, const int* page_ids, const int* rows, int n_rows, const float* sinks, int nh,
                int nkv, int page_size, float scale, float softcap, int window, int num_pages, int* status,
                cudaStream_t st) {
  if (n_rows <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || page_size <= 0) return -2;
  if (nkv > 65535) return -3;
  return launch_pdl(attn_sink_simt_kernel<T>, dim3(n_rows, nkv), dim3(WARPS * 32), 0, st, (const T*)q, (T*)out,
                    (const T*)cache, token_seq, positions, page_indptr, page_ids, rows, sinks, nh, nkv, page_size,
                    scale, softcap, window, num_pages, status);
}

}  // namespace

#define TKB_SINK_EXPORTS(SUF, T)                                                                                      \
  TKB_EXPORT int tkb_sink_attn_prep_##SUF(const float* qkv, int stride, const float* bias, int unit_norm, float eps,  \
                                          void* q_out, void* cache, const int* positions, const int* token_seq,       \
                                          const int* page_indptr, const int* page_ids, int n_tokens, int nh, int nkv, \
                                          int page_size, int num_pages, int write_cache, int* status, void* st) {     \
    return prep_launch<T>(qkv, stride, bias, unit_norm, eps, q_out, cache, positions, token_seq, page_indptr,         \
                          page_ids, n_tokens, nh, nkv, page_size, num_pages, write_cache, status, (cudaStream_t)st);  \
  }                                                                                                                   \
  TKB_EXPORT int tkb_attn_sink_simt_##SUF(const void* q, void* out, const void* cache, const int* token_seq,          \
                                          const int* positions, const int* page_indptr, const int* page_ids,          \
                                          const int* rows, int n_rows, const float* sinks, int nh, int nkv,           \
                                          int page_size, float scale, float softcap, int window, int num_pages,       \
                                          int* status, void* st) {                                                    \
    return attn_launch<T>(q, out, cache, token_seq, positions, page_indptr, page_ids, rows, n_rows, sinks, nh, nkv,   \
                          page_size, scale, softcap, window, num_pages, status, (cudaStream_t)st);                    \
  }

TKB_SINK_EXPORTS(f32, float)
TKB_SINK_EXPORTS(bf16, __nv_bfloat16)
