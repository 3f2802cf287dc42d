// Layer norm (with the residual add folded in), a short causal convolution over time on every channel with its
// carried inputs kept per request, the two of them in one kernel for steps of single tokens, and the PolyNorm
// activation.  Statistics and sums are float32; each kernel is built for float and bfloat16 activations.
#include "common.cuh"

using namespace tkb;

namespace {

// four consecutive values of the activation type
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

// ------------------------------------------------------------------------------------------------
// x += update (float32, written back), then out = (x - mean) / sqrt(var + eps) * w + b, var = mean((x - mean)^2),
// rounded once to the activation type.  One block a row; the row stays in shared memory between the passes, so the
// variance is taken from the deviations themselves.  The update is [rows, H] in the activation type (delta) and/or
// float32 slices [n_slices][rows, H] of a split product, added in slice order.
template <typename T>
__device__ __forceinline__ float row_update(float* __restrict__ xr, const T* __restrict__ dr,
                                            const float* __restrict__ sl, int n_slices, long long slice_stride, int i) {
  float v = xr[i];
  if (dr != nullptr || n_slices > 0) {
    float d = dr != nullptr ? to_float(dr[i]) : 0.f;
    for (int p = 0; p < n_slices; p++) d += sl[(size_t)p * slice_stride + i];
    v += d;
    xr[i] = v;
  }
  return v;
}

template <typename T>
__global__ void add_layernorm_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                     const float* __restrict__ slices, int n_slices, long long slice_stride,
                                     const float* __restrict__ w, const float* __restrict__ b, T* __restrict__ out,
                                     float eps, int H) {
  extern __shared__ __align__(16) float row[];
  __shared__ float scratch[33];
  trigger_dependents();
  grid_dependency_wait();
  const size_t base = (size_t)blockIdx.x * H;
  float* xr = x + base;
  const T* dr = delta != nullptr ? delta + base : nullptr;
  const float* sl = slices != nullptr ? slices + base : nullptr;
  T* orow = out + base;
  if ((H & 3) == 0) {
    // four values a thread and pass
    float s = 0.f;
    for (int i = 4 * threadIdx.x; i < H; i += 4 * blockDim.x) {
      float4 v = load4(xr + i);
      if (dr != nullptr || n_slices > 0) {
        float4 d = dr != nullptr ? load4(dr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        for (int p = 0; p < n_slices; p++) {
          const float4 q = load4(sl + (size_t)p * slice_stride + i);
          d.x += q.x; d.y += q.y; d.z += q.z; d.w += q.w;
        }
        v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        store4(xr + i, v);
      }
      store4(row + i, v);
      s += (v.x + v.y) + (v.z + v.w);
    }
    const float mean = block_sum(s, scratch) / (float)H;
    float ss = 0.f;
    for (int i = 4 * threadIdx.x; i < H; i += 4 * blockDim.x) {
      const float4 v = load4(row + i);
      const float a = v.x - mean, b2 = v.y - mean, c = v.z - mean, d = v.w - mean;
      ss += (a * a + b2 * b2) + (c * c + d * d);
    }
    const float rstd = rsqrtf(block_sum(ss, scratch) / (float)H + eps);
    for (int i = 4 * threadIdx.x; i < H; i += 4 * blockDim.x) {
      const float4 v = load4(row + i), g = load4(w + i), o = load4(b + i);
      store4(orow + i, make_float4((v.x - mean) * rstd * g.x + o.x, (v.y - mean) * rstd * g.y + o.y,
                                   (v.z - mean) * rstd * g.z + o.z, (v.w - mean) * rstd * g.w + o.w));
    }
    return;
  }
  float s = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = row_update<T>(xr, dr, sl, n_slices, slice_stride, i);
    row[i] = v;
    s += v;
  }
  const float mean = block_sum(s, scratch) / (float)H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float d = row[i] - mean;
    ss += d * d;
  }
  const float rstd = rsqrtf(block_sum(ss, scratch) / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) orow[i] = from_float<T>((row[i] - mean) * rstd * w[i] + b[i]);
}

// ------------------------------------------------------------------------------------------------
// out_t = h_t + sum_j w[c, j] * h_(t - taps + 1 + j) on every channel c, over the tokens of each request in order;
// inputs before the step's first token come from the request's carried inputs carry[slot][taps - 1][H] (oldest
// first, zeros for a new request).  One block a token.  The carried inputs are brought forward by a second
// kernel that runs after every token of the step has read them.
template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ h, T* __restrict__ out, const float* __restrict__ w,
                                  const float* __restrict__ carry, const int* __restrict__ token_seq,
                                  const int* __restrict__ seq_slot, const int* __restrict__ seq_q_start, int H,
                                  int taps) {
  trigger_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int s = token_seq[t];
  if (s < 0) return;
  const int i = t - seq_q_start[s];  // index of this token among the request's tokens of this step
  const float* cr = carry + (size_t)seq_slot[s] * (taps - 1) * H;
  if ((H & 3) == 0) {
    // four channels a thread
    for (int c = 4 * threadIdx.x; c < H; c += 4 * blockDim.x) {
      const float4 own = load4(h + (size_t)t * H + c);
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int j = 0; j < taps; j++) {
        const int k = i - taps + 1 + j;
        const float4 v = k >= 0 ? load4(h + (size_t)(t - i + k) * H + c) : load4(cr + (size_t)(taps - 1 + k) * H + c);
        acc.x = fmaf(w[(size_t)(c + 0) * taps + j], v.x, acc.x);
        acc.y = fmaf(w[(size_t)(c + 1) * taps + j], v.y, acc.y);
        acc.z = fmaf(w[(size_t)(c + 2) * taps + j], v.z, acc.z);
        acc.w = fmaf(w[(size_t)(c + 3) * taps + j], v.w, acc.w);
      }
      store4(out + (size_t)t * H + c, make_float4(own.x + acc.x, own.y + acc.y, own.z + acc.z, own.w + acc.w));
    }
    return;
  }
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float own = to_float(h[(size_t)t * H + c]);
    float acc = 0.f;
    for (int j = 0; j < taps; j++) {
      const int k = i - taps + 1 + j;  // index among this step's tokens; negative: a carried input
      const float v = k >= 0 ? to_float(h[(size_t)(t - i + k) * H + c]) : cr[(size_t)(taps - 1 + k) * H + c];
      acc = fmaf(w[(size_t)c * taps + j], v, acc);
    }
    out[(size_t)t * H + c] = from_float<T>(own + acc);
  }
}

// carry[slot] <- the last taps - 1 inputs of the request after this step's n tokens.  One block a request.
template <typename T>
__global__ void short_conv_carry_kernel(const T* __restrict__ h, float* __restrict__ carry,
                                        const int* __restrict__ seq_slot, const int* __restrict__ seq_q_start,
                                        const int* __restrict__ seq_q_len, int H, int taps) {
  trigger_dependents();
  grid_dependency_wait();
  const int s = blockIdx.x;
  const int n = seq_q_len[s];
  if (n <= 0) return;
  const int start = seq_q_start[s];
  float* cr = carry + (size_t)seq_slot[s] * (taps - 1) * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    // ascending k: entry k takes what entry k + n held, which is written later
    for (int k = 0; k < taps - 1; k++) {
      const int src = n - (taps - 1) + k;  // index among this step's tokens
      cr[(size_t)k * H + c] = src >= 0 ? to_float(h[(size_t)(start + src) * H + c]) : cr[(size_t)(k + n) * H + c];
    }
  }
}

// Steps in which every request brings one token: add + layer norm + convolution + carry in one kernel, one block
// a token (its request's carried inputs are read and written by this block alone).
template <typename T>
__global__ void add_layernorm_conv1_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                           const float* __restrict__ slices, int n_slices, long long slice_stride,
                                           const float* __restrict__ w, const float* __restrict__ b,
                                           const float* __restrict__ cw, float* __restrict__ carry,
                                           const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                                           T* __restrict__ out, float eps, int H, int taps) {
  extern __shared__ __align__(16) float row[];
  __shared__ float scratch[33];
  trigger_dependents();
  grid_dependency_wait();
  const int s = token_seq[blockIdx.x];
  if (s < 0) return;
  const size_t base = (size_t)blockIdx.x * H;
  float* xr = x + base;
  const T* dr = delta != nullptr ? delta + base : nullptr;
  const float* sl = slices != nullptr ? slices + base : nullptr;
  float sum = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = row_update<T>(xr, dr, sl, n_slices, slice_stride, i);
    row[i] = v;
    sum += v;
  }
  const float mean = block_sum(sum, scratch) / (float)H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float d = row[i] - mean;
    ss += d * d;
  }
  const float rstd = rsqrtf(block_sum(ss, scratch) / (float)H + eps);
  float* cr = carry + (size_t)seq_slot[s] * (taps - 1) * H;
  if ((H & 3) == 0 && taps <= 8) {
    // four channels a thread: every load of the thread is under way before the first is used
    for (int c = 4 * threadIdx.x; c < H; c += 4 * blockDim.x) {
      const float4 xv = load4(row + c), g = load4(w + c), o = load4(b + c);
      float4 old[7];
#pragma unroll
      for (int j = 0; j < 7; j++)
        if (j < taps - 1) old[j] = load4(cr + (size_t)j * H + c);
      // the normalised values as the next kernel sees them: rounded to the activation type
      float own[4] = {(xv.x - mean) * rstd * g.x + o.x, (xv.y - mean) * rstd * g.y + o.y,
                      (xv.z - mean) * rstd * g.z + o.z, (xv.w - mean) * rstd * g.w + o.w};
      float res[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        own[u] = to_float(from_float<T>(own[u]));
        const float* cwr = cw + (size_t)(c + u) * taps;
        float acc = cwr[taps - 1] * own[u];
#pragma unroll
        for (int j = 0; j < 7; j++)
          if (j < taps - 1) acc = fmaf(cwr[j], u == 0 ? old[j].x : (u == 1 ? old[j].y : (u == 2 ? old[j].z : old[j].w)), acc);
        res[u] = own[u] + acc;
      }
#pragma unroll
      for (int j = 1; j < 7; j++)
        if (j < taps - 1) store4(cr + (size_t)(j - 1) * H + c, old[j]);
      if (taps > 1) store4(cr + (size_t)(taps - 2) * H + c, make_float4(own[0], own[1], own[2], own[3]));
      store4(out + base + c, make_float4(res[0], res[1], res[2], res[3]));
    }
    return;
  }
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    // the normalised value as the next kernel sees it: rounded to the activation type
    const float own = to_float(from_float<T>((row[c] - mean) * rstd * w[c] + b[c]));
    float acc = cw[(size_t)c * taps + taps - 1] * own;
    for (int j = 0; j < taps - 1; j++) {
      const float v = cr[(size_t)j * H + c];
      acc = fmaf(cw[(size_t)c * taps + j], v, acc);
      if (j > 0) cr[(size_t)(j - 1) * H + c] = v;
    }
    if (taps > 1) cr[(size_t)(taps - 2) * H + c] = own;
    out[base + c] = from_float<T>(own + acc);
  }
}

// ------------------------------------------------------------------------------------------------
// PolyNorm: out = a N(z) + b N(z^2) + c N(z^3) + e with N(u) = u / sqrt(mean(u^2) + eps) over a row, powers taken
// element by element.  z is float32 (the product's accumulator), one block a row.
template <typename T>
__global__ void polynorm_kernel(const float* __restrict__ z, const float* __restrict__ coef, T* __restrict__ out,
                                float eps, int F) {
  __shared__ float scratch[33];
  trigger_dependents();
  grid_dependency_wait();
  const float* zr = z + (size_t)blockIdx.x * F;
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
  for (int i = threadIdx.x; i < F; i += blockDim.x) {
    const float v = zr[i], v2 = v * v, v3 = v2 * v;
    s1 += v2;
    s2 += v2 * v2;
    s3 += v3 * v3;
  }
  const float r1 = rsqrtf(block_sum(s1, scratch) / (float)F + eps);
  const float r2 = rsqrtf(block_sum(s2, scratch) / (float)F + eps);
  const float r3 = rsqrtf(block_sum(s3, scratch) / (float)F + eps);
  const float a = coef[0] * r1, b = coef[1] * r2, c = coef[2] * r3, e = coef[3];
  T* orow = out + (size_t)blockIdx.x * F;
  for (int i = threadIdx.x; i < F; i += blockDim.x) {
    const float v = zr[i], v2 = v * v;
    orow[i] = from_float<T>(a * v + b * v2 + c * v2 * v + e);
  }
}

inline int row_threads(int H) { return H >= 2048 ? 512 : (H >= 512 ? 256 : 128); }

template <typename T>
int add_layernorm_launch(float* x, const void* delta, const float* slices, int n_slices, long long slice_stride,
                         const float* w, const float* b, void* out, float eps, int rows, int H, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (H <= 0 || (size_t)H * 4 > 200 * 1024) return -2;
  const size_t smem = (size_t)H * 4;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(add_layernorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return launch_pdl(add_layernorm_kernel<T>, dim3(rows), dim3(row_threads(H)), smem, st, x, (const T*)delta, slices,
                    n_slices, slice_stride, w, b, (T*)out, eps, H);
}

template <typename T>
int add_layernorm_conv1_launch(float* x, const void* delta, const float* slices, int n_slices, long long slice_stride,
                               const float* w, const float* b, const float* cw, float* carry, const int* token_seq,
                               const int* seq_slot, void* out, float eps, int rows, int H, int taps, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (H <= 0 || taps < 1 || (size_t)H * 4 > 200 * 1024) return -2;
  const size_t smem = (size_t)H * 4;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(add_layernorm_conv1_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return launch_pdl(add_layernorm_conv1_kernel<T>, dim3(rows), dim3(row_threads(H)), smem, st, x, (const T*)delta, slices,
                    n_slices, slice_stride, w, b, cw, carry, token_seq, seq_slot, (T*)out, eps, H, taps);
}

template <typename T>
int short_conv_launch(const void* h, void* out, const float* w, float* carry, const int* token_seq, const int* seq_slot,
                      const int* seq_q_start, const int* seq_q_len, int n_tokens, int n_seqs, int H, int taps,
                      cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || taps < 1) return -2;
  int rc = launch_pdl(short_conv_kernel<T>, dim3(n_tokens), dim3(row_threads(H)), 0, st, (const T*)h, (T*)out, w,
                      (const float*)carry, token_seq, seq_slot, seq_q_start, H, taps);
  if (rc != 0 || taps == 1 || n_seqs <= 0) return rc;
  return launch_pdl(short_conv_carry_kernel<T>, dim3(n_seqs), dim3(row_threads(H)), 0, st, (const T*)h, carry, seq_slot,
                    seq_q_start, seq_q_len, H, taps);
}

template <typename T>
int polynorm_launch(const float* z, const float* coef, void* out, float eps, int rows, int F, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (F <= 0) return -2;
  return launch_pdl(polynorm_kernel<T>, dim3(rows), dim3(row_threads(F)), 0, st, z, coef, (T*)out, eps, F);
}

}  // namespace

#define TKB_NORM_CONV_EXPORTS(SUF, T)                                                                                  \
  TKB_EXPORT int tkb_add_layernorm_##SUF(float* x, const void* delta, const float* slices, int n_slices,               \
                                         long long slice_stride, const float* w, const float* b, void* out, float eps, \
                                         int rows, int H, void* st) {                                                  \
    return add_layernorm_launch<T>(x, delta, slices, n_slices, slice_stride, w, b, out, eps, rows, H, (cudaStream_t)st); \
  }                                                                                                                    \
  TKB_EXPORT int tkb_add_layernorm_conv1_##SUF(float* x, const void* delta, const float* slices, int n_slices,         \
                                               long long slice_stride, const float* w, const float* b, const float* cw, \
                                               float* carry, const int* token_seq, const int* seq_slot, void* out,     \
                                               float eps, int rows, int H, int taps, void* st) {                       \
    return add_layernorm_conv1_launch<T>(x, delta, slices, n_slices, slice_stride, w, b, cw, carry, token_seq, seq_slot, \
                                         out, eps, rows, H, taps, (cudaStream_t)st);                                   \
  }                                                                                                                    \
  TKB_EXPORT int tkb_short_conv_##SUF(const void* h, void* out, const float* w, float* carry, const int* token_seq,    \
                                      const int* seq_slot, const int* seq_q_start, const int* seq_q_len, int n_tokens, \
                                      int n_seqs, int H, int taps, void* st) {                                         \
    return short_conv_launch<T>(h, out, w, carry, token_seq, seq_slot, seq_q_start, seq_q_len, n_tokens, n_seqs, H,    \
                                taps, (cudaStream_t)st);                                                               \
  }                                                                                                                    \
  TKB_EXPORT int tkb_polynorm_##SUF(const float* z, const float* coef, void* out, float eps, int rows, int F,          \
                                    void* st) {                                                                        \
    return polynorm_launch<T>(z, coef, out, eps, rows, F, (cudaStream_t)st);                                           \
  }

TKB_NORM_CONV_EXPORTS(f32, float)
TKB_NORM_CONV_EXPORTS(bf16, __nv_bfloat16)
