// Kernels of blocks that normalise a sublayer's OUTPUT and add it to the residual stream, and of the parts that
// such models bring along:
//
//   scaled_norm_add   x += mult * scale[c] * w[c] * (y + bias)[c] / sqrt(mean((y + bias)^2) + eps)   (x float32, in
//                     place), and the new x in the activation type for the sublayer that reads it next; y whole
//                     rows or the float32 slices of a K-split product
//   cast_rows         float32 rows in the activation type
//   add_sinusoid      x[t][2i] += sin(p_t * f_i),  x[t][2i+1] += cos(p_t * f_i)   (f_i a float64 table)
//   clamped_glu       g = min(gate, L), u = clamp(up, -L, L), out = g * sigmoid(alpha * g) * (u + 1)
//   gated_group_norm  a row of float32 values, gated and RMS-normed in equal parts:
//                       mode 0: out = N(y) * w * sigmoid(gate)        (the norm first)
//                       mode 1: out = N(y * silu(gate)) * w           (the gate first)
//
// Statistics, sums and the residual stream are float32 whatever the activation type.  One block a row.
#include "common.cuh"

using namespace tkb;

namespace {

inline int row_threads(int n) {
  int t = 32;
  while (t < n / 4 && t < 512) t <<= 1;
  return t;
}

template <typename T>
__global__ void __launch_bounds__(512)
scaled_norm_add_kernel(float* __restrict__ x, const float* __restrict__ y, int n_slices, long long slice_stride,
                       const float* __restrict__ bias, const float* __restrict__ w, const float* __restrict__ scale,
                       float mult, float eps, T* __restrict__ h_out, int H) {
  __shared__ float red[33];
  trigger_dependents();
  grid_dependency_wait();
  const size_t row = (size_t)blockIdx.x * H;
  // y may arrive as the float32 slices of a K-split product: they are added in slice order, both times alike
  auto value = [&](int c) {
    float v = y[row + c];
    for (int s = 1; s < n_slices; s++) v += y[(size_t)s * slice_stride + row + c];
    return v + (bias ? bias[c] : 0.f);
  };
  float ss = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float v = value(c);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / (float)H + eps);
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float v = value(c);
    float u = v * r * w[c];
    if (scale) u *= scale[c];
    const float nx = fmaf(mult, u, x[row + c]);
    x[row + c] = nx;
    if (h_out) h_out[row + c] = from_float<T>(nx);
  }
}

template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ x, T* __restrict__ out, size_t n) {
  trigger_dependents();
  grid_dependency_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_float<T>(x[i]);
}

// Frequencies, angle, sine and cosine in float64 (a float32 product of a position in the thousands and a frequency is off
// by 1e-4 of a radian); what is added to the row is their float32 rounding.
__global__ void add_sinusoid_kernel(float* __restrict__ x, const int* __restrict__ positions,
                                    const double* __restrict__ freq, int H) {
  trigger_dependents();
  grid_dependency_wait();
  const double p = (double)positions[blockIdx.x];
  float* row = x + (size_t)blockIdx.x * H;
  for (int i = threadIdx.x; 2 * i < H; i += blockDim.x) {
    double s, c;
    sincos(p * freq[i], &s, &c);
    row[2 * i] += (float)s;
    if (2 * i + 1 < H) row[2 * i + 1] += (float)c;
  }
}

// interleave 0: a row is [gate | up]; 8: columns in groups of 16, 8 gate columns then the 8 up columns of the same features
template <typename TI, typename TO>
__global__ void clamped_glu_kernel(const TI* __restrict__ gate_up, TO* __restrict__ out, int inner, float limit,
                                   float alpha, int interleave) {
  trigger_dependents();
  grid_dependency_wait();
  const TI* row = gate_up + (size_t)blockIdx.x * 2 * inner;
  TO* orow = out + (size_t)blockIdx.x * inner;
  for (int i = threadIdx.x; i < inner; i += blockDim.x) {
    const int gi = interleave ? ((i >> 3) << 4) + (i & 7) : i;
    const int ui = interleave ? gi + 8 : inner + i;
    const float g = fminf(to_float(row[gi]), limit);
    const float u = fminf(fmaxf(to_float(row[ui]), -limit), limit);
    orow[i] = from_float<TO>(g / (1.f + expf(-alpha * g)) * (u + 1.f));
  }
}

// One block a (row, part).  gate_first: the values are multiplied by silu(gate) before the statistics.
template <typename T>
__global__ void __launch_bounds__(512)
gated_group_norm_kernel(const float* __restrict__ y, int y_stride, const float* __restrict__ gate, int gate_stride,
                        const float* __restrict__ w, T* __restrict__ out, int out_stride, int part, float eps,
                        int gate_first) {
  __shared__ float red[33];
  trigger_dependents();
  grid_dependency_wait();
  const int c0 = blockIdx.y * part;
  const float* yr = y + (size_t)blockIdx.x * y_stride + c0;
  const float* gr = gate + (size_t)blockIdx.x * gate_stride + c0;
  float ss = 0.f;
  for (int c = threadIdx.x; c < part; c += blockDim.x) {
    float v = yr[c];
    if (gate_first) {
      const float g = gr[c];
      v *= g / (1.f + expf(-g));
    }
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / (float)part + eps);
  T* orow = out + (size_t)blockIdx.x * out_stride + c0;
  for (int c = threadIdx.x; c < part; c += blockDim.x) {
    float v = yr[c];
    const float g = gr[c];
    if (gate_first) v = v * (g / (1.f + expf(-g))) * r * w[c0 + c];
    else v = v * r * w[c0 + c] / (1.f + expf(-g));
    orow[c] = from_float<T>(v);
  }
}

}  // namespace

#define TKB_POST_NORM_EXPORTS(SUF, T)                                                                                 \
  TKB_EXPORT int tkb_scaled_norm_add_##SUF(float* x, const float* y, int n_slices, long long slice_stride,            \
                                           const float* bias, const float* w, const float* scale, float mult,         \
                                           float eps, void* h_out, int rows, int H, void* st) {                       \
    if (rows <= 0) return 0;                                                                                          \
    if (H <= 0 || n_slices < 1) return -2;                                                                            \
    return launch_pdl(scaled_norm_add_kernel<T>, dim3(rows), dim3(row_threads(H)), 0, (cudaStream_t)st, x, y,         \
                      n_slices, slice_stride, bias, w, scale, mult, eps, (T*)h_out, H);                               \
  }                                                                                                                   \
  TKB_EXPORT int tkb_cast_rows_##SUF(const float* x, void* out, long long n, void* st) {                              \
    if (n <= 0) return 0;                                                                                             \
    const long long blocks = (n + 1023) / 1024;                                                                       \
    return launch_pdl(cast_rows_kernel<T>, dim3((unsigned)(blocks < 4096 ? blocks : 4096)), dim3(256), 0,             \
                      (cudaStream_t)st, x, (T*)out, (size_t)n);                                                       \
  }                                                                                                                   \
  TKB_EXPORT int tkb_gated_group_norm_##SUF(const float* y, int y_stride, const float* gate, int gate_stride,         \
                                            const float* w, void* out, int out_stride, int rows, int width,           \
                                            int groups, float eps, int gate_first, void* st) {                        \
    if (rows <= 0) return 0;                                                                                          \
    if (groups <= 0 || width <= 0 || width % groups) return -2;                                                       \
    if (groups > 65535) return -3;                                                                                    \
    return launch_pdl(gated_group_norm_kernel<T>, dim3(rows, groups), dim3(row_threads(width / groups)), 0,           \
                      (cudaStream_t)st, y, y_stride, gate, gate_stride, w, (T*)out, out_stride, width / groups, eps,  \
                      gate_first);                                                                                    \
  }

TKB_POST_NORM_EXPORTS(f32, float)
TKB_POST_NORM_EXPORTS(bf16, __nv_bfloat16)

TKB_EXPORT int tkb_add_sinusoid(float* x, const int* positions, const double* freq, int rows, int H, void* st) {
  if (rows <= 0) return 0;
  return launch_pdl(add_sinusoid_kernel, dim3(rows), dim3(row_threads(H * 2)), 0, (cudaStream_t)st, x, positions,
                    freq, H);
}

// gate_up [rows, 2 * inner] (gate columns, then up columns) in the activation type or float32; out [rows, inner]
#define TKB_GLU_EXPORT(NAME, TI, TO)                                                                                  \
  TKB_EXPORT int NAME(const void* gate_up, void* out, int rows, int inner, float limit, float alpha, int interleave,  \
                      void* st) {                                                                                     \
    if (rows <= 0) return 0;                                                                                          \
    if (inner <= 0 || (interleave != 0 && (interleave != 8 || inner % 8))) return -2;                                 \
    return launch_pdl(clamped_glu_kernel<TI, TO>, dim3(rows), dim3(row_threads(inner * 4)), 0, (cudaStream_t)st,      \
                      (const TI*)gate_up, (TO*)out, inner, limit, alpha, interleave);                                 \
  }
TKB_GLU_EXPORT(tkb_clamped_glu_f32_f32, float, float)
TKB_GLU_EXPORT(tkb_clamped_glu_f32_bf16, float, __nv_bfloat16)
TKB_GLU_EXPORT(tkb_clamped_glu_bf16_bf16, __nv_bfloat16, __nv_bfloat16)
