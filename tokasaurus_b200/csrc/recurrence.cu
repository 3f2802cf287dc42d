// A gated linear recurrence with a matrix state per head (the HGRN2 form: the forget gate also decides what is
// written):
//     S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,      o_t = S_t^T q_t,
//     q = silu(q_raw),   f = low + (1 - low) * sigmoid(f_raw + f_bias),
// followed by an RMS norm of every head's o over its vdim values (weight shared by the heads).  The raw
// projections arrive as float32 rows [q_raw (H*dim) | f_raw (H*dim) | v (H*vdim)]; gates, state, sums and the norm are
// float32.  The state lives in the request's slot as S^T: state[slot][head][vdim][dim].
//
// Compile with -DTKB_REC_DPT=<dims per thread> and -DTKB_REC_CPT=<columns per thread>.
//
// One block owns one (request, head) and walks over the request's tokens of this step in order.  Eight threads
// share a column j of S (dims lane, lane + 8, ...), so a step of the recurrence is DPT fused multiply-adds and a
// three-step shuffle sum a thread.  Tokens are taken in chunks: all threads turn a chunk's raw rows into gates
// in shared memory, the chunk is walked in order, then the chunk's outputs are normalised and stored.
#include "common.cuh"

#ifndef TKB_REC_DPT
#error "compile with -DTKB_REC_DPT=<dims per thread>"
#endif
#ifndef TKB_REC_CPT
#define TKB_REC_CPT 1
#endif

using namespace tkb;

namespace {

constexpr int DPT = TKB_REC_DPT;
constexpr int CPT = TKB_REC_CPT;
constexpr int LANES = 8;   // threads that share a column
constexpr int CHUNK = 16;  // tokens staged at a time

template <typename T>
__global__ void __launch_bounds__(1024)
gated_recurrence_kernel(const float* __restrict__ qfv, int row_stride, float* __restrict__ state,
                        const float* __restrict__ f_bias, const float* __restrict__ low,
                        const float* __restrict__ norm_w, T* __restrict__ out, const int* __restrict__ seq_slot,
                        const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len, int heads, int dim,
                        int vdim, float eps, int write_state) {
  extern __shared__ float smem[];
  float* qs = smem;                 // [CHUNK][dim]
  float* fs = qs + CHUNK * dim;     // [CHUNK][dim]
  float* gs = fs + CHUNK * dim;     // [CHUNK][dim]   1 - f
  float* vs = gs + CHUNK * dim;     // [CHUNK][vdim]
  float* os = vs + CHUNK * vdim;    // [CHUNK][vdim]
  trigger_dependents();
  grid_dependency_wait();
  const int s = blockIdx.x, head = blockIdx.y;
  const int n = seq_q_len[s];
  if (n <= 0) return;
  const int start = seq_q_start[s];
  const int tid = threadIdx.x, lane = tid & (LANES - 1), col0 = tid / LANES;
  const int cols_per_pass = blockDim.x / LANES;
  float* st = state + ((size_t)seq_slot[s] * heads + head) * (size_t)vdim * dim;

  float S[CPT][DPT];
#pragma unroll
  for (int c = 0; c < CPT; c++) {
    const int j = col0 + c * cols_per_pass;
#pragma unroll
    for (int i = 0; i < DPT; i++) {
      const int d = lane + LANES * i;
      S[c][i] = (j < vdim && d < dim) ? st[(size_t)j * dim + d] : 0.f;
    }
  }
  const float* q_raw = qfv + (size_t)head * dim;
  const float* f_raw = qfv + (size_t)heads * dim + (size_t)head * dim;
  const float* v_raw = qfv + (size_t)2 * heads * dim + (size_t)head * vdim;
  const float* fb = f_bias + (size_t)head * dim;
  const float* lw = low + (size_t)head * dim;

  for (int t0 = 0; t0 < n; t0 += CHUNK) {
    const int nt = min(CHUNK, n - t0);
    __syncthreads();  // the chunk before is out of shared memory
    for (int idx = tid; idx < nt * dim; idx += blockDim.x) {
      const int t = idx / dim, d = idx - t * dim;
      const size_t row = (size_t)(start + t0 + t) * row_stride;
      const float qr = q_raw[row + d];
      const float fr = f_raw[row + d] + fb[d];
      const float sig = 1.f / (1.f + expf(-fr));
      const float l = lw[d];
      const float f = l + (1.f - l) * sig;
      qs[t * dim + d] = qr / (1.f + expf(-qr));
      fs[t * dim + d] = f;
      gs[t * dim + d] = 1.f - f;
    }
    for (int idx = tid; idx < nt * vdim; idx += blockDim.x) {
      const int t = idx / vdim, j = idx - t * vdim;
      vs[t * vdim + j] = v_raw[(size_t)(start + t0 + t) * row_stride + j];
    }
    __syncthreads();
    for (int t = 0; t < nt; t++) {
      const float* q = qs + t * dim;
      const float* f = fs + t * dim;
      const float* g = gs + t * dim;
#pragma unroll
      for (int c = 0; c < CPT; c++) {
        const int j = col0 + c * cols_per_pass;
        const float v = j < vdim ? vs[t * vdim + j] : 0.f;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < DPT; i++) {
          const int d = lane + LANES * i;
          if (d < dim) {
            S[c][i] = fmaf(f[d], S[c][i], g[d] * v);
            acc = fmaf(S[c][i], q[d], acc);
          }
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        acc += __shfl_xor_sync(0xffffffffu, acc, 4);
        if (lane == 0 && j < vdim) os[t * vdim + j] = acc;
      }
    }
    __syncthreads();
    // RMS norm of each token's o over vdim: one warp a token
    const int warp = tid >> 5, wl = tid & 31, nwarps = blockDim.x >> 5;
    for (int t = warp; t < nt; t += nwarps) {
      float ss = 0.f;
      for (int j = wl; j < vdim; j += 32) ss += os[t * vdim + j] * os[t * vdim + j];
      ss = warp_sum(ss);
      const float r = rsqrtf(ss / (float)vdim + eps);
      T* orow = out + (size_t)(start + t0 + t) * heads * vdim + (size_t)head * vdim;
      for (int j = wl; j < vdim; j += 32) orow[j] = from_float<T>(os[t * vdim + j] * r * norm_w[j]);
    }
  }
  if (write_state) {
#pragma unroll
    for (int c = 0; c < CPT; c++) {
      const int j = col0 + c * cols_per_pass;
#pragma unroll
      for (int i = 0; i < DPT; i++) {
        const int d = lane + LANES * i;
        if (j < vdim && d < dim) st[(size_t)j * dim + d] = S[c][i];
      }
    }
  }
}

template <typename T>
int launch(const float* qfv, int row_stride, float* state, const float* f_bias, const float* low, const float* norm_w,
           void* out, const int* seq_slot, const int* seq_q_start, const int* seq_q_len, int n_seqs, int heads, int dim,
           int vdim, float eps, int write_state, cudaStream_t st) {
  if (n_seqs <= 0) return 0;
  if (heads <= 0 || dim <= 0 || vdim <= 0 || dim > LANES * DPT || heads > 65535) return -2;
  int cols = (vdim + CPT - 1) / CPT;          // columns a pass
  int threads = ((cols * LANES + 31) / 32) * 32;
  if (threads > 1024 || (threads / LANES) * CPT < vdim) return -2;
  const size_t smem = (size_t)CHUNK * (3 * dim + 2 * vdim) * sizeof(float);
  if (smem > 200 * 1024) return -2;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(gated_recurrence_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return launch_pdl(gated_recurrence_kernel<T>, dim3(n_seqs, heads), dim3(threads), smem, st, qfv, row_stride, state,
                    f_bias, low, norm_w, (T*)out, seq_slot, seq_q_start, seq_q_len, heads, dim, vdim, eps, write_state);
}

}  // namespace

// qfv: float32 [tokens, row_stride]; state: float32 [slots, heads, vdim, dim]; out: [tokens, heads * vdim].
TKB_EXPORT int tkb_gated_recurrence_f32(const float* qfv, int row_stride, float* state, const float* f_bias,
                                        const float* low, const float* norm_w, void* out, const int* seq_slot,
                                        const int* seq_q_start, const int* seq_q_len, int n_seqs, int heads, int dim,
                                        int vdim, float eps, int write_state, void* st) {
  return launch<float>(qfv, row_stride, state, f_bias, low, norm_w, out, seq_slot, seq_q_start, seq_q_len, n_seqs, heads,
                       dim, vdim, eps, write_state, (cudaStream_t)st);
}
TKB_EXPORT int tkb_gated_recurrence_bf16(const float* qfv, int row_stride, float* state, const float* f_bias,
                                         const float* low, const float* norm_w, void* out, const int* seq_slot,
                                         const int* seq_q_start, const int* seq_q_len, int n_seqs, int heads, int dim,
                                         int vdim, float eps, int write_state, void* st) {
  return launch<__nv_bfloat16>(qfv, row_stride, state, f_bias, low, norm_w, out, seq_slot, seq_q_start, seq_q_len, n_seqs,
                               heads, dim, vdim, eps, write_state, (cudaStream_t)st);
}
TKB_EXPORT int tkb_gated_recurrence_dpt() { return DPT; }
TKB_EXPORT int tkb_gated_recurrence_cpt() { return CPT; }
