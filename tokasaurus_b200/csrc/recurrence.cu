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
// One block owns some columns of the state of one (request, head) and walks over the request's tokens of this step
// in order.  Eight threads share a column j of S (dims lane, lane + 8, ...), so a step of the recurrence is DPT
// fused multiply-adds and a three-step shuffle sum a thread.  Tokens are taken in chunks: all threads turn a chunk's
// raw rows into gates in shared memory, the chunk is walked in order, then the chunk's outputs are stored.  A block
// that owns all columns of its head normalises them itself; with the columns of a head split over several blocks
// (few requests with many tokens: the walk over the tokens is what takes the time, so it is spread over as many
// SMs as there are) the raw outputs go to a float32 buffer and a second kernel normalises them.
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
constexpr int SPLIT_THREADS_MAX = 256;  // the split form's blocks: few threads, many registers each

// In place on the raw rows: q_raw -> silu(q_raw), f_raw -> low + (1 - low) * sigmoid(f_raw + f_bias).  One block a
// token.  The split form below reads gates made by this kernel: a block of few threads would wait for its loads
// and exponentials chunk after chunk, all tokens at once do not.
__global__ void recurrence_gates_kernel(float* __restrict__ qfv, int row_stride, const float* __restrict__ f_bias,
                                        const float* __restrict__ low, int hd) {
  trigger_dependents();
  grid_dependency_wait();
  float* row = qfv + (size_t)blockIdx.x * row_stride;
  for (int i = threadIdx.x; i < hd; i += blockDim.x) {
    const float qr = row[i];
    const float fr = row[hd + i] + f_bias[i];
    const float l = low[i];
    row[i] = qr / (1.f + expf(-qr));
    row[hd + i] = l + (1.f - l) / (1.f + expf(-fr));
  }
}

template <typename T, bool PREGATED>
__global__ void __launch_bounds__(1024)
gated_recurrence_kernel(const float* __restrict__ qfv, int row_stride, float* __restrict__ state,
                        const float* __restrict__ f_bias, const float* __restrict__ low,
                        const float* __restrict__ norm_w, T* __restrict__ out, const int* __restrict__ seq_slot,
                        const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len, int heads, int dim,
                        int vdim, float eps, int write_state, int cols_per_block, float* __restrict__ raw_out) {
  extern __shared__ float smem[];
  float* qs = smem;                 // [CHUNK][dim]
  float* fs = qs + CHUNK * dim;     // [CHUNK][dim]
  float* vs = fs + CHUNK * dim;     // [CHUNK][vdim]
  float* os = vs + CHUNK * vdim;    // [CHUNK][vdim]
  trigger_dependents();
  grid_dependency_wait();
  const int s = blockIdx.x, head = blockIdx.y;
  const int n = seq_q_len[s];
  if (n <= 0) return;
  const int start = seq_q_start[s];
  const int tid = threadIdx.x, lane = tid & (LANES - 1);
  const int cols_per_pass = blockDim.x / LANES;
  const int col_begin = blockIdx.z * cols_per_block;
  const int col_end = min(vdim, col_begin + cols_per_block);
  const int col0 = col_begin + tid / LANES;
  float* st = state + ((size_t)seq_slot[s] * heads + head) * (size_t)vdim * dim;

  float S[CPT][DPT];
#pragma unroll
  for (int c = 0; c < CPT; c++) {
    const int j = col0 + c * cols_per_pass;
#pragma unroll
    for (int i = 0; i < DPT; i++) {
      const int d = lane + LANES * i;
      S[c][i] = (j < col_end && d < dim) ? st[(size_t)j * dim + d] : 0.f;
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
    if (PREGATED) {
#pragma unroll 4
      for (int idx = tid; idx < nt * dim; idx += blockDim.x) {
        const int t = idx / dim, d = idx - t * dim;
        const size_t row = (size_t)(start + t0 + t) * row_stride;
        qs[idx] = q_raw[row + d];
        fs[idx] = f_raw[row + d];
      }
    } else {
      for (int idx = tid; idx < nt * dim; idx += blockDim.x) {
        const int t = idx / dim, d = idx - t * dim;
        const size_t row = (size_t)(start + t0 + t) * row_stride;
        const float qr = q_raw[row + d];
        const float fr = f_raw[row + d] + fb[d];
        const float l = lw[d];
        qs[idx] = qr / (1.f + expf(-qr));
        fs[idx] = l + (1.f - l) / (1.f + expf(-fr));
      }
    }
#pragma unroll 4
    for (int idx = tid; idx < nt * vdim; idx += blockDim.x) {
      const int t = idx / vdim, j = idx - t * vdim;
      vs[idx] = v_raw[(size_t)(start + t0 + t) * row_stride + j];
    }
    __syncthreads();
    for (int t = 0; t < nt; t++) {
      const float* q = qs + t * dim;
      const float* f = fs + t * dim;
#pragma unroll
      for (int c = 0; c < CPT; c++) {
        const int j = col0 + c * cols_per_pass;
        const float v = j < col_end ? vs[t * vdim + j] : 0.f;
        // S <- f S + (1 - f) v = v + f (S - v); four running sums so that no chain of adds is longer than DPT / 4
        float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < DPT; i++) {
          const int d = lane + LANES * i;
          if (d < dim) {
            S[c][i] = fmaf(f[d], S[c][i] - v, v);
            part[i & 3] = fmaf(S[c][i], q[d], part[i & 3]);
          }
        }
        float acc = (part[0] + part[1]) + (part[2] + part[3]);
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        acc += __shfl_xor_sync(0xffffffffu, acc, 4);
        if (lane == 0 && j < col_end) os[t * vdim + j] = acc;
      }
    }
    __syncthreads();
    if (raw_out != nullptr) {
      for (int idx = tid; idx < nt * (col_end - col_begin); idx += blockDim.x) {
        const int t = idx / (col_end - col_begin), j = col_begin + idx - t * (col_end - col_begin);
        raw_out[(size_t)(start + t0 + t) * heads * vdim + (size_t)head * vdim + j] = os[t * vdim + j];
      }
      continue;
    }
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
        if (j < col_end && d < dim) st[(size_t)j * dim + d] = S[c][i];
      }
    }
  }
}

// The split form: a block owns cols_per_block columns of one (request, head), reads gates that
// recurrence_gates_kernel made, and writes raw outputs.  With few threads a block the loads of a chunk would be
// waited for one batch after the other, so the chunks come by cp.async (16 bytes a copy), the next chunk under way
// while the current one is walked.  Needs dim, vdim, cols_per_block and the row stride to be multiples of 4.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}

__global__ void __launch_bounds__(SPLIT_THREADS_MAX)
gated_recurrence_split_kernel(const float* __restrict__ qfv, int row_stride, float* __restrict__ state,
                              const int* __restrict__ seq_slot, const int* __restrict__ seq_q_start,
                              const int* __restrict__ seq_q_len, int heads, int dim, int vdim, int write_state,
                              int cols_per_block, float* __restrict__ raw_out) {
  extern __shared__ __align__(16) float smem[];
  // A thread's state values: with DPT a multiple of 4 the DPT consecutive dims lane * DPT ..., so that its gates
  // come out of shared memory as 16-byte vectors (a quarter of the loads); each thread's stretch of a row is
  // then SP floats apart, SP / 4 odd, which keeps the eight threads of a column on different banks.  Otherwise dims
  // lane, lane + 8, ... and plain loads.  A row of gates holds dim values, then zeros (no bounds in the walk).
  constexpr bool VEC = DPT % 4 == 0;
  constexpr int SP = VEC ? DPT + (((DPT / 4) % 2 == 0) ? 4 : 0) : DPT;
  constexpr int DIMP = LANES * SP;
  const int stage_floats = CHUNK * (2 * DIMP + cols_per_block);
  float* os = smem + 2 * stage_floats;  // [CHUNK][cols_per_block]
  trigger_dependents();
  grid_dependency_wait();
  const int s = blockIdx.x, head = blockIdx.y;
  const int n = seq_q_len[s];
  if (n <= 0) return;
  const int start = seq_q_start[s];
  const int tid = threadIdx.x, lane = tid & (LANES - 1);
  const int cols_per_pass = blockDim.x / LANES;
  const int col_begin = blockIdx.z * cols_per_block;
  const int col_end = min(vdim, col_begin + cols_per_block);
  const int ncols = col_end - col_begin;
  const int col0 = tid / LANES;  // within the block's columns
  float* st = state + ((size_t)seq_slot[s] * heads + head) * (size_t)vdim * dim;
  float S[CPT][DPT];
#pragma unroll
  for (int c = 0; c < CPT; c++) {
    const int j = col0 + c * cols_per_pass;
#pragma unroll
    for (int i = 0; i < DPT; i++) {
      const int d = VEC ? lane * DPT + i : lane + LANES * i;
      S[c][i] = (j < ncols && d < dim) ? st[(size_t)(col_begin + j) * dim + d] : 0.f;
    }
  }
  const float* q_src = qfv + (size_t)head * dim;
  const float* f_src = qfv + (size_t)heads * dim + (size_t)head * dim;
  const float* v_src = qfv + (size_t)2 * heads * dim + (size_t)head * vdim + col_begin;
  const int d4 = dim >> 2, c4 = ncols >> 2;
  auto fetch = [&](int t0, int buf) {
    const int nt = min(CHUNK, n - t0);
    float* qs = smem + buf * stage_floats;
    float* fs = qs + CHUNK * DIMP;
    float* vs = fs + CHUNK * DIMP;
    for (int idx = tid; idx < nt * d4; idx += blockDim.x) {
      const int t = idx / d4, k = (idx - t * d4) * 4;
      const size_t row = (size_t)(start + t0 + t) * row_stride;
      const int at = VEC ? (k / DPT) * SP + (k % DPT) : k;
      cp_async16(qs + t * DIMP + at, q_src + row + k);
      cp_async16(fs + t * DIMP + at, f_src + row + k);
    }
    for (int idx = tid; idx < nt * c4; idx += blockDim.x) {
      const int t = idx / c4, k = (idx - t * c4) * 4;
      cp_async16(vs + t * cols_per_block + k, v_src + (size_t)(start + t0 + t) * row_stride + k);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // beyond dim: f = 0 and q = 0, so such a state entry takes the value v and adds nothing to any sum
  for (int idx = tid; idx < 2 * stage_floats; idx += blockDim.x) smem[idx] = 0.f;
  __syncthreads();
  fetch(0, 0);
  int buf = 0;
  for (int t0 = 0; t0 < n; t0 += CHUNK, buf ^= 1) {
    const int nt = min(CHUNK, n - t0);
    if (t0 + CHUNK < n) {
      fetch(t0 + CHUNK, buf ^ 1);  // the buffer the chunk before this one was walked in; its readers passed the barrier below
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const float* qs = smem + buf * stage_floats;
    const float* fs = qs + CHUNK * DIMP;
    const float* vs = fs + CHUNK * DIMP;
    for (int t = 0; t < nt; t++) {
      const float* q = qs + t * DIMP;
      const float* f = fs + t * DIMP;
#pragma unroll
      for (int c = 0; c < CPT; c++) {
        const int j = col0 + c * cols_per_pass;
        const float v = j < ncols ? vs[t * cols_per_block + j] : 0.f;
        float part[4] = {0.f, 0.f, 0.f, 0.f};
        if (VEC) {
#pragma unroll
          for (int i4 = 0; i4 < DPT / 4; i4++) {
            const float4 f4 = *reinterpret_cast<const float4*>(f + lane * SP + 4 * i4);
            const float4 q4 = *reinterpret_cast<const float4*>(q + lane * SP + 4 * i4);
            float* Sc = &S[c][(4 * i4) % DPT];
            Sc[0] = fmaf(f4.x, Sc[0] - v, v);
            Sc[1] = fmaf(f4.y, Sc[1] - v, v);
            Sc[2] = fmaf(f4.z, Sc[2] - v, v);
            Sc[3] = fmaf(f4.w, Sc[3] - v, v);
            part[0] = fmaf(Sc[0], q4.x, part[0]);
            part[1] = fmaf(Sc[1], q4.y, part[1]);
            part[2] = fmaf(Sc[2], q4.z, part[2]);
            part[3] = fmaf(Sc[3], q4.w, part[3]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < DPT; i++) {
            const int d = lane + LANES * i;
            S[c][i] = fmaf(f[d], S[c][i] - v, v);
            part[i & 3] = fmaf(S[c][i], q[d], part[i & 3]);
          }
        }
        float acc = (part[0] + part[1]) + (part[2] + part[3]);
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        acc += __shfl_xor_sync(0xffffffffu, acc, 4);
        if (lane == 0 && j < ncols) os[t * cols_per_block + j] = acc;
      }
    }
    __syncthreads();  // os complete; everybody is done with this chunk's buffer
    for (int idx = tid; idx < nt * ncols; idx += blockDim.x) {
      const int t = idx / ncols, j = idx - t * ncols;
      raw_out[(size_t)(start + t0 + t) * heads * vdim + (size_t)head * vdim + col_begin + j] = os[t * cols_per_block + j];
    }
    // the next iteration's barrier (after its wait) stands between these reads of os and the next writes to it
  }
  if (write_state) {
#pragma unroll
    for (int c = 0; c < CPT; c++) {
      const int j = col0 + c * cols_per_pass;
#pragma unroll
      for (int i = 0; i < DPT; i++) {
        const int d = VEC ? lane * DPT + i : lane + LANES * i;
        if (j < ncols && d < dim) st[(size_t)(col_begin + j) * dim + d] = S[c][i];
      }
    }
  }
}

// out[t][head] = raw[t][head] / sqrt(mean(raw[t][head]^2) + eps) * w: one warp a (token, head).
template <typename T>
__global__ void head_rmsnorm_kernel(const float* __restrict__ raw, const float* __restrict__ w, T* __restrict__ out,
                                    int n_rows, int vdim, float eps) {
  trigger_dependents();
  grid_dependency_wait();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  const float* r = raw + (size_t)row * vdim;
  float ss = 0.f;
  for (int j = lane; j < vdim; j += 32) ss += r[j] * r[j];
  const float k = rsqrtf(warp_sum(ss) / (float)vdim + eps);
  for (int j = lane; j < vdim; j += 32) out[(size_t)row * vdim + j] = from_float<T>(r[j] * k * w[j]);
}

template <typename T>
int launch(float* qfv, int row_stride, float* state, const float* f_bias, const float* low, const float* norm_w,
           void* out, const int* seq_slot, const int* seq_q_start, const int* seq_q_len, int n_seqs, int n_tokens,
           int heads, int dim, int vdim, float eps, int write_state, float* raw, cudaStream_t st) {
  if (n_seqs <= 0) return 0;
  if (heads <= 0 || dim <= 0 || vdim <= 0 || dim > LANES * DPT || heads > 65535) return -2;
  // columns a block: all of the head's, unless the requests and heads alone leave SMs idle and a buffer for raw
  // outputs is at hand; then as many blocks a head as fill the SMs about twice, at least four columns each
  int split = 1;
  if (raw != nullptr && n_tokens > n_seqs) {
    const int want = (2 * tkb::sm_count() + n_seqs * heads - 1) / (n_seqs * heads);
    split = max(1, min(want, vdim / 4));
  }
  int cols_per_block = (vdim + split - 1) / split;
  cols_per_block = (cols_per_block + 3) / 4 * 4;
  split = (vdim + cols_per_block - 1) / cols_per_block;
  const int cols = (cols_per_block + CPT - 1) / CPT;  // columns a pass
  const int threads = ((cols * LANES + 31) / 32) * 32;
  if (threads > 1024 || (threads / LANES) * CPT < cols_per_block) return -2;
  const size_t smem = (size_t)CHUNK * (2 * dim + 2 * vdim) * sizeof(float);
  if (smem > 200 * 1024) return -2;
  if (smem > 48 * 1024) {
    cudaFuncSetAttribute(gated_recurrence_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(gated_recurrence_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  float* raw_out = split > 1 ? raw : nullptr;
  if (raw_out == nullptr)
    return launch_pdl(gated_recurrence_kernel<T, false>, dim3(n_seqs, heads, 1), dim3(threads), smem, st,
                      (const float*)qfv, row_stride, state, f_bias, low, norm_w, (T*)out, seq_slot, seq_q_start,
                      seq_q_len, heads, dim, vdim, eps, write_state, cols_per_block, raw_out);
  int rc = launch_pdl(recurrence_gates_kernel, dim3(n_tokens), dim3(heads * dim >= 1024 ? 256 : 128), 0, st, qfv,
                      row_stride, f_bias, low, heads * dim);
  if (rc != 0) return rc;
  const bool by_16 = dim % 4 == 0 && vdim % 4 == 0 && row_stride % 4 == 0 && (((uintptr_t)qfv) & 15) == 0;
  constexpr int SPLIT_SP = (DPT % 4 == 0) ? DPT + (((DPT / 4) % 2 == 0) ? 4 : 0) : DPT;  // as in the kernel
  const size_t smem_split = (size_t)CHUNK * (2 * (2 * LANES * SPLIT_SP + cols_per_block) + cols_per_block) * sizeof(float);
  if (by_16 && smem_split <= 200 * 1024 && threads <= SPLIT_THREADS_MAX) {
    if (smem_split > 48 * 1024)
      cudaFuncSetAttribute(gated_recurrence_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_split);
    rc = launch_pdl(gated_recurrence_split_kernel, dim3(n_seqs, heads, split), dim3(threads), smem_split, st,
                    (const float*)qfv, row_stride, state, seq_slot, seq_q_start, seq_q_len, heads, dim, vdim, write_state,
                    cols_per_block, raw_out);
  } else {
    rc = launch_pdl(gated_recurrence_kernel<T, true>, dim3(n_seqs, heads, split), dim3(threads), smem, st,
                    (const float*)qfv, row_stride, state, f_bias, low, norm_w, (T*)out, seq_slot, seq_q_start, seq_q_len,
                    heads, dim, vdim, eps, write_state, cols_per_block, raw_out);
  }
  if (rc != 0) return rc;
  const int rows = n_tokens * heads;
  return launch_pdl(head_rmsnorm_kernel<T>, dim3((rows + 7) / 8), dim3(256), 0, st, (const float*)raw_out, norm_w, (T*)out,
                    rows, vdim, eps);
}

}  // namespace

// qfv: float32 [tokens, row_stride]; state: float32 [slots, heads, vdim, dim]; out: [tokens, heads * vdim];
// raw: float32 [tokens, heads * vdim] scratch for the split form, or null (every block then owns a whole head).
// The split form turns the q and f columns of qfv into gates in place.
TKB_EXPORT int tkb_gated_recurrence_f32(float* qfv, int row_stride, float* state, const float* f_bias,
                                        const float* low, const float* norm_w, void* out, const int* seq_slot,
                                        const int* seq_q_start, const int* seq_q_len, int n_seqs, int n_tokens,
                                        int heads, int dim, int vdim, float eps, int write_state, float* raw, void* st) {
  return launch<float>(qfv, row_stride, state, f_bias, low, norm_w, out, seq_slot, seq_q_start, seq_q_len, n_seqs,
                       n_tokens, heads, dim, vdim, eps, write_state, raw, (cudaStream_t)st);
}
TKB_EXPORT int tkb_gated_recurrence_bf16(float* qfv, int row_stride, float* state, const float* f_bias,
                                         const float* low, const float* norm_w, void* out, const int* seq_slot,
                                         const int* seq_q_start, const int* seq_q_len, int n_seqs, int n_tokens,
                                         int heads, int dim, int vdim, float eps, int write_state, float* raw, void* st) {
  return launch<__nv_bfloat16>(qfv, row_stride, state, f_bias, low, norm_w, out, seq_slot, seq_q_start, seq_q_len, n_seqs,
                               n_tokens, heads, dim, vdim, eps, write_state, raw, (cudaStream_t)st);
}
TKB_EXPORT int tkb_gated_recurrence_dpt() { return DPT; }
TKB_EXPORT int tkb_gated_recurrence_cpt() { return CPT; }
