// A linear recurrence with a matrix state per head and ONE decay number per head and token:
//
//     S_t = a_t S_(t-1) + (c_t k_t) v_t^T,        o_t = S_t^T q_t + D v_t
//
// (S is dim x vdim; k_t, q_t have dim entries, v_t has vdim).  Two mixers are instances of it:
//   * decayed linear attention: a_t = lambda_head (a constant), c_t = 1, D = 0, q, k, v = silu of the projections, one
//     q and k per head;
//   * the selective state space (state-space duality form): a_t = exp(-exp(A_head) dt_t), c_t = dt_t, k = B, q = C
//     shared by the heads of a group, v = x, D a number per head; x, B and C come out of a causal convolution over
//     time with bias and SiLU, dt_t = softplus(dt_raw + dt_bias).
// Everything here is float32: projections arrive as float32 rows, the state lives in the request's slot as S^T,
// state[slot][head][vdim][dim], and the outputs leave as float32 rows for the norm that follows.
//
// Kernels: ssm_prep (convolution + SiLU for every channel of [x | B | C], dt and the decay; one block a token; inputs
// from before the step come from the request's carried inputs), conv_carry (brings the carried inputs forward after
// every token has read them), decay_walk (the recurrence).
//
// The walk: one block owns some columns of the state of one (request, head) and goes over the request's tokens of
// this step in order.  Eight threads share a column j of S (dims lane, lane + 8, ...): a step is DPT multiply-adds
// and a three-step shuffle sum a thread.  Tokens are staged in chunks of 16 in shared memory.  With few requests and
// many tokens a head's columns are spread over as many blocks as fill the SMs twice: the chain over the tokens is
// what takes the time.
//
// Compile with -DTKB_DR_DPT=<ceil(dim / 8)> and -DTKB_DR_CPT=<ceil(vdim / 128)>.
#include "common.cuh"

#ifndef TKB_DR_DPT
#error "compile with -DTKB_DR_DPT=<dims per thread>"
#endif
#ifndef TKB_DR_CPT
#define TKB_DR_CPT 1
#endif

using namespace tkb;

namespace {

constexpr int DPT = TKB_DR_DPT;
constexpr int CPT = TKB_DR_CPT;
constexpr int LANES = 8;
constexpr int DIM_PAD = DPT * LANES;
constexpr int CHUNK = 16;

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
// log(1 + e^z); beyond 20 the sum is z itself in float32
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// proj: float32 [T, stride]; channels xbc_off .. xbc_off + C are convolved, columns dt_off .. dt_off + H are step sizes
__global__ void __launch_bounds__(512)
ssm_prep_kernel(const float* __restrict__ proj, int stride, int xbc_off, int C, int taps,
                const float* __restrict__ conv_w, const float* __restrict__ conv_b, const float* __restrict__ state,
                long long slot_stride, long long carry_off, const int* __restrict__ token_seq,
                const int* __restrict__ seq_slot, const int* __restrict__ seq_q_start, float* __restrict__ xbc,
                int dt_off, int H, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                float* __restrict__ dt_dec) {
  trigger_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int s = token_seq[t];
  if (s < 0) return;
  const int i = t - seq_q_start[s];
  const float* carry = state + (size_t)seq_slot[s] * slot_stride + carry_off;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = conv_b ? conv_b[c] : 0.f;
    for (int j = 0; j < taps; j++) {
      const int back = taps - 1 - j;  // how many tokens before this one
      float u;
      if (i - back >= 0) u = proj[(size_t)(t - back) * stride + xbc_off + c];
      else u = carry[(size_t)(i + j) * C + c];
      acc = fmaf(conv_w[(size_t)c * taps + j], u, acc);
    }
    xbc[(size_t)t * C + c] = silu_f(acc);
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float dt = softplus_f(proj[(size_t)t * stride + dt_off + h] + dt_bias[h]);
    dt_dec[(size_t)t * 2 * H + h] = dt;
    dt_dec[(size_t)t * 2 * H + H + h] = expf(-expf(a_log[h]) * dt);
  }
}

// One block a request: the last taps - 1 inputs of [carried inputs ; this step's inputs] become the carried inputs.
__global__ void __launch_bounds__(512)
conv_carry_kernel(const float* __restrict__ proj, int stride, int xbc_off, int C, int taps, float* __restrict__ state,
                  long long slot_stride, long long carry_off, const int* __restrict__ seq_slot,
                  const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len) {
  trigger_dependents();
  grid_dependency_wait();
  const int s = blockIdx.x;
  const int n = seq_q_len[s];
  if (n <= 0) return;
  const int start = seq_q_start[s];
  float* carry = state + (size_t)seq_slot[s] * slot_stride + carry_off;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    for (int r = 0; r < taps - 1; r++) {  // ascending: row n + r is read before it is written
      const int at = n + r;               // index in [carried ; new]
      carry[(size_t)r * C + c] = at < taps - 1 ? carry[(size_t)at * C + c]
                                               : proj[(size_t)(start + at - (taps - 1)) * stride + xbc_off + c];
    }
  }
}

template <bool ACT>
__global__ void __launch_bounds__(1024)
decay_walk_kernel(const float* __restrict__ q, int q_stride, const float* __restrict__ k, int k_stride, int qk_div,
                  const float* __restrict__ v, int v_stride, const float* __restrict__ dt_dec,
                  const float* __restrict__ decay_head, const float* __restrict__ skip, float* __restrict__ state,
                  long long slot_stride, float* __restrict__ out, const int* __restrict__ seq_slot,
                  const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len, int heads, int dim, int vdim,
                  int write_state, int cols_per_block) {
  extern __shared__ float smem[];
  const int cols = min(cols_per_block, vdim);
  float* qs = smem;                       // [CHUNK][DIM_PAD]
  float* ks = qs + CHUNK * DIM_PAD;       // [CHUNK][DIM_PAD]
  float* vs = ks + CHUNK * DIM_PAD;       // [CHUNK][cols]
  float* os = vs + CHUNK * cols;          // [CHUNK][cols]
  float* as = os + CHUNK * cols;          // [CHUNK] decay
  float* cs = as + CHUNK;                 // [CHUNK] key scale
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
  if (col_begin >= col_end) return;
  const int lc0 = tid / LANES;  // local column of the first pass
  float* st = state + (size_t)seq_slot[s] * slot_stride + (size_t)head * vdim * dim;

  float S[CPT][DPT];
#pragma unroll
  for (int c = 0; c < CPT; c++) {
    const int j = col_begin + lc0 + c * cols_per_pass;
#pragma unroll
    for (int i = 0; i < DPT; i++) {
      const int d = lane + LANES * i;
      S[c][i] = (j < col_end && d < dim) ? st[(size_t)j * dim + d] : 0.f;
    }
  }
  const float* qh = q + (size_t)(head / qk_div) * dim;
  const float* kh = k + (size_t)(head / qk_div) * dim;
  const float* vh = v + (size_t)head * vdim + col_begin;
  const float a_const = decay_head ? decay_head[head] : 1.f;
  const float d_skip = skip ? skip[head] : 0.f;
  const int ncols = col_end - col_begin;

  for (int t0 = 0; t0 < n; t0 += CHUNK) {
    const int nt = min(CHUNK, n - t0);
    __syncthreads();  // the chunk before is out of shared memory
    for (int idx = tid; idx < nt * DIM_PAD; idx += blockDim.x) {
      const int t = idx / DIM_PAD, d = idx - t * DIM_PAD;
      float qv = 0.f, kv = 0.f;
      if (d < dim) {
        qv = qh[(size_t)(start + t0 + t) * q_stride + d];
        kv = kh[(size_t)(start + t0 + t) * k_stride + d];
        if (ACT) { qv = silu_f(qv); kv = silu_f(kv); }
      }
      qs[idx] = qv;
      ks[idx] = kv;
    }
    for (int idx = tid; idx < nt * ncols; idx += blockDim.x) {
      const int t = idx / ncols, j = idx - t * ncols;
      float vv = vh[(size_t)(start + t0 + t) * v_stride + j];
      if (ACT) vv = silu_f(vv);
      vs[t * cols + j] = vv;
    }
    if (tid < nt) {
      as[tid] = dt_dec ? dt_dec[(size_t)(start + t0 + tid) * 2 * heads + heads + head] : a_const;
      cs[tid] = dt_dec ? dt_dec[(size_t)(start + t0 + tid) * 2 * heads + head] : 1.f;
    }
    __syncthreads();
    for (int t = 0; t < nt; t++) {
      const float a = as[t], ck = cs[t];
      const float* qt = qs + t * DIM_PAD;
      const float* kt = ks + t * DIM_PAD;
#pragma unroll
      for (int c = 0; c < CPT; c++) {
        const int lc = lc0 + c * cols_per_pass;
        const float vj = lc < ncols ? vs[t * cols + lc] : 0.f;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < DPT; i++) {
          const int d = lane + LANES * i;
          S[c][i] = fmaf(a, S[c][i], (kt[d] * ck) * vj);
          acc = fmaf(S[c][i], qt[d], acc);
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        acc += __shfl_xor_sync(0xffffffffu, acc, 4);
        if (lane == 0 && lc < ncols) os[t * cols + lc] = fmaf(d_skip, vj, acc);
      }
    }
    __syncthreads();
    for (int idx = tid; idx < nt * ncols; idx += blockDim.x) {
      const int t = idx / ncols, j = idx - t * ncols;
      out[(size_t)(start + t0 + t) * heads * vdim + (size_t)head * vdim + col_begin + j] = os[t * cols + j];
    }
  }
  if (write_state) {
#pragma unroll
    for (int c = 0; c < CPT; c++) {
      const int j = col_begin + lc0 + c * cols_per_pass;
#pragma unroll
      for (int i = 0; i < DPT; i++) {
        const int d = lane + LANES * i;
        if (j < col_end && d < dim) st[(size_t)j * dim + d] = S[c][i];
      }
    }
  }
}

template <bool ACT>
int walk_launch(const float* q, int q_stride, const float* k, int k_stride, int qk_div, const float* v, int v_stride,
                const float* dt_dec, const float* decay_head, const float* skip, float* state, long long slot_stride,
                float* out, const int* seq_slot, const int* seq_q_start, const int* seq_q_len, int n_seqs, int n_tokens,
                int heads, int dim, int vdim, int write_state, cudaStream_t st) {
  if (n_seqs <= 0 || n_tokens <= 0) return 0;
  if (dim <= 0 || dim > DIM_PAD || vdim <= 0 || vdim > CPT * 128 || heads <= 0 || qk_div <= 0) return -2;
  if (heads > 65535) return -3;
  int cols_per_block = vdim;
  if (n_tokens > n_seqs) {  // portions: spread a head's columns over blocks until the SMs are filled twice
    const int want = 2 * sm_count();
    const int have = n_seqs * heads;
    const int splits = have >= want ? 1 : (want + have - 1) / have;
    cols_per_block = (vdim + splits - 1) / splits;
    cols_per_block = ((cols_per_block + 3) / 4) * 4;
    if (cols_per_block > vdim) cols_per_block = vdim;
  }
  const int splits = (vdim + cols_per_block - 1) / cols_per_block;
  int per_pass = (cols_per_block + CPT - 1) / CPT;
  if (per_pass > 128) per_pass = 128;
  int threads = ((per_pass * LANES + 31) / 32) * 32;
  const int cols = cols_per_block < vdim ? cols_per_block : vdim;
  const size_t smem = (size_t)(CHUNK * (2 * DIM_PAD + 2 * cols) + 2 * CHUNK) * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(decay_walk_kernel<ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return launch_pdl(decay_walk_kernel<ACT>, dim3(n_seqs, heads, splits), dim3(threads), smem, st, q, q_stride, k,
                    k_stride, qk_div, v, v_stride, dt_dec, decay_head, skip, state, slot_stride, out, seq_slot,
                    seq_q_start, seq_q_len, heads, dim, vdim, write_state, cols_per_block);
}

}  // namespace

TKB_EXPORT int tkb_ssm_prep(const float* proj, int stride, int xbc_off, int C, int taps, const float* conv_w,
                            const float* conv_b, float* state, long long slot_stride, long long carry_off,
                            const int* token_seq, const int* seq_slot, const int* seq_q_start, const int* seq_q_len,
                            int n_tokens, int n_seqs, float* xbc, int dt_off, int H, const float* dt_bias,
                            const float* a_log, float* dt_dec, int write_state, void* st) {
  if (n_tokens <= 0) return 0;
  if (taps < 1 || C <= 0 || H <= 0) return -2;
  int threads = 32;
  while (threads < C && threads < 512) threads <<= 1;
  int rc = launch_pdl(ssm_prep_kernel, dim3(n_tokens), dim3(threads), 0, (cudaStream_t)st, proj, stride, xbc_off, C,
                      taps, conv_w, conv_b, (const float*)state, slot_stride, carry_off, token_seq, seq_slot,
                      seq_q_start, xbc, dt_off, H, dt_bias, a_log, dt_dec);
  if (rc != 0 || !write_state || taps < 2 || n_seqs <= 0) return rc;
  return launch_pdl(conv_carry_kernel, dim3(n_seqs), dim3(threads), 0, (cudaStream_t)st, proj, stride, xbc_off, C,
                    taps, state, slot_stride, carry_off, seq_slot, seq_q_start, seq_q_len);
}

// act != 0: q, k and v pass through SiLU on their way in.  dt_dec: float32 [T, 2 * heads] (key scale, then decay) or
// null, then decay_head [heads] is the decay and the key scale is 1.  skip: [heads] or null.
TKB_EXPORT int tkb_decay_walk(const float* q, int q_stride, const float* k, int k_stride, int qk_div, const float* v,
                              int v_stride, const float* dt_dec, const float* decay_head, const float* skip,
                              float* state, long long slot_stride, float* out, const int* seq_slot,
                              const int* seq_q_start, const int* seq_q_len, int n_seqs, int n_tokens, int heads, int dim,
                              int vdim, int write_state, int act, void* st) {
  if (act)
    return walk_launch<true>(q, q_stride, k, k_stride, qk_div, v, v_stride, dt_dec, decay_head, skip, state, slot_stride,
                             out, seq_slot, seq_q_start, seq_q_len, n_seqs, n_tokens, heads, dim, vdim, write_state,
                             (cudaStream_t)st);
  return walk_launch<false>(q, q_stride, k, k_stride, qk_div, v, v_stride, dt_dec, decay_head, skip, state, slot_stride,
                            out, seq_slot, seq_q_start, seq_q_len, n_seqs, n_tokens, heads, dim, vdim, write_state,
                            (cudaStream_t)st);
}
