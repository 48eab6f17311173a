// Matrix-memory recurrent layer (mLSTM) over the slot pool.
//
// Per head, with log input gate i_t, log forget gate f_t and a running maximum m (m_0 = 0):
//     m_t = max(f_t + m_{t-1}, i_t)
//     S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T          (S: dim x vdim)
//     n_t = exp(f_t + m_{t-1} - m_t) n_{t-1} + exp(i_t - m_t) k_t
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
// followed by o_t / rms(o_t) per head, the norm weight and the output gate sigmoid(g_t).  S, n, m live in 32-bit floats in
// the slot pool and are carried from step to step; a sequence whose slot holds no tokens yet starts from zero.
//
// pcs_mlstm_gates  one block per token: the two gate pre-activations of every head as 32-bit dot products, capped by
//                  cap * tanh(. / cap); the forget gate additionally through logsigmoid.
// pcs_mlstm_scan   the token-by-token kernel (one block per sequence, head and slice of value columns, S in shared memory)
//                  and the per-head output norm with the output gate.
#include "seq_common.cuh"

namespace pcs {

__device__ __forceinline__ float logsigmoidf_(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

template <typename T>
__global__ void __launch_bounds__(256) mlstm_gates_kernel(const T* __restrict__ h, long long h_stride, const T* __restrict__ w_i,
                                                          const T* __restrict__ w_f, const float* __restrict__ b_i,
                                                          const float* __restrict__ b_f, float* __restrict__ ig,
                                                          float* __restrict__ fg, int width, int heads, float cap) {
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const T* hr = h + t * h_stride;
  for (int o = warp; o < 2 * heads; o += nw) {
    const int head = o >> 1, is_f = o & 1;
    const T* w = (is_f ? w_f : w_i) + static_cast<long long>(head) * width;
    float a = 0.f;
    for (int i = lane; i < width; i += 32) a = fmaf(ldf(hr + i), ldf(w + i), a);
    a = warp_sum(a);
    if (lane == 0) {
      const float z = cap * tanhf((a + (is_f ? b_f[head] : b_i[head])) / cap);
      if (is_f) fg[static_cast<long long>(t) * heads + head] = logsigmoidf_(z);
      else ig[static_cast<long long>(t) * heads + head] = z;
    }
  }
}

// Grid (sequence, head, slice of value columns): the columns of S evolve independently given the gates, k and q, so a head's
// state is cut into slices of VS columns, one block each (a 256 x 512 state does not fit one SM's shared memory, and a
// decode step gets heads x slices blocks instead of heads).  The scalar n . q is recomputed by every slice; only slice 0
// stores n and m.  The block writes the unnormalised o_t = S_t^T q_t / den into a 32-bit buffer; the per-head norm needs all
// slices and runs afterwards (mlstm_out_kernel).  blockDim.x = round_up(VS * R, 32): thread (r, c) owns rows r, r + R, ...
// of column c; threads past VS * R only take part in loads and reductions.
template <typename T>
__global__ void __launch_bounds__(1024) mlstm_scan_kernel(const pcs_mlstm_params p, float* __restrict__ o_raw,
                                                          float* __restrict__ nm_new, int VS, int R) {
  extern __shared__ float sm[];
  __shared__ float red[33];
  const int D = p.dim, V = p.vdim, H = p.heads;
  const int v0 = blockIdx.z * VS, vs = min(VS, V - v0);
  float* S = sm;                 // [D][VS]
  float* nvec = S + D * VS;      // [D]
  float* ks = nvec + D;          // [D]
  float* qs = ks + D;            // [D]
  float* vsm = qs + D;           // [VS]
  float* part = vsm + VS;        // [R][VS]
  const int b = blockIdx.x, head = blockIdx.y, tid = threadIdx.x, nthr = blockDim.x;
  const int slot = p.seq_slot[b], pos0 = p.seq_pos0[b], len = p.seq_len[b], off = p.seq_off[b];
  if (len <= 0) return;
  float* Sg = p.s_pool + (static_cast<long long>(slot) * H + head) * D * V;
  float* ng = p.n_pool + (static_cast<long long>(slot) * H + head) * D;
  float* mg = p.m_pool + static_cast<long long>(slot) * H + head;
  const bool fresh = pos0 == 0;
  for (int e = tid; e < D * vs; e += nthr) {
    const int d = e / vs, c = e - d * vs;
    S[d * VS + c] = fresh ? 0.f : Sg[d * V + v0 + c];
  }
  for (int d = tid; d < D; d += nthr) nvec[d] = fresh ? 0.f : ng[d];
  float m = fresh ? 0.f : *mg;
  const int c = tid % VS, r = tid / VS;
  const bool active = r < R && c < vs;
  __syncthreads();
  for (int i = 0; i < len; ++i) {
    const long long t = off + i;
    const T* row = static_cast<const T*>(p.proj) + t * p.row_stride;
    for (int d = tid; d < D; d += nthr) {
      ks[d] = ldf(row + p.k_off + head * D + d);
      qs[d] = ldf(row + p.q_off + head * D + d) * p.q_scale;
    }
    for (int e = tid; e < vs; e += nthr) vsm[e] = ldf(row + p.v_off + head * V + v0 + e);
    const float ig = p.ig[t * H + head], fg = p.fg[t * H + head];
    const float m_new = fmaxf(fg + m, ig);
    const float a = expf(fg + m - m_new), bb = expf(ig - m_new);
    m = m_new;
    __syncthreads();
    float nq = 0.f;
    for (int d = tid; d < D; d += nthr) {
      const float nn = fmaf(a, nvec[d], bb * ks[d]);
      nvec[d] = nn;
      nq = fmaf(nn, qs[d], nq);
    }
    if (active) {
      const float bv = bb * vsm[c];
      float num = 0.f;
      for (int d = r; d < D; d += R) {
        const float sv = fmaf(a, S[d * VS + c], ks[d] * bv);
        S[d * VS + c] = sv;
        num = fmaf(sv, qs[d], num);
      }
      part[r * VS + c] = num;
    }
    nq = block_sum(nq, red);  // its barriers also publish `part`
    const float den = fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
    if (tid < vs) {
      float o = 0.f;
      for (int rr = 0; rr < R; ++rr) o += part[rr * VS + tid];
      o_raw[t * (static_cast<long long>(H) * V) + head * V + v0 + tid] = o / den;
    }
    __syncthreads();  // ks / qs / vsm / part are rewritten by the next token
  }
  for (int e = tid; e < D * vs; e += nthr) {
    const int d = e / vs, cc = e - d * vs;
    Sg[d * V + v0 + cc] = S[d * VS + cc];
  }
  // the other slices of this head may not have read the old n and m yet: the new ones are parked and committed afterwards
  if (blockIdx.z == 0) {
    float* dst = nm_new + (static_cast<long long>(b) * H + head) * (D + 1);
    for (int d = tid; d < D; d += nthr) dst[d] = nvec[d];
    if (tid == 0) dst[D] = m;
  }
}

__global__ void __launch_bounds__(128) mlstm_commit_kernel(const pcs_mlstm_params p, const float* __restrict__ nm_new) {
  const int b = blockIdx.x, head = blockIdx.y, D = p.dim, H = p.heads;
  if (p.seq_len[b] <= 0) return;
  const int slot = p.seq_slot[b];
  const float* src = nm_new + (static_cast<long long>(b) * H + head) * (D + 1);
  float* ng = p.n_pool + (static_cast<long long>(slot) * H + head) * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) ng[d] = src[d];
  if (threadIdx.x == 0) p.m_pool[static_cast<long long>(slot) * H + head] = src[D];
}

// out[t, head, :] = o / rms(o) * norm_w * sigmoid(g): one block per (token, head).
template <typename T>
__global__ void __launch_bounds__(256) mlstm_out_kernel(const pcs_mlstm_params p, const float* __restrict__ o_raw) {
  __shared__ float red[33];
  const long long t = blockIdx.x;
  const int head = blockIdx.y, V = p.vdim, H = p.heads;
  const float* o = o_raw + t * (static_cast<long long>(H) * V) + head * V;
  const T* g = static_cast<const T*>(p.proj) + t * p.row_stride + p.g_off + head * V;
  const T* nw = static_cast<const T*>(p.norm_w) + head * V;
  float ss = 0.f;
  for (int c = threadIdx.x; c < V; c += blockDim.x) ss = fmaf(o[c], o[c], ss);
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / static_cast<float>(V) + p.eps);
  T* out = static_cast<T*>(p.out) + t * (static_cast<long long>(H) * V) + head * V;
  for (int c = threadIdx.x; c < V; c += blockDim.x) stf(out + c, o[c] * inv * ldf(nw + c) * sigmoidf_(ldf(g + c)));
}

}  // namespace pcs

PCS_API int pcs_mlstm_gates(const void* h, int64_t h_stride, const void* w_i, const void* w_f, const float* b_i, const float* b_f,
                            float* ig, float* fg, int n_tokens, int width, int heads, float cap, int dtype, void* stream) {
  if (n_tokens == 0) return PCS_OK;
  PCS_REQUIRE(h && w_i && w_f && b_i && b_f && ig && fg && width > 0 && heads > 0 && cap > 0.f, "pcs_mlstm_gates: bad arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  PCS_DISPATCH(dtype, pcs::mlstm_gates_kernel<T><<<n_tokens, 256, 0, st>>>(static_cast<const T*>(h), h_stride, static_cast<const T*>(w_i),
                                                                           static_cast<const T*>(w_f), b_i, b_f, ig, fg, width, heads, cap));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_mlstm_scan(const pcs_mlstm_params* p, void* stream) {
  PCS_REQUIRE(p, "pcs_mlstm_scan: null params");
  if (p->n_seqs == 0 || p->n_tokens == 0) return PCS_OK;
  PCS_REQUIRE(p->proj && p->ig && p->fg && p->norm_w && p->out && p->s_pool && p->n_pool && p->m_pool && p->seq_slot && p->seq_pos0 &&
              p->seq_len && p->seq_off && p->o_raw, "pcs_mlstm_scan: null tensor");
  PCS_REQUIRE(p->heads > 0 && p->heads <= 65535 && p->dim > 0 && p->vdim > 0 && p->n_tokens > 0, "pcs_mlstm_scan: bad sizes");
  // slice width: at most 128 columns, and small enough that the slice of S fits shared memory
  int VS = p->vdim < 128 ? p->vdim : 128;
  while (VS > 8 && static_cast<size_t>(p->dim) * VS * sizeof(float) > 160 * 1024) VS /= 2;
  int R = 512 / VS;
  if (R < 1) R = 1;
  if (R > p->dim) R = p->dim;
  const int slices = (p->vdim + VS - 1) / VS;
  const int threads = ((VS * R + 31) / 32) * 32;
  const size_t smem = (static_cast<size_t>(p->dim) * VS + 3 * p->dim + VS + static_cast<size_t>(R) * VS) * sizeof(float);
  PCS_REQUIRE(smem <= 220 * 1024, "pcs_mlstm_scan: a state of %d rows exceeds shared memory", p->dim);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (smem > 48 * 1024) {
    PCS_DISPATCH(p->dtype, PCS_CHECK_CUDA(cudaFuncSetAttribute(pcs::mlstm_scan_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                              220 * 1024)));
  }
  dim3 grid(p->n_seqs, p->heads, slices);
  float* nm_new = p->o_raw + static_cast<long long>(p->n_tokens) * p->heads * p->vdim;  // behind the raw outputs
  PCS_DISPATCH(p->dtype, pcs::mlstm_scan_kernel<T><<<grid, threads, smem, st>>>(*p, p->o_raw, nm_new, VS, R));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::mlstm_commit_kernel<<<dim3(p->n_seqs, p->heads), 128, 0, st>>>(*p, nm_new);
  PCS_CHECK_CUDA(cudaGetLastError());
  dim3 grid2(p->n_tokens, p->heads);
  PCS_DISPATCH(p->dtype, pcs::mlstm_out_kernel<T><<<grid2, 256, 0, st>>>(*p, p->o_raw));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch(3);
  return PCS_OK;
}
