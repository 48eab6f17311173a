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
// pcs_mlstm_scan   the token-by-token kernel: one block per (sequence, head), S in shared memory, thread (r, c) owns the
//                  rows r, r + R, ... of column c.
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

// blockDim.x = round_up(vdim * R, 32); threads >= vdim * R only take part in loads and reductions.
template <typename T>
__global__ void __launch_bounds__(1024) mlstm_scan_kernel(const pcs_mlstm_params p, int R) {
  extern __shared__ float sm[];
  __shared__ float red[33];
  const int D = p.dim, V = p.vdim, H = p.heads;
  float* S = sm;                 // [D][V]
  float* nvec = S + D * V;       // [D]
  float* ks = nvec + D;          // [D]
  float* qs = ks + D;            // [D]
  float* vs = qs + D;            // [V]
  float* part = vs + V;          // [R][V]
  const int b = blockIdx.x, head = blockIdx.y, tid = threadIdx.x, nthr = blockDim.x;
  const int slot = p.seq_slot[b], pos0 = p.seq_pos0[b], len = p.seq_len[b], off = p.seq_off[b];
  if (len <= 0) return;
  float* Sg = p.s_pool + (static_cast<long long>(slot) * H + head) * D * V;
  float* ng = p.n_pool + (static_cast<long long>(slot) * H + head) * D;
  float* mg = p.m_pool + static_cast<long long>(slot) * H + head;
  const bool fresh = pos0 == 0;
  for (int e = tid; e < D * V; e += nthr) S[e] = fresh ? 0.f : Sg[e];
  for (int d = tid; d < D; d += nthr) nvec[d] = fresh ? 0.f : ng[d];
  float m = fresh ? 0.f : *mg;
  const int c = tid % V, r = tid / V;
  const bool active = r < R;
  const T* nw = static_cast<const T*>(p.norm_w) + head * V;
  __syncthreads();
  for (int i = 0; i < len; ++i) {
    const long long t = off + i;
    const T* row = static_cast<const T*>(p.proj) + t * p.row_stride;
    for (int d = tid; d < D; d += nthr) {
      ks[d] = ldf(row + p.k_off + head * D + d);
      qs[d] = ldf(row + p.q_off + head * D + d) * p.q_scale;
    }
    for (int e = tid; e < V; e += nthr) vs[e] = ldf(row + p.v_off + head * V + e);
    const float ig = p.ig[t * H + head], fg = p.fg[t * H + head];
    const float m_new = fmaxf(fg + m, ig);
    const float a = expf(fg + m - m_new), bb = expf(ig - m_new);
    m = m_new;
    __syncthreads();
    // state update and the partial numerators
    float nq = 0.f;
    for (int d = tid; d < D; d += nthr) {
      const float nn = fmaf(a, nvec[d], bb * ks[d]);
      nvec[d] = nn;
      nq = fmaf(nn, qs[d], nq);
    }
    if (active) {
      const float bv = bb * vs[c];
      float num = 0.f;
      for (int d = r; d < D; d += R) {
        const float s = fmaf(a, S[d * V + c], ks[d] * bv);
        S[d * V + c] = s;
        num = fmaf(s, qs[d], num);
      }
      part[r * V + c] = num;
    }
    nq = block_sum(nq, red);  // its barriers also publish `part`
    const float den = fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
    float o = 0.f;
    if (tid < V) {
      for (int rr = 0; rr < R; ++rr) o += part[rr * V + tid];
      o /= den;
    }
    // a head wider than the block would need a loop here; the launcher keeps vdim <= blockDim.x
    const float ss = block_sum(tid < V ? o * o : 0.f, red);
    if (tid < V) {
      const float inv = 1.f / sqrtf(ss / static_cast<float>(V) + p.eps);
      const float gate = sigmoidf_(ldf(row + p.g_off + head * V + tid));
      stf(static_cast<T*>(p.out) + t * (static_cast<long long>(H) * V) + head * V + tid, o * inv * ldf(nw + tid) * gate);
    }
    __syncthreads();  // ks / qs / vs / part are rewritten by the next token
  }
  for (int e = tid; e < D * V; e += nthr) Sg[e] = S[e];
  for (int d = tid; d < D; d += nthr) ng[d] = nvec[d];
  if (tid == 0) *mg = m;
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
  if (p->n_seqs == 0) return PCS_OK;
  PCS_REQUIRE(p->proj && p->ig && p->fg && p->norm_w && p->out && p->s_pool && p->n_pool && p->m_pool && p->seq_slot && p->seq_pos0 &&
              p->seq_len && p->seq_off, "pcs_mlstm_scan: null tensor");
  PCS_REQUIRE(p->heads > 0 && p->heads <= 65535 && p->dim > 0 && p->vdim > 0, "pcs_mlstm_scan: bad sizes");
  PCS_REQUIRE(p->vdim <= 1024, "pcs_mlstm_scan: vdim %d exceeds one block", p->vdim);
  int R = 512 / p->vdim;
  if (R < 1) R = 1;
  if (R > p->dim) R = p->dim;
  const int threads = ((p->vdim * R + 31) / 32) * 32;
  const size_t smem = (static_cast<size_t>(p->dim) * p->vdim + 3 * p->dim + p->vdim + static_cast<size_t>(R) * p->vdim) * sizeof(float);
  PCS_REQUIRE(smem <= 220 * 1024, "pcs_mlstm_scan: a %d x %d state exceeds shared memory", p->dim, p->vdim);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (smem > 48 * 1024) {
    PCS_DISPATCH(p->dtype, PCS_CHECK_CUDA(cudaFuncSetAttribute(pcs::mlstm_scan_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                              220 * 1024)));
  }
  dim3 grid(p->n_seqs, p->heads);
  PCS_DISPATCH(p->dtype, pcs::mlstm_scan_kernel<T><<<grid, threads, smem, st>>>(*p, R));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}
