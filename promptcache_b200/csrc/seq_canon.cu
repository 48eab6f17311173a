// Embedding with a hashed token-pair table, and the residual sum + RMS norm + short causal convolution over time.
//
// pcs_embed_bigram  one block per token: the token's embedding row plus the row (prev * a + cur * b) mod buckets of a second
//                   table (its last row for a sequence's first token), summed in 32-bit into the residual stream.
// pcs_norm_conv     one block per token.  u = norm(x) is needed for the token and for its taps - 1 predecessors: rows of the
//                   same step are normed again from x (they are in L2; a row's statistics cost one reduction), rows of
//                   earlier steps come from the slot's tail, which exists twice so that the copy a step reads is never the
//                   one it writes.  The last taps - 1 tokens of an entry write their u into the other copy, the entry's last
//                   token also moves the rows that stay (steps shorter than taps - 1).  Everything is 32-bit; the result is
//                   rounded once, to the compute type, for the projection that follows.
#include "seq_common.cuh"

namespace pcs {

template <typename T>
__global__ void __launch_bounds__(256) embed_bigram_kernel(const T* __restrict__ table, const T* __restrict__ pair,
                                                           const int64_t* __restrict__ ids, const int64_t* __restrict__ prev_ids,
                                                           float* __restrict__ out, int width, int vocab, long long buckets,
                                                           long long mul_prev, long long mul_cur) {
  const int t = blockIdx.x;
  long long id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  const long long prev = prev_ids[t];
  long long r = buckets;
  if (prev >= 0) r = ((prev % buckets) * mul_prev + (id % buckets) * mul_cur) % buckets;  // the multipliers are reduced by the host
  const T* e = table + id * width;
  const T* b = pair + r * width;
  float* o = out + static_cast<long long>(t) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = ldf(e + i) + ldf(b + i);
}

constexpr int kMaxTaps = 16;

template <typename T>
__global__ void __launch_bounds__(256) norm_conv_kernel(const pcs_normconv_params p) {
  __shared__ float red[33];
  const int t = blockIdx.x, W = p.width, tid = threadIdx.x;
  float* x = p.x + static_cast<long long>(t) * W;
  const T* g = static_cast<const T*>(p.g);
  const float g1 = p.g_len == 1 ? ldf(g) : 0.f;
  float ss = 0.f;
  if (p.y) {
    const T* y = static_cast<const T*>(p.y) + static_cast<long long>(t) * p.y_stride;
    for (int i = tid; i < W; i += 256) {
      const float v = fmaf(p.y_mult, ldf(y + i), x[i]);
      x[i] = v;
      ss = fmaf(v, v, ss);
    }
    if (p.h_out == nullptr) return;
  } else {
    for (int i = tid; i < W; i += 256) ss = fmaf(x[i], x[i], ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / static_cast<float>(W) + p.eps);
  T* h = static_cast<T*>(p.h_out) + static_cast<long long>(t) * W;
  if (p.conv_w == nullptr) {
    for (int i = tid; i < W; i += 256) stf(h + i, x[i] * inv * (p.g_len == 1 ? g1 : ldf(g + i)));
    return;
  }
  const int R = p.taps - 1;
  const int b = p.tok_seq[t], pos = p.tok_pos[t], slot = p.seq_slot[b], pos0 = p.seq_pos0[b], len = p.seq_len[b], par = p.seq_par[b] & 1;
  const float* tail_r = p.tail + (static_cast<long long>(slot) * 2 + par) * R * W;        // rows: positions pos0 - R .. pos0 - 1
  float* tail_w = p.tail + (static_cast<long long>(slot) * 2 + (par ^ 1)) * R * W;        // rows: positions pos0 + len - R .. pos0 + len - 1
  // the predecessors' statistics: predecessor j (1 .. R) is the token at position pos - j
  float inv_prev[kMaxTaps];
#pragma unroll
  for (int j = 1; j < kMaxTaps; ++j) {
    inv_prev[j] = 0.f;
    if (j <= R && pos - j >= pos0) {  // uniform over the block
      const float* xp = x - static_cast<long long>(j) * W;
      float s = 0.f;
      for (int i = tid; i < W; i += 256) s = fmaf(xp[i], xp[i], s);
      s = block_sum(s, red);
      inv_prev[j] = 1.f / sqrtf(s / static_cast<float>(W) + p.eps);
    }
  }
  const T* cw = static_cast<const T*>(p.conv_w);
  const int last_row = pos - (pos0 + len - 1 - R) - 1;  // this token's row in the written tail, if >= 0
  for (int i = tid; i < W; i += 256) {
    const float gi = p.g_len == 1 ? g1 : ldf(g + i);
    const float u = x[i] * inv * gi;
    float acc = u * (1.f + ldf(cw + static_cast<long long>(R) * W + i));
#pragma unroll
    for (int j = 1; j < kMaxTaps; ++j) {
      if (j <= R && pos - j >= 0) {
        float uj;
        if (pos - j >= pos0) uj = x[i - static_cast<long long>(j) * W] * inv_prev[j] * gi;
        else uj = tail_r[static_cast<long long>(R - (pos0 - (pos - j))) * W + i];
        acc = fmaf(ldf(cw + static_cast<long long>(R - j) * W + i), uj, acc);
      }
    }
    stf(h + i, acc);
    if (last_row >= 0) tail_w[static_cast<long long>(last_row) * W + i] = u;
  }
  if (pos == pos0 + len - 1 && len < R) {  // rows that stay: new row r holds position pos0 + len - R + r = old row r + len
    for (int r = 0; r < R - len; ++r)
      for (int i = tid; i < W; i += 256) tail_w[static_cast<long long>(r) * W + i] = tail_r[static_cast<long long>(r + len) * W + i];
  }
}

// The same for rows of at most 256 * PPT 16-byte pieces (pointers, strides and the width multiples of a piece) and at most four
// taps: a thread keeps its pieces of the row and of the predecessors' rows in registers, every load is requested before the
// first reduction, and the rows' sums of squares meet in ONE reduction.
template <typename T, int PPT>
__global__ void __launch_bounds__(256) norm_conv_vec_kernel(const pcs_normconv_params p) {
  constexpr int N = Vec<T>::n, MR = 3;
  __shared__ float red[MR + 1][9];
  const int t = blockIdx.x, W = p.width, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* x = p.x + static_cast<long long>(t) * W;
  const T* g = static_cast<const T*>(p.g);
  const T* cw = static_cast<const T*>(p.conv_w);
  const int R = cw ? p.taps - 1 : 0;
  int pos = 0, pos0 = 0, len = 1, slot = 0, par = 0;
  if (cw) {
    const int b = p.tok_seq[t];
    pos = p.tok_pos[t]; slot = p.seq_slot[b]; pos0 = p.seq_pos0[b]; len = p.seq_len[b]; par = p.seq_par[b] & 1;
  }
  const float* tail_r = p.tail + (static_cast<long long>(slot) * 2 + par) * R * W;
  float* tail_w = p.tail + (static_cast<long long>(slot) * 2 + (par ^ 1)) * R * W;
  float xv[PPT][N], pv[MR][PPT][N], ss[MR + 1];
#pragma unroll
  for (int j = 0; j <= MR; ++j) ss[j] = 0.f;
#pragma unroll
  for (int u = 0; u < PPT; ++u) {
    const int i = (tid + u * 256) * N;
    if (i < W) {
      ldx(x + i, xv[u]);
      if (p.y) {
        float yv[N];
        ld16(static_cast<const T*>(p.y) + static_cast<long long>(t) * p.y_stride + i, yv);
#pragma unroll
        for (int e = 0; e < N; ++e) xv[u][e] = fmaf(p.y_mult, yv[e], xv[u][e]);
        stx(x + i, xv[u]);
      }
#pragma unroll
      for (int j = 1; j <= MR; ++j) {
        if (j <= R && pos - j >= 0) {
          if (pos - j >= pos0) ldx(x - static_cast<long long>(j) * W + i, pv[j - 1][u]);               // a row of this step: normed below
          else ldx(tail_r + static_cast<long long>(R - (pos0 - (pos - j))) * W + i, pv[j - 1][u]);     // an earlier step's: normed already
        } else {
#pragma unroll
          for (int e = 0; e < N; ++e) pv[j - 1][u][e] = 0.f;
        }
      }
#pragma unroll
      for (int e = 0; e < N; ++e) ss[0] = fmaf(xv[u][e], xv[u][e], ss[0]);
#pragma unroll
      for (int j = 1; j <= MR; ++j)
#pragma unroll
        for (int e = 0; e < N; ++e) ss[j] = fmaf(pv[j - 1][u][e], pv[j - 1][u][e], ss[j]);
    }
  }
  if (p.h_out == nullptr) return;
#pragma unroll
  for (int j = 0; j <= MR; ++j) {
    ss[j] = warp_sum(ss[j]);
    if (lane == 0) red[j][warp] = ss[j];
  }
  __syncthreads();
  float inv[MR + 1];
#pragma unroll
  for (int j = 0; j <= MR; ++j) {
    float a = 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q) a += red[j][q];
    inv[j] = 1.f / sqrtf(a / static_cast<float>(W) + p.eps);
    if (j > 0 && !(pos - j >= pos0)) inv[j] = 1.f;   // rows from the tail (or before the start: zeros) are not normed again
  }
  const float g1 = p.g_len == 1 ? ldf(g) : 0.f;
  const int last_row = pos - (pos0 + len - R);
  T* h = static_cast<T*>(p.h_out) + static_cast<long long>(t) * W;
#pragma unroll
  for (int u = 0; u < PPT; ++u) {
    const int i = (tid + u * 256) * N;
    if (i < W) {
      float gv[N], uv[N], o[N];
      if (p.g_len == 1) {
#pragma unroll
        for (int e = 0; e < N; ++e) gv[e] = g1;
      } else {
        ld16(g + i, gv);
      }
#pragma unroll
      for (int e = 0; e < N; ++e) { uv[e] = xv[u][e] * inv[0] * gv[e]; o[e] = uv[e]; }
      if (cw) {
        float wv[N];
        ld16(cw + static_cast<long long>(R) * W + i, wv);
#pragma unroll
        for (int e = 0; e < N; ++e) o[e] = uv[e] * (1.f + wv[e]);
#pragma unroll
        for (int j = 1; j <= MR; ++j)
          if (j <= R) {
            ld16(cw + static_cast<long long>(R - j) * W + i, wv);
            const bool here = pos - j >= pos0;
#pragma unroll
            for (int e = 0; e < N; ++e) o[e] = fmaf(wv[e], pv[j - 1][u][e] * inv[j] * (here ? gv[e] : 1.f), o[e]);
          }
        if (last_row >= 0) stx(tail_w + static_cast<long long>(last_row) * W + i, uv);
      }
      st16(h + i, o);
    }
  }
  if (cw && pos == pos0 + len - 1 && len < R) {
    for (int r = 0; r < R - len; ++r)
      for (int i = tid; i < W; i += 256) tail_w[static_cast<long long>(r) * W + i] = tail_r[static_cast<long long>(r + len) * W + i];
  }
}

}  // namespace pcs

PCS_API int pcs_embed_bigram(const void* table, const void* pair, const int64_t* ids, const int64_t* prev_ids, float* out, int n_tokens,
                             int width, int vocab, int64_t buckets, int64_t mul_prev, int64_t mul_cur, int dtype, void* stream) {
  if (n_tokens == 0) return PCS_OK;
  PCS_REQUIRE(table && pair && ids && prev_ids && out && n_tokens > 0 && width > 0 && vocab > 0, "pcs_embed_bigram: bad arguments");
  PCS_REQUIRE(buckets > 0 && buckets < (1LL << 31), "pcs_embed_bigram: buckets %lld out of range", static_cast<long long>(buckets));
  // reduced multipliers keep every product below 2^62
  const long long mp = ((mul_prev % buckets) + buckets) % buckets, mc = ((mul_cur % buckets) + buckets) % buckets;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  PCS_DISPATCH(dtype, pcs::embed_bigram_kernel<T><<<n_tokens, 256, 0, st>>>(static_cast<const T*>(table), static_cast<const T*>(pair), ids, prev_ids,
                                                                            out, width, vocab, buckets, mp, mc));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_norm_conv(const pcs_normconv_params* p, void* stream) {
  PCS_REQUIRE(p, "pcs_norm_conv: null params");
  if (p->n_tokens == 0) return PCS_OK;
  PCS_REQUIRE(p->x && p->n_tokens > 0 && p->width > 0, "pcs_norm_conv: bad arguments");
  PCS_REQUIRE(p->h_out == nullptr || (p->g && (p->g_len == 1 || p->g_len == p->width)), "pcs_norm_conv: the norm weight is one number or one per channel");
  PCS_REQUIRE(p->h_out != nullptr || p->y != nullptr, "pcs_norm_conv: nothing to do");
  if (p->conv_w) {
    PCS_REQUIRE(p->y == nullptr, "pcs_norm_conv: the residual sum and the convolution cannot share a launch");
    PCS_REQUIRE(p->h_out, "pcs_norm_conv: the convolution needs h_out");
    PCS_REQUIRE(p->taps >= 1 && p->taps <= pcs::kMaxTaps, "pcs_norm_conv: taps %d outside 1..%d", p->taps, pcs::kMaxTaps);
    PCS_REQUIRE((p->tail || p->taps == 1) && p->tok_seq && p->tok_pos && p->seq_slot && p->seq_pos0 && p->seq_len && p->seq_par,
                "pcs_norm_conv: the convolution needs the tail and the batch description");
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int piece = p->dtype == PCS_BF16 ? 8 : 4;
  const long long esz = p->dtype == PCS_BF16 ? 2 : 4;
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  const bool vec = p->width % piece == 0 && p->width <= 512 * piece && al(p->x) && al(p->h_out) && al(p->tail) &&
                   (p->y == nullptr || (al(p->y) && (p->y_stride * esz) % 16 == 0)) && (p->g_len == 1 || al(p->g)) && al(p->conv_w) &&
                   (p->conv_w == nullptr || p->taps <= 4);
  if (vec) {
    if (p->width <= 256 * piece) PCS_DISPATCH(p->dtype, pcs::norm_conv_vec_kernel<T, 1><<<p->n_tokens, 256, 0, st>>>(*p));
    else PCS_DISPATCH(p->dtype, pcs::norm_conv_vec_kernel<T, 2><<<p->n_tokens, 256, 0, st>>>(*p));
    PCS_CHECK_CUDA(cudaGetLastError());
    pcs::count_launch();
    return PCS_OK;
  }
  PCS_DISPATCH(p->dtype, pcs::norm_conv_kernel<T><<<p->n_tokens, 256, 0, st>>>(*p));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}
