// Chunkwise form of the stabilised matrix-memory recurrence for prompts (bfloat16 projections, tensor cores).
//
// The token-by-token recurrence
//     m_t = max(f_t + m_{t-1}, i_t),   S_t = e^{f_t + m_{t-1} - m_t} S_{t-1} + e^{i_t - m_t} k_t v_t^T,   n_t likewise
// is linear in (S, n), so 64 tokens can be taken at once.  With b_t the running sum of f inside the chunk, a_s = i_s - b_s
// and g_t = max(m_in, max_{s<=t} a_s) (m_in: the stabiliser the chunk starts from), m_t = b_t + g_t and
//     S_t^T q_t = e^{m_in - g_t} (S_in^T q_t) + sum_{s<=t} e^{a_s - g_t} (q_t . k_s) v_s          (every exponent <= 0)
// and the state after the chunk's last token e is S_e = e^{m_in - g_e} S_in + sum_s e^{a_s - g_e} k_s v_s^T.
// The normaliser n rides along as ONE MORE VALUE COLUMN whose v is 1: the same products give n_t . q_t and the new n.
//
// One block = (sequence, head, 32 or 16 value columns), 4 warps, the chunks of the entry one after the other.  Products are
// m16n8k16 bfloat16 tensor-core operations with 32-bit accumulators; q, k, v are bfloat16 already (exact operands), every
// 32-bit factor (the weights e^{a_s - g_t} (q.k), the state, the weighted values) enters as TWO bfloat16 operands hi + lo.
// The state itself stays 32-bit in shared memory between chunks and in the pool between steps; gates, sums of gates, maxima
// and exponentials are 32-bit.  A warp owns 16 of the chunk's 64 tokens for the outputs and a quarter of the state's rows
// for the update.
#include "seq_common.cuh"
#include "seq_mma.cuh"

namespace pcs {

namespace {

constexpr int CL = 64;         // tokens per chunk
constexpr int CTHREADS = 128;
// CVS value columns per block (32, or 16 when 32 would leave most SMs without a block).  The widened tiles have
// CNC = CVS + 16 columns: the values, the normaliser's column, zero padding (an even number of groups of 8), in rows of
// CROW = CNC + 8 bfloat16 elements (112 or 80 bytes: ldmatrix without bank conflicts).

__device__ __forceinline__ void split1(float x, __nv_bfloat16& hi, __nv_bfloat16& lo) {
  hi = __float2bfloat16_rn(x);
  lo = __float2bfloat16_rn(x - __bfloat162float(hi));
}

}  // namespace

template <int CVS>
__global__ void __launch_bounds__(CTHREADS) mlstm_chunk_kernel(const pcs_mlstm_params p, float* __restrict__ o_raw,
                                                               float* __restrict__ nm_new) {
  constexpr int CNC = CVS + 16, CROW = CNC + 8, CNT = CNC / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D = p.dim, V = p.vdim, H = p.heads;
  const int QROW = D + 8;  // bfloat16 elements per row of the q and k tiles
  float* Sf = reinterpret_cast<float*>(smem_raw);              // [D][CNC]   the state (and n in column CVS), 32-bit
  __nv_bfloat16* Sh = reinterpret_cast<__nv_bfloat16*>(Sf + D * CNC);  // [D][CROW]  its hi and lo parts as operands
  __nv_bfloat16* Sl = Sh + D * CROW;
  __nv_bfloat16* Qs = Sl + D * CROW;                           // [CL][QROW]
  __nv_bfloat16* Ks = Qs + CL * QROW;
  __nv_bfloat16* Vs = Ks + CL * QROW;                          // [CL][CROW] values, a column of ones, zeros
  __nv_bfloat16* Vh = Vs + CL * CROW;                          // the values times e^{a_s - g_e}, hi and lo
  __nv_bfloat16* Vl = Vh + CL * CROW;
  float* f_s = reinterpret_cast<float*>(Vl + CL * CROW);       // per token of the chunk: f, i, a, g, e^{m_in - g}, e^{-m}, e^{a - g_e}
  float* i_s = f_s + CL;
  float* a_s = i_s + CL;
  float* g_s = a_s + CL;
  float* c_s = g_s + CL;
  float* em_s = c_s + CL;
  float* we_s = em_s + CL;
  float* fin = we_s + CL;  // [0] = m after the chunk, [1] = e^{m_in - g_e}

  const int b = blockIdx.x, head = blockIdx.y, v0 = blockIdx.z * CVS;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, grp = lane >> 2, qd = lane & 3;
  const int slot = p.seq_slot[b], pos0 = p.seq_pos0[b], len = p.seq_len[b], off = p.seq_off[b];
  if (len <= 0) return;
  const int vs = min(CVS, V - v0);
  float* Sg = p.s_pool + (static_cast<long long>(slot) * H + head) * D * V;
  const float* ng = p.n_pool + (static_cast<long long>(slot) * H + head) * D;
  const bool fresh = pos0 == 0;
  for (int e = tid; e < D * CNC; e += CTHREADS) {
    const int d = e / CNC, c = e - d * CNC;
    float x = 0.f;
    if (!fresh) {
      if (c < vs) x = Sg[static_cast<long long>(d) * V + v0 + c];
      else if (c == CVS) x = ng[d];
    }
    Sf[e] = x;
    split1(x, Sh[d * CROW + c], Sl[d * CROW + c]);
  }
  float m_in = fresh ? 0.f : p.m_pool[static_cast<long long>(slot) * H + head];
  const __nv_bfloat16* proj = static_cast<const __nv_bfloat16*>(p.proj);
  const int row_a = warp * 16 + grp, row_b = row_a + 8;
  const uint32_t q_base = static_cast<uint32_t>(__cvta_generic_to_shared(Qs)) + ((warp * 16 + (lane & 15)) * QROW + (lane >> 4) * 8) * 2;
  // [k][n] tiles read as the second operand (transposed fragments): rows lane & 15, 8 columns further for the upper lanes
  const int bt_off = ((lane & 15) * CROW + (lane >> 4) * 8) * 2;
  const uint32_t sh_base = static_cast<uint32_t>(__cvta_generic_to_shared(Sh)) + bt_off;
  const uint32_t sl_base = static_cast<uint32_t>(__cvta_generic_to_shared(Sl)) + bt_off;
  const uint32_t vs_base = static_cast<uint32_t>(__cvta_generic_to_shared(Vs)) + bt_off;
  const uint32_t vh_base = static_cast<uint32_t>(__cvta_generic_to_shared(Vh)) + bt_off;
  const uint32_t vl_base = static_cast<uint32_t>(__cvta_generic_to_shared(Vl)) + bt_off;
  // k tile [token][d] in 8x8 pieces: tokens (lane & 7), + 8 for lanes 16..31; dims 8 further for lanes 8..15 and 24..31.  Read
  // plainly it is the second operand of q k^T (two groups of 8 tokens x 16 dims), read transposed the first operand of
  // k^T (v w) (16 state rows x 16 tokens)
  const uint32_t kt_base = static_cast<uint32_t>(__cvta_generic_to_shared(Ks)) + (((lane & 7) + ((lane >> 4) & 1) * 8) * QROW + ((lane >> 3) & 1) * 8) * 2;
  const int pieces = D / 8;

  for (int i0 = 0; i0 < len; i0 += CL) {
    const int nvalid = min(CL, len - i0);
    // ---- the chunk's q, k, v rows and gates into shared memory: every 16-byte piece is an asynchronous copy, so the whole
    //      tile is in flight at once; the next chunk's rows are asked into L2 meanwhile ----
    for (int e = tid; e < CL * pieces; e += CTHREADS) {
      const int r = e / pieces, c = (e - r * pieces) * 8;
      if (r < nvalid) {
        const __nv_bfloat16* row = proj + static_cast<long long>(off + i0 + r) * p.row_stride;
        cp_async16(Qs + r * QROW + c, row + p.q_off + head * D + c);
        cp_async16(Ks + r * QROW + c, row + p.k_off + head * D + c);
      } else {
        *reinterpret_cast<uint4*>(Qs + r * QROW + c) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(Ks + r * QROW + c) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    for (int e = tid; e < CL * CNT; e += CTHREADS) {
      const int r = e / CNT, c = (e - r * CNT) * 8;
      if (r < nvalid && c < CVS && v0 + c < V) {
        cp_async16(Vs + r * CROW + c, proj + static_cast<long long>(off + i0 + r) * p.row_stride + p.v_off + head * V + v0 + c);
      } else {
        uint4 vv = make_uint4(0u, 0u, 0u, 0u);
        if (r < nvalid && c == CVS) vv.x = 0x00003f80u;  // bfloat16 1.0 in column CVS
        *reinterpret_cast<uint4*>(Vs + r * CROW + c) = vv;
      }
    }
    cp_async_commit();
    if (i0 + CL < len) {  // one 128-byte line per request: q and k rows of the next chunk, and its value slice
      const int nxt = min(CL, len - i0 - CL), lines = (D * 2 + 127) / 128;
      for (int e = tid; e < nxt * lines; e += CTHREADS) {
        const int r = e / lines, c = (e - r * lines) * 64;
        const __nv_bfloat16* row = proj + static_cast<long long>(off + i0 + CL + r) * p.row_stride;
        prefetch_l2(row + p.q_off + head * D + c);
        prefetch_l2(row + p.k_off + head * D + c);
        if (c == 0) prefetch_l2(row + p.v_off + head * V + v0);
      }
    }
    if (tid < CL) {
      const bool ok = tid < nvalid;
      const long long t = static_cast<long long>(off + i0 + tid) * H + head;
      f_s[tid] = ok ? p.fg[t] : 0.f;
      i_s[tid] = ok ? p.ig[t] : -INFINITY;
    }
    cp_async_wait<0>();
    __syncthreads();
    // ---- warp 0: sums of f, running maxima and the per-token factors (two tokens per lane) ----
    if (warp == 0) {
      const float f0 = f_s[2 * lane], f1 = f_s[2 * lane + 1];
      float x = f0 + f1;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
      }
      const float b1 = x, b0 = x - f1;
      const float a0 = i_s[2 * lane] - b0, a1 = i_s[2 * lane + 1] - b1;
      float cm = fmaxf(a0, a1);
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float y = __shfl_up_sync(0xffffffffu, cm, o);
        if (lane >= o) cm = fmaxf(cm, y);
      }
      float before = __shfl_up_sync(0xffffffffu, cm, 1);
      if (lane == 0) before = -INFINITY;
      const float g0 = fmaxf(fmaxf(m_in, before), a0), g1 = fmaxf(g0, a1);
      const int e = nvalid - 1;
      const float ge = __shfl_sync(0xffffffffu, (e & 1) ? g1 : g0, e >> 1);
      const float be = __shfl_sync(0xffffffffu, (e & 1) ? b1 : b0, e >> 1);
      a_s[2 * lane] = a0; a_s[2 * lane + 1] = a1;
      g_s[2 * lane] = g0; g_s[2 * lane + 1] = g1;
      c_s[2 * lane] = expf(m_in - g0); c_s[2 * lane + 1] = expf(m_in - g1);
      em_s[2 * lane] = expf(-(b0 + g0)); em_s[2 * lane + 1] = expf(-(b1 + g1));
      we_s[2 * lane] = expf(a0 - ge); we_s[2 * lane + 1] = expf(a1 - ge);  // tokens past the entry's end: a = -inf, weight 0
      if (lane == 0) { fin[0] = be + ge; fin[1] = expf(m_in - ge); }
    }
    // ---- scores q . k: 16 tokens x 64 tokens per warp ----
    float s[CL / 8][4];
#pragma unroll
    for (int i = 0; i < CL / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a0, a1, a2, a3;
      ldsm_x4(q_base + kk * 32, a0, a1, a2, a3);
#pragma unroll
      for (int nt = 0; nt < CL / 8; nt += 2) {
        uint32_t k0, k1, k2, k3;  // tokens nt*8.. (k0: dims kk*16.., k1: +8), tokens (nt+1)*8.. (k2, k3)
        ldsm_x4(kt_base + (nt * 8 * QROW + kk * 16) * 2, k0, k1, k2, k3);
        mma_bf16(s[nt], a0, a1, a2, a3, k0, k1);
        mma_bf16(s[nt + 1], a0, a1, a2, a3, k2, k3);
      }
    }
    __syncthreads();  // the factors are there
    // ---- the weighted values (v | 1) e^{a_s - g_e}, hi and lo, for the state update ----
    for (int e = tid; e < CL * (CNC / 2); e += CTHREADS) {
      const int r = e / (CNC / 2), c = (e - r * (CNC / 2)) * 2;
      const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(Vs + r * CROW + c));
      const float w = we_s[r];
      uint32_t lo;
      const uint32_t hi = split_pair(v.x * w, v.y * w, lo);
      *reinterpret_cast<uint32_t*>(Vh + r * CROW + c) = hi;
      *reinterpret_cast<uint32_t*>(Vl + r * CROW + c) = lo;
    }
    // ---- weights e^{a_s - g_t} (q_t . k_s) / sqrt(dim), s <= t ----
    {
      const float ga = g_s[row_a], gb = g_s[row_b];
#pragma unroll
      for (int nt = 0; nt < CL / 8; ++nt) {
        const int col = nt * 8 + qd * 2;
        const float2 av = *reinterpret_cast<const float2*>(a_s + col);
        s[nt][0] = col <= row_a ? s[nt][0] * p.q_scale * __expf(av.x - ga) : 0.f;
        s[nt][1] = col + 1 <= row_a ? s[nt][1] * p.q_scale * __expf(av.y - ga) : 0.f;
        s[nt][2] = col <= row_b ? s[nt][2] * p.q_scale * __expf(av.x - gb) : 0.f;
        s[nt][3] = col + 1 <= row_b ? s[nt][3] * p.q_scale * __expf(av.y - gb) : 0.f;
      }
    }
    // ---- (q S_in | q . n_in), scaled by e^{m_in - g_t} / sqrt(dim) ----
    float acc[CNT][4];
#pragma unroll
    for (int i = 0; i < CNT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a0, a1, a2, a3;
      ldsm_x4(q_base + kk * 32, a0, a1, a2, a3);
      // all hi products, then all lo products: CNT independent accumulators between two products into the same one
      uint32_t hf[CNT / 2][4], lf[CNT / 2][4];
#pragma unroll
      for (int u = 0; u < CNT / 2; ++u) {
        ldsm_x4_t(sh_base + (kk * 16 * CROW + u * 16) * 2, hf[u][0], hf[u][1], hf[u][2], hf[u][3]);
        ldsm_x4_t(sl_base + (kk * 16 * CROW + u * 16) * 2, lf[u][0], lf[u][1], lf[u][2], lf[u][3]);
      }
#pragma unroll
      for (int u = 0; u < CNT / 2; ++u) {
        mma_bf16(acc[2 * u], a0, a1, a2, a3, hf[u][0], hf[u][1]);
        mma_bf16(acc[2 * u + 1], a0, a1, a2, a3, hf[u][2], hf[u][3]);
      }
#pragma unroll
      for (int u = 0; u < CNT / 2; ++u) {
        mma_bf16(acc[2 * u], a0, a1, a2, a3, lf[u][0], lf[u][1]);
        mma_bf16(acc[2 * u + 1], a0, a1, a2, a3, lf[u][2], lf[u][3]);
      }
    }
    {
      const float ca = c_s[row_a] * p.q_scale, cb = c_s[row_b] * p.q_scale;
#pragma unroll
      for (int i = 0; i < CNT; ++i) { acc[i][0] *= ca; acc[i][1] *= ca; acc[i][2] *= cb; acc[i][3] *= cb; }
    }
    // ---- + weights x (v | 1) ----
#pragma unroll
    for (int j = 0; j < CL / 16; ++j) {
      uint32_t lo0, lo1, lo2, lo3;
      const uint32_t hi0 = split_pair(s[2 * j][0], s[2 * j][1], lo0);
      const uint32_t hi1 = split_pair(s[2 * j][2], s[2 * j][3], lo1);
      const uint32_t hi2 = split_pair(s[2 * j + 1][0], s[2 * j + 1][1], lo2);
      const uint32_t hi3 = split_pair(s[2 * j + 1][2], s[2 * j + 1][3], lo3);
      uint32_t vf[CNT / 2][4];
#pragma unroll
      for (int u = 0; u < CNT / 2; ++u) ldsm_x4_t(vs_base + (j * 16 * CROW + u * 16) * 2, vf[u][0], vf[u][1], vf[u][2], vf[u][3]);
#pragma unroll
      for (int u = 0; u < CNT / 2; ++u) {
        mma_bf16(acc[2 * u], hi0, hi1, hi2, hi3, vf[u][0], vf[u][1]);
        mma_bf16(acc[2 * u + 1], hi0, hi1, hi2, hi3, vf[u][2], vf[u][3]);
      }
#pragma unroll
      for (int u = 0; u < CNT / 2; ++u) {
        mma_bf16(acc[2 * u], lo0, lo1, lo2, lo3, vf[u][0], vf[u][1]);
        mma_bf16(acc[2 * u + 1], lo0, lo1, lo2, lo3, vf[u][2], vf[u][3]);
      }
    }
    // ---- o_t = numerator / (max(|n_t . q_t|, e^{-m_t}) + 1e-6); the denominator's product sits in column CVS ----
    {
      const float nq_a = __shfl_sync(0xffffffffu, acc[CVS / 8][0], lane & ~3), nq_b = __shfl_sync(0xffffffffu, acc[CVS / 8][2], lane & ~3);
      const float inv_a = 1.f / (fmaxf(fabsf(nq_a), em_s[row_a]) + 1e-6f), inv_b = 1.f / (fmaxf(fabsf(nq_b), em_s[row_b]) + 1e-6f);
      float* oa = o_raw + static_cast<long long>(off + i0 + row_a) * H * V + head * V + v0;
      float* ob = o_raw + static_cast<long long>(off + i0 + row_b) * H * V + head * V + v0;
#pragma unroll
      for (int vn = 0; vn < CVS / 8; ++vn) {
        const int c = vn * 8 + qd * 2;
        if (c < vs) {  // vdim is a multiple of 8: both columns of the pair exist
          if (row_a < nvalid) *reinterpret_cast<float2*>(oa + c) = make_float2(acc[vn][0] * inv_a, acc[vn][1] * inv_a);
          if (row_b < nvalid) *reinterpret_cast<float2*>(ob + c) = make_float2(acc[vn][2] * inv_b, acc[vn][3] * inv_b);
        }
      }
    }
    const float m_out = fin[0], c_e = fin[1];
    __syncthreads();  // the weighted values are complete, and every warp has read the old state's operands
    // ---- state: S <- e^{m_in - g_e} S + k^T ((v | 1) w); a warp owns every fourth group of 16 rows ----
    for (int mt = warp; mt < D / 16; mt += 4) {
      const int d_a = mt * 16 + grp, d_b = d_a + 8;
      float st[CNT][4];
#pragma unroll
      for (int vn = 0; vn < CNT; ++vn) {
        const float2 xa = *reinterpret_cast<const float2*>(Sf + d_a * CNC + vn * 8 + qd * 2);
        const float2 xb = *reinterpret_cast<const float2*>(Sf + d_b * CNC + vn * 8 + qd * 2);
        st[vn][0] = xa.x * c_e; st[vn][1] = xa.y * c_e; st[vn][2] = xb.x * c_e; st[vn][3] = xb.y * c_e;
      }
#pragma unroll
      for (int ks = 0; ks < CL / 16; ++ks) {
        uint32_t a0, a1, a2, a3;
        ldsm_x4_t(kt_base + (ks * 16 * QROW + mt * 16) * 2, a0, a1, a2, a3);
        uint32_t hf[CNT / 2][4], lf[CNT / 2][4];
#pragma unroll
        for (int u = 0; u < CNT / 2; ++u) {
          ldsm_x4_t(vh_base + (ks * 16 * CROW + u * 16) * 2, hf[u][0], hf[u][1], hf[u][2], hf[u][3]);
          ldsm_x4_t(vl_base + (ks * 16 * CROW + u * 16) * 2, lf[u][0], lf[u][1], lf[u][2], lf[u][3]);
        }
#pragma unroll
        for (int u = 0; u < CNT / 2; ++u) {
          mma_bf16(st[2 * u], a0, a1, a2, a3, hf[u][0], hf[u][1]);
          mma_bf16(st[2 * u + 1], a0, a1, a2, a3, hf[u][2], hf[u][3]);
        }
#pragma unroll
        for (int u = 0; u < CNT / 2; ++u) {
          mma_bf16(st[2 * u], a0, a1, a2, a3, lf[u][0], lf[u][1]);
          mma_bf16(st[2 * u + 1], a0, a1, a2, a3, lf[u][2], lf[u][3]);
        }
      }
#pragma unroll
      for (int vn = 0; vn < CNT; ++vn) {
        const int c = vn * 8 + qd * 2;
        *reinterpret_cast<float2*>(Sf + d_a * CNC + c) = make_float2(st[vn][0], st[vn][1]);
        *reinterpret_cast<float2*>(Sf + d_b * CNC + c) = make_float2(st[vn][2], st[vn][3]);
        uint32_t lo;
        uint32_t hi = split_pair(st[vn][0], st[vn][1], lo);
        *reinterpret_cast<uint32_t*>(Sh + d_a * CROW + c) = hi;
        *reinterpret_cast<uint32_t*>(Sl + d_a * CROW + c) = lo;
        hi = split_pair(st[vn][2], st[vn][3], lo);
        *reinterpret_cast<uint32_t*>(Sh + d_b * CROW + c) = hi;
        *reinterpret_cast<uint32_t*>(Sl + d_b * CROW + c) = lo;
      }
    }
    m_in = m_out;
    __syncthreads();  // the new state is complete before the next chunk reads it; the tiles may be overwritten
  }
  // ---- the state back into the pool; the slice of the first columns hands n and m to the commit ----
  for (int e = tid; e < D * vs; e += CTHREADS) {
    const int d = e / vs, c = e - d * vs;
    Sg[static_cast<long long>(d) * V + v0 + c] = Sf[d * CNC + c];
  }
  if (blockIdx.z == 0) {
    float* dst = nm_new + (static_cast<long long>(b) * H + head) * (D + 1);
    for (int d = tid; d < D; d += CTHREADS) dst[d] = Sf[d * CNC + CVS];
    if (tid == 0) dst[D] = m_in;
  }
}

size_t mlstm_chunk_smem(int dim, int cvs) {
  const size_t cnc = cvs + 16, crow = cnc + 8;
  return static_cast<size_t>(dim) * cnc * sizeof(float) + (2 * static_cast<size_t>(dim) * crow + 2 * static_cast<size_t>(CL) * (dim + 8) +
                                                             3 * static_cast<size_t>(CL) * crow) * sizeof(__nv_bfloat16) +
         (7 * CL + 4) * sizeof(float);
}

int launch_mlstm_chunk(const pcs_mlstm_params& p, float* nm_new, cudaStream_t st) {
  static bool configured = false;
  if (!configured) {
    PCS_CHECK_CUDA(cudaFuncSetAttribute(mlstm_chunk_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    PCS_CHECK_CUDA(cudaFuncSetAttribute(mlstm_chunk_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    configured = true;
  }
  // 32 columns per block unless that leaves the GPU mostly empty (one long prompt): narrower slices recompute the q . k
  // scores in more blocks but halve everything else a block does per chunk
  const long long blocks32 = static_cast<long long>(p.n_seqs) * p.heads * ((p.vdim + 31) / 32);
  if (blocks32 >= 148 || p.vdim <= 16) {
    dim3 grid(p.n_seqs, p.heads, (p.vdim + 31) / 32);
    mlstm_chunk_kernel<32><<<grid, CTHREADS, mlstm_chunk_smem(p.dim, 32), st>>>(p, p.o_raw, nm_new);
  } else {
    dim3 grid(p.n_seqs, p.heads, (p.vdim + 15) / 16);
    mlstm_chunk_kernel<16><<<grid, CTHREADS, mlstm_chunk_smem(p.dim, 16), st>>>(p, p.o_raw, nm_new);
  }
  PCS_CHECK_CUDA(cudaGetLastError());
  return PCS_OK;
}

}  // namespace pcs
