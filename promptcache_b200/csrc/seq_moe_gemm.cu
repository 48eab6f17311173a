// Mixture of experts for many rows (prompts, bfloat16): rows sorted by expert, then two grouped tensor-core products.
//
// pcs_moe_plan   one block: counts the (token, choice) pairs of every expert, lays the experts' rows out one after the other,
//                cuts them into tiles of 64 rows that never straddle two experts, and writes the sorted pair list.  Pairs
//                whose choice is a pass-through output take no row.  Everything stays on the device: the products below
//                are launched for the largest possible number of tiles and blocks past the real number return at once.
// pcs_moe_gemm   block = (row tile, 64 output features), 4 warps of 32 x 32, K in steps of 32 through two cp.async stages,
//                ldmatrix + m16n8k16 bfloat16 products with 32-bit accumulators.
//                  stage 0: rows gathered from h by pair; gate and up features of the tile's expert side by side, the
//                           epilogue writes silu(gate) * up in the sorted order (bfloat16);
//                  stage 1: rows of that matrix times the expert's down matrix, written 32-bit to the PAIR's row, so the
//                           weighted sum afterwards runs in the order of the choices whatever the sort did.
//                A row's sums depend on K alone, not on where the sort placed it or on what else is in the batch.
#include "seq_common.cuh"
#include "seq_mma.cuh"

namespace pcs {

namespace {

constexpr int GM = 64, GN = 64, GK = 32, GPAD = 8, G_THREADS = 128;
constexpr int kPlanMaxExperts = 1024;

__host__ __device__ inline int plan_max_tiles(int n_pairs, int n_experts) { return (n_pairs + GM - 1) / GM + n_experts; }

__global__ void __launch_bounds__(1024) moe_plan_kernel(const int32_t* __restrict__ idx, int n_pairs, int E, int32_t* __restrict__ plan) {
  __shared__ int cnt[kPlanMaxExperts];
  __shared__ int cur[kPlanMaxExperts];
  const int max_tiles = plan_max_tiles(n_pairs, E);
  int32_t* tiles = plan + 1;
  int32_t* sorted = plan + 1 + 3 * max_tiles;
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = idx[p];
    if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      cur[e] = off;
      for (int r0 = 0; r0 < cnt[e]; r0 += GM) {
        tiles[3 * nt] = e;
        tiles[3 * nt + 1] = off + r0;
        tiles[3 * nt + 2] = min(GM, cnt[e] - r0);
        ++nt;
      }
      off += cnt[e];
    }
    plan[0] = nt;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = idx[p];
    if (e >= 0 && e < E) sorted[atomicAdd(&cur[e], 1)] = p;
  }
}

// STAGE 0: A = h rows gathered by pair, B = gate | up rows of w_gu[e]; STAGE 1: A = act rows, B = w_down[e]
template <int STAGE>
__global__ void __launch_bounds__(G_THREADS) moe_gemm_kernel(const __nv_bfloat16* __restrict__ a, long long a_stride, const __nv_bfloat16* __restrict__ w,
                                                             const int32_t* __restrict__ plan, void* __restrict__ out, int n_pairs, int top, int E,
                                                             int ff, int W) {
  constexpr int NB = STAGE == 0 ? 2 : 1;  // B tiles per block
  constexpr int LD = GK + GPAD;
  __shared__ __align__(16) __nv_bfloat16 As[2][GM * LD];
  __shared__ __align__(16) __nv_bfloat16 Bs[2][NB * GN * LD];
  __shared__ int row_src[GM];
  const int tile = blockIdx.x;
  if (tile >= plan[0]) return;
  const int max_tiles = plan_max_tiles(n_pairs, E);
  const int e = plan[1 + 3 * tile], row0 = plan[2 + 3 * tile], rows = plan[3 + 3 * tile];
  const int32_t* sorted = plan + 1 + 3 * max_tiles;
  const int K = STAGE == 0 ? W : ff, N = STAGE == 0 ? ff : W;
  const int n0 = blockIdx.y * GN;
  const __nv_bfloat16* wb = STAGE == 0 ? w + static_cast<long long>(e) * 2 * ff * W : w + static_cast<long long>(e) * W * ff;
  for (int r = threadIdx.x; r < GM; r += G_THREADS) row_src[r] = r < rows ? sorted[row0 + r] : -1;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wm = warp >> 1, wn = warp & 1, grp = lane >> 2, qd = lane & 3;

  auto load = [&](int st, int k0) {
    for (int c = threadIdx.x; c < GM * (GK / 8); c += G_THREADS) {
      const int r = c / (GK / 8), kc = (c - r * (GK / 8)) * 8;
      __nv_bfloat16* d = &As[st][r * LD + kc];
      const int pr = row_src[r];
      if (pr >= 0 && k0 + kc < K) {
        const __nv_bfloat16* src = STAGE == 0 ? a + static_cast<long long>(pr / top) * a_stride : a + static_cast<long long>(row0 + r) * a_stride;
        cp_async16(d, src + k0 + kc);
      } else {
        *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    for (int c = threadIdx.x; c < NB * GN * (GK / 8); c += G_THREADS) {
      const int r = c / (GK / 8), kc = (c - r * (GK / 8)) * 8;
      const int part = r / GN, n = n0 + (r - part * GN);
      __nv_bfloat16* d = &Bs[st][r * LD + kc];
      if (n < N && k0 + kc < K) cp_async16(d, wb + (static_cast<long long>(part) * ff + n) * K + k0 + kc);
      else *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
    }
  };

  float acc[NB][2][4][4];
#pragma unroll
  for (int b = 0; b < NB; ++b)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[b][i][j][0] = acc[b][i][j][1] = acc[b][i][j][2] = acc[b][i][j][3] = 0.f;

  load(0, 0);
  cp_async_commit();
  const int steps = (K + GK - 1) / GK;
  for (int s = 0; s < steps; ++s) {
    const int st = s & 1;
    if (s + 1 < steps) load(st ^ 1, (s + 1) * GK);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t a_base = static_cast<uint32_t>(__cvta_generic_to_shared(&As[st][0])) + ((wm * 32 + (lane & 15)) * LD + (lane >> 4) * 8) * 2;
    const uint32_t b_base = static_cast<uint32_t>(__cvta_generic_to_shared(&Bs[st][0])) + ((wn * 32 + (lane & 7)) * LD + (lane >> 3) * 8) * 2;
    uint32_t af[2][2][4];  // [m tile][k16 step]
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) ldsm_x4(a_base + (i * 16 * LD + kk * 16) * 2, af[i][kk][0], af[i][kk][1], af[i][kk][2], af[i][kk][3]);
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      uint32_t bf[4][4];  // [n tile]: k 0..15 in [0],[1], k 16..31 in [2],[3]
#pragma unroll
      for (int j = 0; j < 4; ++j) ldsm_x4(b_base + ((b * GN + j * 8) * LD) * 2, bf[j][0], bf[j][1], bf[j][2], bf[j][3]);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_bf16(acc[b][i][j], af[i][0][0], af[i][0][1], af[i][0][2], af[i][0][3], bf[j][0], bf[j][1]);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_bf16(acc[b][i][j], af[i][1][0], af[i][1][1], af[i][1][2], af[i][1][3], bf[j][2], bf[j][3]);
    }
    __syncthreads();  // the next step's copies overwrite the other stage, which the step after reads
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = wm * 32 + i * 16 + grp + half * 8;
      if (r >= rows) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + wn * 32 + j * 8 + qd * 2;
        if (n >= N) continue;
        if (STAGE == 0) {
          const float g0 = acc[0][i][j][half * 2], g1 = acc[0][i][j][half * 2 + 1];
          const float u0 = acc[NB - 1][i][j][half * 2], u1 = acc[NB - 1][i][j][half * 2 + 1];
          __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out) + static_cast<long long>(row0 + r) * ff + n;
          *reinterpret_cast<uint32_t*>(o) = pack_bf16(g0 * sigmoidf_(g0) * u0, g1 * sigmoidf_(g1) * u1);
        } else {
          float* o = static_cast<float*>(out) + static_cast<long long>(row_src[r]) * W + n;
          *reinterpret_cast<float2*>(o) = make_float2(acc[0][i][j][half * 2], acc[0][i][j][half * 2 + 1]);
        }
      }
    }
}

}  // namespace
}  // namespace pcs

PCS_API int64_t pcs_moe_plan_ints(int n_pairs, int n_experts) {
  if (n_pairs <= 0 || n_experts <= 0) return 1;
  return 1 + 3LL * pcs::plan_max_tiles(n_pairs, n_experts) + n_pairs;
}

PCS_API int pcs_moe_plan(const int32_t* idx, int n_pairs, int n_experts, int32_t* plan, void* stream) {
  if (n_pairs == 0 || n_experts == 0) return PCS_OK;
  PCS_REQUIRE(idx && plan && n_pairs > 0 && n_experts > 0 && n_experts <= pcs::kPlanMaxExperts, "pcs_moe_plan: bad arguments (at most %d experts)",
              pcs::kPlanMaxExperts);
  pcs::moe_plan_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(idx, n_pairs, n_experts, plan);
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_moe_gemm(int stage, const void* a, int64_t a_stride, const void* w, const int32_t* plan, void* out, int n_pairs, int top,
                         int n_experts, int ff, int width, void* stream) {
  if (n_pairs == 0 || n_experts == 0) return PCS_OK;
  PCS_REQUIRE(a && w && plan && out && n_pairs > 0 && top > 0 && ff > 0 && width > 0 && (stage == 0 || stage == 1), "pcs_moe_gemm: bad arguments");
  PCS_REQUIRE(ff % 8 == 0 && width % 8 == 0 && a_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
              "pcs_moe_gemm: sizes, the row stride and the pointers must be multiples of 16 bytes");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int n = stage == 0 ? ff : width;
  dim3 grid(pcs::plan_max_tiles(n_pairs, n_experts), (n + pcs::GN - 1) / pcs::GN);
  PCS_REQUIRE(grid.y <= 65535, "pcs_moe_gemm: too many output features");
  const __nv_bfloat16* ap = static_cast<const __nv_bfloat16*>(a);
  const __nv_bfloat16* wp = static_cast<const __nv_bfloat16*>(w);
  if (stage == 0) pcs::moe_gemm_kernel<0><<<grid, pcs::G_THREADS, 0, st>>>(ap, a_stride, wp, plan, out, n_pairs, top, n_experts, ff, width);
  else pcs::moe_gemm_kernel<1><<<grid, pcs::G_THREADS, 0, st>>>(ap, a_stride, wp, plan, out, n_pairs, top, n_experts, ff, width);
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}
