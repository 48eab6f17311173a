// Linear layer for a handful of rows (decoding): out[m, n] = sum_k x[m, k] W[n, k] + b[n], weights streamed once.
//
// With one to eight rows the product is bound by reading W; a library matrix product launches a tile kernel that leaves
// most of the memory system idle at this shape.  Here a block owns eight output features and its 256 threads share K: a
// thread takes every 256th 16-byte piece, requests that piece of all eight weight rows at once (eight loads in flight),
// multiplies them with the matching piece of every input row (which stays in L1) and keeps 32-bit sums; lanes meet in a
// butterfly, warps through shared memory.  The order of every sum depends on K alone.
#include "seq_common.cuh"

namespace pcs {

__device__ __forceinline__ void cvt16(const uint4& v, float (&o)[4], const float*) {
  o[0] = __uint_as_float(v.x); o[1] = __uint_as_float(v.y); o[2] = __uint_as_float(v.z); o[3] = __uint_as_float(v.w);
}
__device__ __forceinline__ void cvt16(const uint4& v, float (&o)[8], const __nv_bfloat16*) {
  o[0] = __uint_as_float(v.x << 16); o[1] = __uint_as_float(v.x & 0xffff0000u);
  o[2] = __uint_as_float(v.y << 16); o[3] = __uint_as_float(v.y & 0xffff0000u);
  o[4] = __uint_as_float(v.z << 16); o[5] = __uint_as_float(v.z & 0xffff0000u);
  o[6] = __uint_as_float(v.w << 16); o[7] = __uint_as_float(v.w & 0xffff0000u);
}

constexpr int kLinRows = 8;  // output features per block

template <typename T, int MB>
__global__ void __launch_bounds__(256) linear_rows_kernel(const T* __restrict__ x, long long x_stride, const T* __restrict__ w,
                                                          const T* __restrict__ bias, T* __restrict__ out, long long out_stride,
                                                          int M, int N, int K) {
  constexpr int NV = Vec<T>::n;
  __shared__ float red[8][kLinRows * MB];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * kLinRows, nr = min(kLinRows, N - n0);
  float acc[kLinRows][MB];
#pragma unroll
  for (int r = 0; r < kLinRows; ++r)
#pragma unroll
    for (int m = 0; m < MB; ++m) acc[r][m] = 0.f;
  for (int k = tid * NV; k < K; k += 256 * NV) {
    uint4 wv[kLinRows];
#pragma unroll
    for (int r = 0; r < kLinRows; ++r)  // a block past the last feature re-reads the last row; its sums are not stored
      wv[r] = *reinterpret_cast<const uint4*>(w + static_cast<long long>(n0 + min(r, nr - 1)) * K + k);
    float xv[MB][NV];
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      const uint4 raw = *reinterpret_cast<const uint4*>(x + min(m, M - 1) * x_stride + k);
      cvt16(raw, xv[m], static_cast<const T*>(nullptr));
    }
#pragma unroll
    for (int r = 0; r < kLinRows; ++r) {
      float wf[NV];
      cvt16(wv[r], wf, static_cast<const T*>(nullptr));
#pragma unroll
      for (int m = 0; m < MB; ++m)
#pragma unroll
        for (int e = 0; e < NV; ++e) acc[r][m] = fmaf(xv[m][e], wf[e], acc[r][m]);
    }
  }
#pragma unroll
  for (int r = 0; r < kLinRows; ++r)
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      const float s = warp_sum(acc[r][m]);
      if (lane == 0) red[warp][r * MB + m] = s;
    }
  __syncthreads();
  if (tid < kLinRows * MB) {
    const int r = tid / MB, m = tid - r * MB;
    if (r < nr && m < M) {
      float s = 0.f;
#pragma unroll
      for (int q = 0; q < 8; ++q) s += red[q][tid];
      stf(out + m * out_stride + n0 + r, s + (bias ? ldf(bias + n0 + r) : 0.f));
    }
  }
}

}  // namespace pcs

PCS_API int pcs_linear_rows(const void* x, int64_t x_stride, const void* w, const void* bias, void* out, int64_t out_stride, int m, int n,
                            int k, int dtype, void* stream) {
  if (m == 0 || n == 0) return PCS_OK;
  PCS_REQUIRE(x && w && out && m > 0 && m <= 8 && n > 0 && k > 0, "pcs_linear_rows: bad arguments (1 to 8 rows)");
  const int piece = dtype == PCS_BF16 ? 8 : 4;
  const long long esz = dtype == PCS_BF16 ? 2 : 4;
  PCS_REQUIRE(k % piece == 0 && (x_stride * esz) % 16 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
              "pcs_linear_rows: K, the row stride and the pointers must be multiples of 16 bytes");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int blocks = (n + pcs::kLinRows - 1) / pcs::kLinRows;
#define PCS_LINEAR_ROWS(MBV)                                                                                                          \
  PCS_DISPATCH(dtype, (pcs::linear_rows_kernel<T, MBV><<<blocks, 256, 0, st>>>(static_cast<const T*>(x), x_stride, static_cast<const T*>(w), \
                                                                              static_cast<const T*>(bias), static_cast<T*>(out), out_stride, m, n, k)))
  if (m == 1) PCS_LINEAR_ROWS(1);
  else if (m == 2) PCS_LINEAR_ROWS(2);
  else if (m <= 4) PCS_LINEAR_ROWS(4);
  else PCS_LINEAR_ROWS(8);
#undef PCS_LINEAR_ROWS
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}
