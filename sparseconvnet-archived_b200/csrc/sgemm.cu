// Row-major fp32 matrix products with the shapes of the reference's four cuBLAS wrappers (utilities.cu:132-169):
// C[l x r] = alpha * op(A) * op(B) + beta * C, op(A) l x m, op(B) m x r, where a transposed operand is stored as the
// transpose (A^t: m x l in memory).  Not on the forward path (the layers run the fused kernels); kept so that code written
// against those wrappers has something to call.  64 x 64 output tiles, 16-wide steps of m staged in shared memory, a
// 4 x 4 block of outputs per thread, products in fp32 with fused multiply-adds (cuBLAS orders its sums differently: equal
// to rounding, not bit for bit).
#include "scn_common.cuh"

namespace scn {
namespace {
constexpr int TM = 64, TN = 64, TK = 16;

template <bool TA, bool TB>
__global__ void __launch_bounds__(256) k_sgemm(const float *__restrict__ A, const float *__restrict__ B, float *__restrict__ C, int l, int m, int r,
                                                float alpha, float beta) {
  __shared__ float As[TK][TM + 1], Bs[TK][TN + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4; // 16 x 16 threads, 4 x 4 outputs each
  const int row0 = blockIdx.y * TM, col0 = blockIdx.x * TN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < m; k0 += TK) {
    for (int e = threadIdx.x; e < TK * TM; e += 256) {
      // the index that is contiguous in memory runs fastest over the threads
      const int k = TA ? e / TM : e % TK, i = TA ? e % TM : e / TK;
      const int gi = row0 + i, gk = k0 + k;
      As[k][i] = (gi < l && gk < m) ? (TA ? A[(long long)gk * l + gi] : A[(long long)gi * m + gk]) : 0.f;
    }
    for (int e = threadIdx.x; e < TK * TN; e += 256) {
      const int k = TB ? e % TK : e / TN, j = TB ? e / TK : e % TN;
      const int gj = col0 + j, gk = k0 + k;
      Bs[k][j] = (gj < r && gk < m) ? (TB ? B[(long long)gj * m + gk] : B[(long long)gk * r + gj]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gi = row0 + ty * 4 + i;
    if (gi >= l) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gj = col0 + tx * 4 + j;
      if (gj >= r) continue;
      float *c = C + (long long)gi * r + gj;
      *c = beta == 0.f ? alpha * acc[i][j] : alpha * acc[i][j] + beta * *c; // (beta = 0: C is not read, as in BLAS)
    }
  }
}
} // namespace
} // namespace scn

using namespace scn;

extern "C" int scn_sgemm_rowmajor(int transA, int transB, const float *d_A, const float *d_B, float *d_C, int l, int m, int r, float alpha,
                                  float beta, scn_stream_t stream) {
  clear_error();
  if (l < 0 || m < 0 || r < 0) return fail(SCN_ERR_INVALID, "bad matrix sizes");
  if (l == 0 || r == 0) return SCN_OK;
  if (!d_C || (m > 0 && (!d_A || !d_B))) return fail(SCN_ERR_INVALID, "null pointer");
  const dim3 grid((r + TN - 1) / TN, (l + TM - 1) / TM);
  if (grid.y > 65535) return fail(SCN_ERR_UNSUPPORTED, "more than 65535 x 64 rows");
  cudaStream_t s = (cudaStream_t)stream;
  if (transA && transB) k_sgemm<true, true><<<grid, 256, 0, s>>>(d_A, d_B, d_C, l, m, r, alpha, beta);
  else if (transA) k_sgemm<true, false><<<grid, 256, 0, s>>>(d_A, d_B, d_C, l, m, r, alpha, beta);
  else if (transB) k_sgemm<false, true><<<grid, 256, 0, s>>>(d_A, d_B, d_C, l, m, r, alpha, beta);
  else k_sgemm<false, false><<<grid, 256, 0, s>>>(d_A, d_B, d_C, l, m, r, alpha, beta);
  SCN_LAUNCH_CHECK("k_sgemm");
  return SCN_OK;
}
