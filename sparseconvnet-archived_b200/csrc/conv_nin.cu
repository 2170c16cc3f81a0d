// Fused rule-gather + NetworkInNetwork forward: dispatcher, the fp32 CUDA-core kernel used
// for small contractions (K = fs*nIn of a few dozen, which are HBM-bound) and as the
// arithmetic reference for the tensor-core kernel, and the row softmax of the classifier.
#include <cstdlib>
#include <cstring>
#include "scn_common.cuh"
#include "conv_nin_tc.cuh"

namespace scn {
namespace {

// out[r][n] = act(p * sum_k A[r][k] W[k][n] + p * B[n]),  A[r][f*nIn + c] = in[rules[r*fs+f]][c].
// CTA tile BM x BN, K slabs of BK, each thread a TM x TN register tile.  The gathered A tile
// only ever lives in shared memory: the [rows x K] matrix the reference materialises
// (ConvolutionalLayer.cu:124-133) is never written to HBM.
template <int BM, int BN, int BK, int TM, int TN, int ACT>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
k_conv_nin_simt(const float *__restrict__ in, const int *__restrict__ rules, int rows, int fs, int nIn,
                const float *__restrict__ W, const float *__restrict__ B, const float *__restrict__ prelu,
                int N, float p, float *__restrict__ out) {
  constexpr int THREADS = (BM / TM) * (BN / TN);
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN];
  const int K = fs * nIn;
  const int row0 = blockIdx.x * BM, col0 = blockIdx.y * BN;
  const int tx = threadIdx.x % (BN / TN), ty = threadIdx.x / (BN / TN);
  float acc[TM][TN];
#pragma unroll
  for (int a = 0; a < TM; ++a)
#pragma unroll
    for (int b = 0; b < TN; ++b) acc[a][b] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int e = threadIdx.x; e < BM * BK; e += THREADS) {
      const int m = e / BK, kk = e % BK;
      const int k = k0 + kk, r = row0 + m;
      float v = 0.f;
      if (r < rows && k < K) {
        const int f = k / nIn, c = k - f * nIn;
        const int src = rules ? __ldg(rules + (long long)r * fs + f) : r;
        if (src >= 0) v = __ldg(in + (long long)src * nIn + c);
      }
      As[kk][m] = v;
    }
    for (int e = threadIdx.x; e < BK * BN; e += THREADS) {
      const int kk = e / BN, n = e % BN;
      const int k = k0 + kk, col = col0 + n;
      Bs[kk][n] = (k < K && col < N) ? __ldg(W + (long long)k * N + col) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int r = row0 + ty * TM + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int col = col0 + tx * TN + j;
      if (col >= N) continue;
      // NetworkInNetworkLayer.cu:187-195: SGEMM with alpha = beta = p over a bias-filled C
      float v = p * acc[i][j] + p * __ldg(B + col);
      out[(long long)r * N + col] = activate_t<ACT>(v, ACT == SCN_PRELU ? __ldg(prelu + col) : 0.f);
    }
  }
}


// Small contraction (K = fs*nIn <= 64, e.g. the first 3x3 convolution over 3 channels,
// K = 27): the layer is HBM-bound (it writes rows x N and reads almost nothing), so the
// kernel is organised around the output write.  The whole W lives in shared memory; a CTA
// walks row tiles, gathers each tile's A rows into shared memory (transposed, so that four
// rows' values at one k are one 16-byte read), and each thread owns 4 rows x 4 consecutive
// columns: per k two 16-byte shared loads feed 16 FMAs, and the epilogue stores float4s that
// are contiguous across the threads of a row.
template <int ACT>
__global__ void __launch_bounds__(256)
k_conv_nin_smallk(const float *__restrict__ in, const int *__restrict__ rules, int rows, int fs, int nIn,
                  const float *__restrict__ W, const float *__restrict__ B, const float *__restrict__ prelu, int N,
                  float p, float *__restrict__ out) {
  extern __shared__ __align__(16) float sk_smem[];
  const int K = fs * nIn, NV = N >> 2;
  const int TY = blockDim.x / NV, TR = TY * 4;
  float *Ws = sk_smem;           // [K][N]
  float *As = sk_smem + K * N;   // [K][TR]
  const int tx = threadIdx.x % NV, ty = threadIdx.x / NV;
  const bool active = ty < TY;
  for (int e = threadIdx.x; e < K * N; e += blockDim.x) Ws[e] = __ldg(W + e);
  float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f), s4 = b4;
  if (active) {
    b4 = __ldg(reinterpret_cast<const float4 *>(B) + tx);
    if (ACT == SCN_PRELU) s4 = __ldg(reinterpret_cast<const float4 *>(prelu) + tx);
  }
  const int nTiles = (rows + TR - 1) / TR;
  for (int tile = blockIdx.x; tile < nTiles; tile += gridDim.x) {
    const int row0 = tile * TR;
    __syncthreads();
    for (int e = threadIdx.x; e < TR * K; e += blockDim.x) {
      const int r = e / K, k = e - r * K;
      const int row = row0 + r;
      float v = 0.f;
      if (row < rows) {
        const int f = k / nIn, c = k - f * nIn;
        const int src = rules ? __ldg(rules + (long long)row * fs + f) : row;
        if (src >= 0) v = __ldg(in + (long long)src * nIn + c);
      }
      As[k * TR + r] = v;
    }
    __syncthreads();
    if (!active) continue;
    float4 acc[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < K; ++k) {
      const float4 w = *reinterpret_cast<const float4 *>(Ws + k * N + tx * 4);
      const float4 a = *reinterpret_cast<const float4 *>(As + k * TR + ty * 4);
      const float av[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[i].x = fmaf(av[i], w.x, acc[i].x); acc[i].y = fmaf(av[i], w.y, acc[i].y);
        acc[i].z = fmaf(av[i], w.z, acc[i].z); acc[i].w = fmaf(av[i], w.w, acc[i].w);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = row0 + ty * 4 + i;
      if (row >= rows) continue;
      float4 o;
      o.x = activate_t<ACT>(p * acc[i].x + p * b4.x, s4.x); o.y = activate_t<ACT>(p * acc[i].y + p * b4.y, s4.y);
      o.z = activate_t<ACT>(p * acc[i].z + p * b4.z, s4.z); o.w = activate_t<ACT>(p * acc[i].w + p * b4.w, s4.w);
      reinterpret_cast<float4 *>(out + (long long)row * N)[tx] = o;
    }
  }
}

// Few outputs (N <= 32, the classifier): one warp per row.  Lanes stride over K, keep N partial
// sums each, the sums are combined with shuffles, lane n finishes output n; SOFTMAX is the row
// softmax of SigmoidLayer.cu:160-177 done across the lanes (running max starts at -10000).
template <int NMAX>
__global__ void __launch_bounds__(256)
k_nin_smalln(const float *__restrict__ in, const int *__restrict__ rules, int rows, int fs, int nIn,
             const float *__restrict__ W, const float *__restrict__ B, const float *__restrict__ prelu, int N,
             float p, int act, float *__restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int K = fs * nIn;
  for (int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += gridDim.x * (blockDim.x >> 5)) {
    float acc[NMAX];
#pragma unroll
    for (int n = 0; n < NMAX; ++n) acc[n] = 0.f;
    for (int k = lane; k < K; k += 32) {
      const int f = k / nIn, c = k - f * nIn;
      const int src = rules ? __ldg(rules + (long long)row * fs + f) : row;
      const float x = src >= 0 ? __ldg(in + (long long)src * nIn + c) : 0.f;
      const float *w = W + (long long)k * N;
#pragma unroll
      for (int n = 0; n < NMAX; ++n)
        if (n < N) acc[n] = fmaf(x, __ldg(w + n), acc[n]);
    }
    float mine = 0.f;
#pragma unroll
    for (int n = 0; n < NMAX; ++n) {
      float v = acc[n];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == n) mine = v;
    }
    const bool valid = lane < N;
    float v = valid ? p * mine + p * __ldg(B + lane) : -10000.0f;
    if (act == SCN_SOFTMAX) {
      float mx = fmaxf(v, -10000.0f);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float e = valid ? expf(v - mx) : 0.f, sum = e;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      v = e / sum;
    } else if (valid) {
      v = activate(v, act, prelu ? __ldg(prelu + lane) : 0.f);
    }
    if (valid) out[(long long)row * N + lane] = v;
  }
}

// The same layer when W fits shared memory (the usual classifier: 608 x 10).  k_nin_smalln waits for L2 in
// each of its K/32 iterations (17 us on 256 rows).  Here a CTA fetches W (row stride made odd in shared
// memory, so that the lanes' reads fall in distinct banks) and the (gathered) input rows of its eight warps
// with batches of independent 16-byte loads held in registers, so that the whole fetch costs two or three
// round trips to L2, and the sums run out of shared memory.  Needs nIn % 4 == 0, (K * N) % 4 == 0 and
// 16-byte aligned arrays.
template <int NMAX>
__global__ void __launch_bounds__(256)
k_nin_smalln_staged(const float *__restrict__ in, const int *__restrict__ rules, int rows, int fs, int nIn,
                    const float *__restrict__ W, const float *__restrict__ B, const float *__restrict__ prelu, int N,
                    float p, int act, float *__restrict__ out) {
  extern __shared__ float sm[];
  constexpr int U = 8, R = 8;
  const int K = fs * nIn, NP = N | 1, K4 = K >> 2;
  float *wS = sm;                   // [K][NP]
  float *xS = sm + (size_t)K * NP;  // [R][K]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  dependents_may_launch();
  const int nW4 = (K * N) >> 2;
  for (int base = 0; base < nW4; base += 256 * U) { // the weights do not come from the kernel in front
    float4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = base + u * 256 + threadIdx.x;
      v[u] = __ldg(reinterpret_cast<const float4 *>(W) + (i < nW4 ? i : 0)); // unconditional: no select waits on the value
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = base + u * 256 + threadIdx.x;
      if (i < nW4) {
        const float e[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int k = (4 * i + c) / N;
          wS[k * NP + (4 * i + c - k * N)] = e[c];
        }
      }
    }
  }
  wait_for_prior_grids();
  for (int row0 = blockIdx.x * R; row0 < rows; row0 += gridDim.x * R) {
    __syncthreads();
    for (int base = 0; base < R * K4; base += 256 * U) {
      int src[U];
#pragma unroll
      for (int u = 0; u < U; ++u) { // rule reads first, then the feature reads that depend on them
        const int i = base + u * 256 + threadIdx.x, r = i / K4, row = row0 + r;
        src[u] = -1;
        if (i < R * K4 && row < rows) src[u] = rules ? __ldg(rules + (long long)row * fs + (4 * (i - r * K4)) / nIn) : row;
      }
      float4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = base + u * 256 + threadIdx.x, r = i / K4, k = 4 * (i - r * K4);
        v[u] = *reinterpret_cast<const float4 *>(in + (long long)(src[u] >= 0 ? src[u] : 0) * nIn + (k % nIn));
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = base + u * 256 + threadIdx.x;
        if (i < R * K4) reinterpret_cast<float4 *>(xS)[i] = src[u] >= 0 ? v[u] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    __syncthreads();
    const int row = row0 + warp;
    if (row >= rows) continue;
    float acc[NMAX];
#pragma unroll
    for (int n = 0; n < NMAX; ++n) acc[n] = 0.f;
    for (int k = lane; k < K; k += 32) {
      const float x = xS[warp * K + k];
      const float *w = wS + k * NP;
#pragma unroll
      for (int n = 0; n < NMAX; ++n)
        if (n < N) acc[n] = fmaf(x, w[n], acc[n]);
    }
    float mine = 0.f;
#pragma unroll
    for (int n = 0; n < NMAX; ++n) {
      float v = acc[n];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == n) mine = v;
    }
    const bool valid = lane < N;
    float v = valid ? p * mine + p * __ldg(B + lane) : -10000.0f;
    if (act == SCN_SOFTMAX) {
      float mx = fmaxf(v, -10000.0f);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float e = valid ? expf(v - mx) : 0.f, sum = e;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      v = e / sum;
    } else if (valid) {
      v = activate(v, act, prelu ? __ldg(prelu + lane) : 0.f);
    }
    if (valid) out[(long long)row * N + lane] = v;
  }
}

// Few rows (one per sample at the top of a network) and any N: one CTA per row, the (gathered) input row
// in shared memory, threads over the output columns, so that W is read coalesced and each thread runs
// K independent FMAs.  The tile kernel would leave all but a couple of SMs idle on such a layer.
template <int ACT>
__global__ void __launch_bounds__(256)
k_nin_fewrows(const float *__restrict__ in, const int *__restrict__ rules, int rows, int fs, int nIn,
              const float *__restrict__ W, const float *__restrict__ B, const float *__restrict__ prelu, int N,
              float p, float *__restrict__ out) {
  extern __shared__ float xS[]; // K floats
  const int K = fs * nIn;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    __syncthreads();
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
      int src = row, c = k;
      if (rules) {
        const int f = k / nIn;
        c = k - f * nIn;
        src = __ldg(rules + (long long)row * fs + f);
      }
      xS[k] = src >= 0 ? __ldg(in + (long long)src * nIn + c) : 0.f;
    }
    __syncthreads();
    for (int n = threadIdx.x; n < N; n += blockDim.x) {
      float acc = 0.f;
#pragma unroll 8
      for (int k = 0; k < K; ++k) acc = fmaf(xS[k], __ldg(W + (long long)k * N + n), acc);
      out[(long long)row * N + n] = activate_t<ACT>(p * acc + p * __ldg(B + n), ACT == SCN_PRELU ? __ldg(prelu + n) : 0.f);
    }
  }
}

// Row softmax of SigmoidLayer.cu:160-177 (running max starts at -10000), in place, one
// warp per row (N is the class count).
__global__ void k_softmax_rows(float *x, int rows, int N) {
  const int lane = threadIdx.x & 31;
  for (int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += gridDim.x * (blockDim.x >> 5)) {
    float *a = x + (long long)r * N;
    float mx = -10000.0f;
    for (int k = lane; k < N; k += 32) mx = fmaxf(mx, a[k]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float acc = 0.0f;
    for (int k = lane; k < N; k += 32) { const float e = expf(a[k] - mx); a[k] = e; acc += e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    for (int k = lane; k < N; k += 32) a[k] /= acc;
  }
}

} // namespace
} // namespace scn

using namespace scn;

extern "C" int scn_conv_auto_precision(void) {
  // SCN_AUTO_PRECISION=split|3xtf32|3xbf16|bf16 overrides the default for a process (read once)
  static const int chosen = [] {
    const char *e = getenv("SCN_AUTO_PRECISION");
    if (e && !strcmp(e, "3xbf16")) return (int)SCN_PREC_3XBF16;
    if (e && !strcmp(e, "bf16")) return (int)SCN_PREC_BF16;
    if (e && !strcmp(e, "3xtf32")) return (int)SCN_PREC_3XTF32;
    return (int)SCN_PREC_SPLIT;
  }();
  return chosen;
}

extern "C" size_t scn_conv_nin_workspace_bytes(int rows_out, int fs, int nIn, int N, int precision) {
  if (rows_out < 1 || fs < 1 || nIn < 1 || N < 1) return 0;
  return tc_workspace_bytes(rows_out, fs, nIn, N, precision == SCN_PREC_AUTO ? scn_conv_auto_precision() : precision);
}

extern "C" int scn_conv_nin_forward(const float *d_in, const int *d_rules, int rows_out, int fs, int nIn,
                                    const float *d_W, const void *d_W_packed, const float *d_B,
                                    const float *d_prelu, int N, float p, int act, int precision, float *d_out,
                                    scn_stream_t stream) {
  return scn_conv_nin_forward_ws(d_in, d_rules, rows_out, fs, nIn, d_W, d_W_packed, d_B, d_prelu, N, p, act, precision, d_out,
                                 nullptr, 0, stream);
}

extern "C" int scn_conv_nin_forward_ws(const float *d_in, const int *d_rules, int rows_out, int fs, int nIn,
                                       const float *d_W, const void *d_W_packed, const float *d_B,
                                       const float *d_prelu, int N, float p, int act, int precision, float *d_out,
                                       void *d_workspace, size_t workspace_bytes, scn_stream_t stream) {
  clear_error();
  if (rows_out < 0 || fs < 1 || nIn < 1 || N < 1) return fail(SCN_ERR_INVALID, "bad conv/NiN sizes");
  if (!d_rules && fs != 1) return fail(SCN_ERR_INVALID, "fs must be 1 without rules");
  if (act < SCN_NOSIGMOID || act > SCN_SIGMOID) return fail(SCN_ERR_INVALID, "unknown activation");
  if (act == SCN_PRELU && !d_prelu) return fail(SCN_ERR_INVALID, "PReLU slopes missing");
  if (act == SCN_SOFTMAX && N > 1024) return fail(SCN_ERR_INVALID, "softmax over more than 1024 classes");
  if (precision < SCN_PREC_AUTO || precision > SCN_PREC_SPLIT) return fail(SCN_ERR_INVALID, "unknown precision");
  if (rows_out == 0) return SCN_OK;
  if (!d_in || !d_W || !d_B || !d_out) return fail(SCN_ERR_INVALID, "null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const int inner = (act == SCN_SOFTMAX) ? SCN_NOSIGMOID : act;

  int use = precision;
  if (precision == SCN_PREC_AUTO) use = (d_W_packed && tc_shape_ok(fs, nIn, N, scn_conv_auto_precision())) ? scn_conv_auto_precision() : SCN_PREC_FP32;
  if (use != SCN_PREC_FP32) {
    if (!tc_shape_ok(fs, nIn, N, use)) return fail(SCN_ERR_UNSUPPORTED, "shape not supported by the tensor-core kernel (need N >= 16 and N % 4 == 0)");
    if (!d_W_packed) return fail(SCN_ERR_INVALID, "tensor-core precision needs packed weights");
    int st = tc_launch(d_in, d_rules, rows_out, fs, nIn, d_W_packed, d_B, d_prelu, N, p, inner, use, d_out, d_workspace, workspace_bytes, s);
    if (st != SCN_OK) return st;
  } else if (N <= 32) {
    // the classifier shape: warp per row, softmax fused
    const size_t staged = ((size_t)fs * nIn * (N | 1) + 8 * (size_t)fs * nIn) * sizeof(float);
    if (staged <= 96 * 1024 && nIn % 4 == 0 && (fs * nIn * N) % 4 == 0 && (((uintptr_t)d_in | (uintptr_t)d_W) & 15) == 0) {
      const int tiles = (rows_out + 7) / 8, blocks = tiles < 4 * sm_count() ? tiles : 4 * sm_count();
      if (N <= 16) {
        if (staged > 48 * 1024) SCN_CUDA_TRY(cudaFuncSetAttribute(k_nin_smalln_staged<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
        (void)launch_dependent(k_nin_smalln_staged<16>, dim3(blocks), dim3(256), staged, s, d_in, d_rules, rows_out, fs, nIn, d_W, d_B, d_prelu, N, p, act, d_out);
      } else {
        if (staged > 48 * 1024) SCN_CUDA_TRY(cudaFuncSetAttribute(k_nin_smalln_staged<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
        (void)launch_dependent(k_nin_smalln_staged<32>, dim3(blocks), dim3(256), staged, s, d_in, d_rules, rows_out, fs, nIn, d_W, d_B, d_prelu, N, p, act, d_out);
      }
      SCN_LAUNCH_CHECK("k_nin_smalln_staged");
      return SCN_OK;
    }
    const int blocks = grid_for((long long)rows_out * 32, 256);
    if (N <= 16) k_nin_smalln<16><<<blocks, 256, 0, s>>>(d_in, d_rules, rows_out, fs, nIn, d_W, d_B, d_prelu, N, p, act, d_out);
    else k_nin_smalln<32><<<blocks, 256, 0, s>>>(d_in, d_rules, rows_out, fs, nIn, d_W, d_B, d_prelu, N, p, act, d_out);
    SCN_LAUNCH_CHECK("k_nin_smalln");
    return SCN_OK;
  } else if (fs * nIn <= 64 && N % 4 == 0 && N <= 256 && (((uintptr_t)d_out | (uintptr_t)d_B | (uintptr_t)d_prelu) & 15) == 0) {
    const int K = fs * nIn, NV = N / 4, TR = (256 / NV) * 4;
    const size_t smem = (size_t)(K * N + K * TR) * sizeof(float);
    if (smem > 48 * 1024) {
      SCN_DISPATCH_ACT(inner, SCN_CUDA_TRY(cudaFuncSetAttribute(k_conv_nin_smallk<ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024)));
    }
    const int tiles = (rows_out + TR - 1) / TR;
    const int blocks = tiles < sm_count() * 4 ? tiles : sm_count() * 4;
    SCN_DISPATCH_ACT(inner, (k_conv_nin_smallk<ACT><<<blocks, 256, smem, s>>>(d_in, d_rules, rows_out, fs, nIn, d_W, d_B, d_prelu, N, p, d_out)));
    SCN_LAUNCH_CHECK("k_conv_nin_smallk");
  } else if (rows_out <= 2048 && (size_t)fs * nIn * sizeof(float) <= 48 * 1024) {
    const int threads = N >= 256 ? 256 : (N + 31) / 32 * 32;
    SCN_DISPATCH_ACT(inner, (k_nin_fewrows<ACT><<<rows_out, threads, (size_t)fs * nIn * sizeof(float), s>>>(d_in, d_rules, rows_out, fs, nIn, d_W, d_B,
                                                                                                 d_prelu, N, p, d_out)));
    SCN_LAUNCH_CHECK("k_nin_fewrows");
  } else {
    constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
    dim3 grid((rows_out + BM - 1) / BM, (N + BN - 1) / BN);
    SCN_DISPATCH_ACT(inner, (k_conv_nin_simt<BM, BN, BK, TM, TN, ACT><<<grid, (BM / TM) * (BN / TN), 0, s>>>(d_in, d_rules, rows_out, fs, nIn, d_W,
                                                                                             d_B, d_prelu, N, p, d_out)));
    SCN_LAUNCH_CHECK("k_conv_nin_simt");
  }
  if (act == SCN_SOFTMAX) {
    k_softmax_rows<<<grid_for((long long)rows_out * 32, 128), 128, 0, s>>>(d_out, rows_out, N);
    SCN_LAUNCH_CHECK("k_softmax_rows");
  }
  return SCN_OK;
}

extern "C" int scn_conv_nin_forward_dyn(const float *d_in, const int *d_rules, int rows_out_bound, const int *d_rows_out, int fs, int nIn,
                                        const void *d_W_packed, const float *d_B, const float *d_prelu, int N, float p, int act,
                                        float *d_out, int precision, scn_stream_t stream) {
  clear_error();
  if (precision != SCN_PREC_3XTF32 && precision != SCN_PREC_SPLIT) return fail(SCN_ERR_UNSUPPORTED, "precision must be SCN_PREC_3XTF32 or SCN_PREC_SPLIT here");
  if (rows_out_bound < 1 || fs < 1 || nIn < 1 || N < 1) return fail(SCN_ERR_INVALID, "bad conv/NiN sizes");
  if (!d_rules && fs != 1) return fail(SCN_ERR_INVALID, "fs must be 1 without rules");
  if (act < SCN_NOSIGMOID || act > SCN_SIGMOID || act == SCN_SOFTMAX) return fail(SCN_ERR_INVALID, "activation not supported here");
  if (act == SCN_PRELU && !d_prelu) return fail(SCN_ERR_INVALID, "PReLU slopes missing");
  if (!d_in || !d_rows_out || !d_W_packed || !d_B || !d_out) return fail(SCN_ERR_INVALID, "null pointer");
  if (!tc_shape_ok(fs, nIn, N, precision)) return fail(SCN_ERR_UNSUPPORTED, "shape not supported by the tensor-core kernel");
  return tc_launch(d_in, d_rules, rows_out_bound, fs, nIn, d_W_packed, d_B, d_prelu, N, p, act, precision, d_out, nullptr, 0,
                   (cudaStream_t)stream, d_rows_out);
}

extern "C" int scn_conv_nin_maxpool_forward(const float *d_in, const int *d_rules, int fs, int nIn, const void *d_W_packed, const float *d_B,
                                            const float *d_prelu, int N, float p, int act, const int *d_pool_rules, int pool_cells,
                                            int rows_pool_bound, const int *d_rows_pool, int rows_unpooled, float *d_out, int *d_choices,
                                            void *d_workspace, size_t workspace_bytes, int precision, scn_stream_t stream) {
  clear_error();
  if (precision != SCN_PREC_3XTF32 && precision != SCN_PREC_SPLIT) return fail(SCN_ERR_UNSUPPORTED, "precision must be SCN_PREC_3XTF32 or SCN_PREC_SPLIT here");
  if (rows_pool_bound < 0 || fs < 1 || nIn < 1 || N < 1) return fail(SCN_ERR_INVALID, "bad conv/NiN sizes");
  if (act < SCN_NOSIGMOID || act > SCN_SIGMOID || act == SCN_SOFTMAX) return fail(SCN_ERR_INVALID, "activation not supported here");
  if (act == SCN_PRELU && !d_prelu) return fail(SCN_ERR_INVALID, "PReLU slopes missing");
  if (rows_pool_bound == 0) return SCN_OK;
  if (!d_in || !d_rules || !d_W_packed || !d_B || !d_pool_rules || !d_out || !d_choices) return fail(SCN_ERR_INVALID, "null pointer");
  if (!tc_shape_ok(fs, nIn, N, precision)) return fail(SCN_ERR_UNSUPPORTED, "shape not supported by the tensor-core kernel");
  return tc_launch(d_in, d_rules, rows_pool_bound, fs, nIn, d_W_packed, d_B, d_prelu, N, p, act, precision, d_out, d_workspace,
                   workspace_bytes, (cudaStream_t)stream, d_rows_pool, d_pool_rules, pool_cells, d_choices, rows_unpooled);
}

extern "C" int scn_conv_nin_nin_forward(const float *d_in, const int *d_rules, int rows_out, int fs, int nIn, const void *d_W_packed,
                                        const float *d_B, const float *d_prelu, int N, float p, int act, const float *d_W2, const float *d_B2,
                                        const float *d_prelu2, int N2, float p2, int act2, float *d_mid, float *d_out, void *d_workspace,
                                        size_t workspace_bytes, int precision, scn_stream_t stream) {
  clear_error();
  if (precision != SCN_PREC_3XTF32 && precision != SCN_PREC_SPLIT) return fail(SCN_ERR_UNSUPPORTED, "precision must be SCN_PREC_3XTF32 or SCN_PREC_SPLIT here");
  if (rows_out < 0 || fs < 1 || nIn < 1 || N < 1 || N2 < 1) return fail(SCN_ERR_INVALID, "bad conv/NiN sizes");
  if (!d_rules && fs != 1) return fail(SCN_ERR_INVALID, "fs must be 1 without rules");
  if (act < SCN_NOSIGMOID || act > SCN_SIGMOID || act == SCN_SOFTMAX) return fail(SCN_ERR_INVALID, "activation not supported for the first layer");
  if (act2 < SCN_NOSIGMOID || act2 > SCN_SIGMOID) return fail(SCN_ERR_INVALID, "unknown activation");
  if ((act == SCN_PRELU && !d_prelu) || (act2 == SCN_PRELU && !d_prelu2)) return fail(SCN_ERR_INVALID, "PReLU slopes missing");
  if (rows_out == 0) return SCN_OK;
  if (!d_in || !d_W_packed || !d_B || !d_W2 || !d_B2 || !d_mid || !d_out) return fail(SCN_ERR_INVALID, "null pointer");
  if (N2 > 16 || N % 4 != 0 || !d_workspace || !tc_shape_ok(fs, nIn, N, precision))
    return fail(SCN_ERR_UNSUPPORTED, "needs the split tensor-core kernel with a K split and at most 16 outputs of the second layer");
  FinishNin f2 = {d_W2, d_B2, d_prelu2, N2, p2, act2, d_out};
  return tc_launch(d_in, d_rules, rows_out, fs, nIn, d_W_packed, d_B, d_prelu, N, p, act, precision, d_mid, d_workspace, workspace_bytes,
                   (cudaStream_t)stream, nullptr, nullptr, 0, nullptr, 0, nullptr, &f2);
}

extern "C" size_t scn_conv_packed_weight_bytes(int K, int N, int precision) { return tc_packed_bytes(K, N, precision); }

extern "C" int scn_conv_pack_weights(const float *d_W, int K, int N, int precision, void *d_W_packed,
                                     scn_stream_t stream) {
  clear_error();
  if (K < 1 || N < 1 || !d_W || !d_W_packed) return fail(SCN_ERR_INVALID, "bad pack arguments");
  return tc_pack(d_W, K, N, precision, d_W_packed, (cudaStream_t)stream);
}

extern "C" int scn_conv_tc_take_error(void) { return tc_take_error(); }
extern "C" const int *scn_conv_tc_error_word(void) { return tc_error_word(); }
