// Backward pass of the layers of the forward path (training step): the error at the softmax, the activation
// derivatives, the learnt layers' weight / bias gradients with the convolution's gather read through the
// rulebook inside the kernel, the scatter of the gathered matrix's gradient back onto the rows it came from,
// the max-pooling and terminal-pooling gradients and the reference's SGD update.  The gradient with respect
// to a learnt layer's input is its forward kernel run on the transposed weights (scn_conv_nin_forward_ws),
// so it takes the tensor-core path wherever the forward does.
#include "scn_common.cuh"
#include "conv_nin_tc.cuh"
#include <algorithm>

namespace scn {
namespace {

// SoftmaxClassifier.cu:7-14: d cost / d (softmax input) = probabilities - one_hot(label).
__global__ void k_softmax_nll_backward(const float *__restrict__ probs, const int *__restrict__ labels, long long n, int N, float *__restrict__ d) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / N;
    const int c = (int)(i - r * N);
    d[i] = probs[i] - (c == labels[r] ? 1.0f : 0.0f);
  }
}

// applySigmoidBackProp in place (SigmoidLayer.cu:24-30, 62-68, 97-103, 137-143, 178-185): the derivative is
// taken from the ACTIVATED features b, as the reference does.
template <int ACT> __device__ __forceinline__ float act_backward(float b, float d, float slope) {
  if (ACT == SCN_RELU) return b > 0.f ? d : 0.f;
  if (ACT == SCN_VLEAKYRELU) return b > 0.f ? d : d * 0.333f;
  if (ACT == SCN_LEAKYRELU) return b > 0.f ? d : d * 0.01f;
  if (ACT == SCN_TANH) return d * (1.f + b) * (1.f - b);
  if (ACT == SCN_SIGMOID) return d * b * (1.f - b);
  if (ACT == SCN_PRELU) return b > 0.f ? d : d * slope;
  return d;
}
template <int ACT>
__global__ void k_activation_backward(const float *__restrict__ b, float *__restrict__ d, long long n4, const float *__restrict__ prelu, int N) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 bv = reinterpret_cast<const float4 *>(b)[i];
    float4 dv = reinterpret_cast<float4 *>(d)[i];
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    if (ACT == SCN_PRELU) s = *reinterpret_cast<const float4 *>(prelu + (int)((i * 4) % N));
    dv.x = act_backward<ACT>(bv.x, dv.x, s.x); dv.y = act_backward<ACT>(bv.y, dv.y, s.y);
    dv.z = act_backward<ACT>(bv.z, dv.z, s.z); dv.w = act_backward<ACT>(bv.w, dv.w, s.w);
    reinterpret_cast<float4 *>(d)[i] = dv;
  }
}
template <int ACT>
__global__ void k_activation_backward_scalar(const float *__restrict__ b, float *__restrict__ d, long long n, const float *__restrict__ prelu, int N) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    d[i] = act_backward<ACT>(b[i], d[i], ACT == SCN_PRELU ? prelu[(int)(i % N)] : 0.f);
}
// PReLU slope gradient (NetworkInNetworkPReLULayer.cu:25-38): dprelu[c] = sum over rows of d * (b > 0 ? 0 : b / slope), taken
// BEFORE d is scaled.  One warp per 32 columns and chunk of rows; partial sums meet in dprelu by atomic adds.
__global__ void k_prelu_slope_gradient(const float *__restrict__ b, const float *__restrict__ d, int rows, int N, const float *__restrict__ prelu,
                                       float *__restrict__ dprelu, int rowsPerChunk) {
  const int c = blockIdx.x * 32 + (threadIdx.x & 31);
  const int r0 = blockIdx.y * rowsPerChunk + (threadIdx.x >> 5), r1 = min(rows, (blockIdx.y + 1) * rowsPerChunk);
  if (c >= N) return;
  const float slope = prelu[c];
  float t = 0.f;
  for (int r = r0; r < r1; r += blockDim.x >> 5) {
    const float bv = b[(long long)r * N + c];
    t += d[(long long)r * N + c] * (bv > 0.f ? 0.f : bv / slope);
  }
  atomicAdd(dprelu + c, t);
}

// dW[K x N] = X^T d and dB[N] = column sums of d (NetworkInNetworkLayer.cu:226-239), X being the layer's input: either a
// plain [rows x K] matrix or (GATHER) the convolution's gathered matrix, read through the rulebook as the forward kernel
// reads it (column k = f * nIn + c of row r is input row rules[r * fs + f], channel c; a negative rule is a zero row).
// 64 x 64 output tile per CTA, 4 x 4 per thread, rows split into chunks over gridDim.z whose partial sums meet by atomic adds.
constexpr int BW_T = 64, BW_R = 16;
template <bool GATHER>
__global__ void __launch_bounds__(256) k_backward_weights(const float *__restrict__ in, const int *__restrict__ rules, int rows, int fs, int nIn,
                                                          const float *__restrict__ dout, int N, float *__restrict__ dW, float *__restrict__ dB,
                                                          int rowsPerChunk) {
  __shared__ __align__(16) float As[BW_R][BW_T];
  __shared__ __align__(16) float Ds[BW_R][BW_T];
  const int K = fs * nIn;
  const int k0 = blockIdx.x * BW_T, n0 = blockIdx.y * BW_T;
  const int r0 = blockIdx.z * rowsPerChunk, r1 = min(rows, r0 + rowsPerChunk);
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  float acc[4][4] = {};
  float colsum[4] = {0.f, 0.f, 0.f, 0.f};
  // each thread stages 4 elements of each tile per step: element e = tid + 256 * i -> (row e / 64, column e % 64)
  int kk[4], ff[4], cc[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int e = tid + 256 * i;
    kk[i] = k0 + (e & 63);
    ff[i] = GATHER ? kk[i] / nIn : 0;
    cc[i] = GATHER ? kk[i] - ff[i] * nIn : kk[i];
  }
  for (int rb = r0; rb < r1; rb += BW_R) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + 256 * i, rr = e >> 6, r = rb + rr;
      float a = 0.f, dv = 0.f;
      if (r < r1) {
        if (kk[i] < K) {
          if (GATHER) {
            const int rule = rules[(long long)r * fs + ff[i]];
            if (rule >= 0) a = in[(long long)rule * nIn + cc[i]];
          } else {
            a = in[(long long)r * K + kk[i]];
          }
        }
        const int n = n0 + (e & 63);
        if (n < N) dv = dout[(long long)r * N + n];
      }
      As[rr][e & 63] = a;
      Ds[rr][e & 63] = dv;
    }
    __syncthreads();
#pragma unroll
    for (int rr = 0; rr < BW_R; ++rr) {
      const float4 a = *reinterpret_cast<const float4 *>(&As[rr][ty * 4]);
      const float4 dv = *reinterpret_cast<const float4 *>(&Ds[rr][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, dd[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], dd[j], acc[i][j]);
      if (ty == 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) colsum[j] += dd[j];
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int k = k0 + ty * 4 + i;
    if (k >= K) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) atomicAdd(dW + (long long)k * N + n, acc[i][j]);
    }
  }
  if (blockIdx.x == 0 && ty == 0 && dB) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) atomicAdd(dB + n, colsum[j]);
    }
  }
}

// out[n * K + k] = in[k * N + n]  (32 x 32 tiles through shared memory)
__global__ void k_transpose(const float *__restrict__ in, int K, int N, float *__restrict__ out) {
  __shared__ float tile[32][33];
  const int kb = blockIdx.x * 32, nb = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int k = kb + i, n = nb + threadIdx.x;
    tile[i][threadIdx.x] = (k < K && n < N) ? in[(long long)k * N + n] : 0.f;
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int n = nb + i, k = kb + threadIdx.x;
    if (n < N && k < K) out[(long long)n * K + k] = tile[threadIdx.x][i];
  }
}

// ConvolutionalLayer.cu:42-59: dIn[rules[c]] += dConv[c] for every rule cell c with a non-negative rule; a warp takes
// a cell's nIn channels, consecutive lanes consecutive channels.
__global__ void k_gather_backward(const float *__restrict__ dconv, const int *__restrict__ rules, long long count, int nIn, float *__restrict__ din) {
  const long long total = count * nIn;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long c = i / nIn;
    const int j = (int)(i - c * nIn);
    const int rule = rules[c];
    if (rule >= 0) atomicAdd(din + (long long)rule * nIn + j, dconv[i]);
  }
}

// MaxPoolingLayer.cu:74-80: the pooled gradient goes to the input the forward pass chose (windows may overlap: atomic adds).
__global__ void k_maxpool_backward(const float *__restrict__ dout, const int *__restrict__ choice, long long n, float *__restrict__ din) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int c = choice[i];
    if (c >= 0) atomicAdd(din + c, dout[i]);
  }
}

// TerminalPoolingLayer.cu:48-62: every row a sample pooled receives the sample's gradient divided by their number.
__global__ void k_terminal_pool_backward(const float *__restrict__ dout, const int *__restrict__ rules, int S, int C, float *__restrict__ din) {
  const int b = blockIdx.x;
  int maxP = 0;
  while (maxP < S && rules[(long long)b * S + maxP] >= 0) ++maxP;
  for (int j = threadIdx.x; j < C; j += blockDim.x) {
    const float t = dout[(long long)b * C + j] / maxP;
    for (int p = 0; p < maxP; ++p) din[(long long)rules[(long long)b * S + p] * C + j] = t;
  }
}

// NetworkInNetworkLayer.cu:26-40 ("NAG light"); keepPositive: the PReLU slopes' variant, which holds the result at 0.001 or
// above (NetworkInNetworkPReLULayer.cu:67-84).
__global__ void k_sgd_update(float *__restrict__ w, float *__restrict__ m, const float *__restrict__ d, long long n, float lr, float momentum,
                             int keepPositive) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float wi = w[i], mi = m[i];
    wi -= mi * momentum;
    mi = momentum * mi - lr * (1 - momentum) * d[i];
    wi += mi * (1 + momentum);
    if (keepPositive) wi = wi > 0.001f ? wi : 0.001f;
    w[i] = wi;
    m[i] = mi;
  }
}

// Training-time dropout keeps every matrix at its full width and zeroes the dropped features instead of shrinking
// the matrices to the present ones (NetworkInNetworkLayer.cu:162-186 shrinks): a zero input column contributes nothing
// to a product and a zeroed gradient column gives zero weight gradients, so the numbers that exist in the reference's
// narrow matrices are the same here, and the tensor-core kernels keep their shapes.
// x[r][n] *= mask[n]
__global__ void k_mask_columns(float *__restrict__ x, long long total, int N, const float *__restrict__ mask) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
    if (mask[i % N] == 0.f) x[i] = 0.f;
}
// k_sgd_update on the entries whose input feature (row, mask index row % rowPeriod) and output feature (column) are
// both present: dGradientDescentShrunkMatrix / ...ShrunkVector (NetworkInNetworkLayer.cu:43-81) leave the others, and
// their momentum, untouched.
__global__ void k_sgd_update_masked(float *__restrict__ w, float *__restrict__ m, const float *__restrict__ d, long long n, int N,
                                    const float *__restrict__ rowMask, int rowPeriod, const float *__restrict__ colMask, float lr, float momentum,
                                    int keepPositive) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / N;
    const int col = (int)(i - row * N);
    if (rowMask && rowMask[row % rowPeriod] == 0.f) continue;
    if (colMask && colMask[col] == 0.f) continue;
    float wi = w[i], mi = m[i];
    wi -= mi * momentum;
    mi = momentum * mi - lr * (1 - momentum) * d[i];
    wi += mi * (1 + momentum);
    if (keepPositive) wi = wi > 0.001f ? wi : 0.001f;
    w[i] = wi;
    m[i] = mi;
  }
}

// Index learning (IndexLearnerLayer.cu:57-66, 8-20): a batch uses only the columns of W [K x N] that its own samples
// index.  w[k][j] = W[k][idx[j]] on the way in, W[k][idx[j]] += alpha * d[k][j] on the way out (no momentum).
__global__ void k_gather_columns(const float *__restrict__ W, int K, int N, const int *__restrict__ idx, int n, float *__restrict__ w) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (long long)K * n; i += (long long)gridDim.x * blockDim.x) {
    const long long k = i / n;
    w[i] = W[k * N + idx[i - k * n]];
  }
}
__global__ void k_scatter_columns_axpy(float *__restrict__ W, int K, int N, const int *__restrict__ idx, int n, const float *__restrict__ d, float alpha) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (long long)K * n; i += (long long)gridDim.x * blockDim.x) {
    const long long k = i / n;
    W[k * N + idx[i - k * n]] += alpha * d[i]; // (the indices of a batch are distinct: no two threads share an element)
  }
}

// ---- the weight gradient on the tensor cores: dW[K x N] = Xg^T[K x rows] * d[rows x N] is the forward kernel's product with
// the roles turned: its "rows" are the K gathered input channels, its contraction runs over the layer's rows, its
// "weights" are the output gradient.  The gathered input is written once, transposed ([Kp x rowsP], Kp and rowsP padded
// with zeros to whole tiles and whole slabs), the gradient is packed like a weight matrix, and the fused kernel
// (three tf32 products, K split over the CTAs, partial sums added in a fixed order) does the rest.
constexpr int GT_TILE = 32;
// out[k][r] = X[r][k] for the gathered input X (row r of a convolution's input matrix: cell f = k / nIn of the rule row,
// channel k % nIn), zero where the rule is negative and in the padding.  32 x 32 tiles through shared memory: reads run
// along the channels, writes along the rows.
__global__ void __launch_bounds__(256) k_gather_transpose(const float *__restrict__ in, const int *__restrict__ rules, int rows, int fs, int nIn,
                                                          int K, int rowsP, float *__restrict__ out) {
  __shared__ float tile[GT_TILE][GT_TILE + 1];
  const int tx = threadIdx.x, ty = threadIdx.y; // 32 x 8
  const long long r0 = (long long)blockIdx.x * GT_TILE;
  const int k0 = blockIdx.y * GT_TILE;
  const int k = k0 + tx;
  const int f = k < K ? k / nIn : 0, c = k - f * nIn;
#pragma unroll
  for (int j = 0; j < GT_TILE; j += 8) {
    const long long r = r0 + ty + j;
    float v = 0.f;
    if (r < rows && k < K) {
      const int src = rules ? __ldg(rules + r * fs + f) : (int)r;
      if (src >= 0) v = __ldg(in + (long long)src * nIn + c);
    }
    tile[ty + j][tx] = v;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < GT_TILE; j += 8) {
    const int kk = k0 + ty + j;
    out[(long long)kk * rowsP + r0 + tx] = tile[tx][ty + j]; // (the grid covers exactly Kp x rowsP)
  }
}
// db[n] += sum over a chunk of rows of d[r][n]
__global__ void __launch_bounds__(256) k_column_sums(const float *__restrict__ d, int rows, int N, int rowsPerChunk, float *__restrict__ db) {
  __shared__ float part[8][33];
  const int tx = threadIdx.x, ty = threadIdx.y, n = blockIdx.x * 32 + tx;
  const long long rBegin = (long long)blockIdx.y * rowsPerChunk, rEnd = min((long long)rows, rBegin + rowsPerChunk);
  float acc = 0.f;
  if (n < N)
    for (long long r = rBegin + ty; r < rEnd; r += 8) acc += __ldg(d + r * N + n);
  part[ty][tx] = acc;
  __syncthreads();
  if (ty == 0 && n < N) {
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) sum += part[j][tx];
    atomicAdd(db + n, sum);
  }
}
struct WeightGradPlan { int K, Kp, rowsP; size_t gatheredBytes, packedBytes, splitBytes, biasBytes, outBytes, total; bool ok; };
WeightGradPlan plan_weight_grad(int rows, int fs, int nIn, int N) {
  WeightGradPlan p = {};
  p.K = fs * nIn;
  p.Kp = (p.K + 127) / 128 * 128;
  p.rowsP = (rows + 31) / 32 * 32;
  p.ok = rows >= 128 && N >= 16 && N % 4 == 0 && (long long)p.Kp * p.rowsP < (1ll << 40);
  if (!p.ok) return p;
  p.gatheredBytes = align_up(sizeof(float) * (size_t)p.Kp * p.rowsP, 256);
  p.packedBytes = align_up(tc_packed_bytes(rows, N, SCN_PREC_3XTF32), 256);
  p.splitBytes = align_up(tc_workspace_bytes(p.Kp, 1, p.rowsP, N, SCN_PREC_3XTF32), 256);
  p.biasBytes = align_up(sizeof(float) * (size_t)N, 256);
  p.outBytes = p.Kp == p.K ? 0 : align_up(sizeof(float) * (size_t)p.Kp * N, 256); // the product's rows for the padded channels need a place
  p.ok = p.packedBytes > 0;
  p.total = p.gatheredBytes + p.packedBytes + p.splitBytes + p.biasBytes + p.outBytes;
  return p;
}
} // namespace
} // namespace scn

using namespace scn;

extern "C" int scn_softmax_nll_backward(const float *d_probs, const int *d_labels, int rows, int nClasses, float *d_dfeatures, scn_stream_t stream) {
  clear_error();
  if (rows < 0 || nClasses < 1) return fail(SCN_ERR_INVALID, "bad softmax sizes");
  if (rows == 0) return SCN_OK;
  if (!d_probs || !d_labels || !d_dfeatures) return fail(SCN_ERR_INVALID, "null pointer");
  const long long n = (long long)rows * nClasses;
  k_softmax_nll_backward<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(d_probs, d_labels, n, nClasses, d_dfeatures);
  SCN_LAUNCH_CHECK("k_softmax_nll_backward");
  return SCN_OK;
}

extern "C" int scn_activation_backward(const float *d_out_features, float *d_dfeatures, int rows, int N, int act, const float *d_prelu,
                                       float *d_dprelu, scn_stream_t stream) {
  clear_error();
  if (rows < 0 || N < 1) return fail(SCN_ERR_INVALID, "bad activation sizes");
  if (act < SCN_NOSIGMOID || act > SCN_SIGMOID) return fail(SCN_ERR_INVALID, "unknown activation");
  if (act == SCN_PRELU && (!d_prelu || !d_dprelu)) return fail(SCN_ERR_INVALID, "PReLU needs its slopes and a place for their gradient");
  if (rows == 0 || act == SCN_NOSIGMOID || act == SCN_SOFTMAX) return SCN_OK; // softmax: the classifier's gradient is already taken at its input
  if (!d_out_features || !d_dfeatures) return fail(SCN_ERR_INVALID, "null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  if (act == SCN_PRELU) {
    SCN_CUDA_TRY(cudaMemsetAsync(d_dprelu, 0, sizeof(float) * N, s));
    const int chunks = std::max(1, std::min((rows + 63) / 64, 4 * sm_count() / ((N + 31) / 32) + 1));
    const int rowsPerChunk = (rows + chunks - 1) / chunks;
    k_prelu_slope_gradient<<<dim3((N + 31) / 32, chunks), 256, 0, s>>>(d_out_features, d_dfeatures, rows, N, d_prelu, d_dprelu, rowsPerChunk);
    SCN_LAUNCH_CHECK("k_prelu_slope_gradient");
  }
  const long long n = (long long)rows * N;
  const bool vec = N % 4 == 0 && (((uintptr_t)d_out_features | (uintptr_t)d_dfeatures | (uintptr_t)d_prelu) & 15) == 0;
  if (vec) { SCN_DISPATCH_ACT(act, (k_activation_backward<ACT><<<grid_for(n / 4, 256), 256, 0, s>>>(d_out_features, d_dfeatures, n / 4, d_prelu, N))); }
  else { SCN_DISPATCH_ACT(act, (k_activation_backward_scalar<ACT><<<grid_for(n, 256), 256, 0, s>>>(d_out_features, d_dfeatures, n, d_prelu, N))); }
  SCN_LAUNCH_CHECK("k_activation_backward");
  return SCN_OK;
}

extern "C" int scn_conv_nin_backward_weights(const float *d_in, const int *d_rules, int rows, int fs, int nIn, const float *d_dout, int N,
                                             float *d_dW, float *d_dB, scn_stream_t stream) {
  clear_error();
  if (rows < 0 || fs < 1 || nIn < 1 || N < 1) return fail(SCN_ERR_INVALID, "bad conv/NiN sizes");
  if (!d_rules && fs != 1) return fail(SCN_ERR_INVALID, "fs must be 1 without rules");
  if (!d_dW) return fail(SCN_ERR_INVALID, "null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const int K = fs * nIn;
  SCN_CUDA_TRY(cudaMemsetAsync(d_dW, 0, sizeof(float) * (size_t)K * N, s));
  if (d_dB) SCN_CUDA_TRY(cudaMemsetAsync(d_dB, 0, sizeof(float) * N, s));
  if (rows == 0) return SCN_OK;
  if (!d_in || !d_dout) return fail(SCN_ERR_INVALID, "null pointer");
  const int tk = (K + BW_T - 1) / BW_T, tn = (N + BW_T - 1) / BW_T;
  int chunks = std::max(1, 6 * sm_count() / (tk * tn));
  chunks = std::min(chunks, (rows + 4 * BW_R - 1) / (4 * BW_R));
  chunks = std::max(1, std::min(chunks, 65535));
  int rowsPerChunk = (rows + chunks - 1) / chunks;
  rowsPerChunk = (rowsPerChunk + BW_R - 1) / BW_R * BW_R;
  chunks = (rows + rowsPerChunk - 1) / rowsPerChunk;
  const dim3 grid(tk, tn, chunks);
  if (d_rules) k_backward_weights<true><<<grid, 256, 0, s>>>(d_in, d_rules, rows, fs, nIn, d_dout, N, d_dW, d_dB, rowsPerChunk);
  else k_backward_weights<false><<<grid, 256, 0, s>>>(d_in, nullptr, rows, 1, nIn, d_dout, N, d_dW, d_dB, rowsPerChunk);
  SCN_LAUNCH_CHECK("k_backward_weights");
  return SCN_OK;
}


extern "C" size_t scn_conv_nin_backward_weights_tc_bytes(int rows, int fs, int nIn, int N) {
  if (rows < 1 || fs < 1 || nIn < 1 || N < 1) return 0;
  const WeightGradPlan p = plan_weight_grad(rows, fs, nIn, N);
  return p.ok ? p.total : 0;
}

extern "C" int scn_conv_nin_backward_weights_tc(const float *d_in, const int *d_rules, int rows, int fs, int nIn, const float *d_dout, int N,
                                                float *d_dW, float *d_dB, void *d_workspace, size_t workspace_bytes, scn_stream_t stream) {
  clear_error();
  if (rows < 1 || fs < 1 || nIn < 1 || N < 1) return fail(SCN_ERR_INVALID, "bad conv/NiN sizes");
  if (!d_rules && fs != 1) return fail(SCN_ERR_INVALID, "fs must be 1 without rules");
  if (!d_in || !d_dout || !d_dW || !d_workspace) return fail(SCN_ERR_INVALID, "null pointer");
  const WeightGradPlan p = plan_weight_grad(rows, fs, nIn, N);
  if (!p.ok) return fail(SCN_ERR_UNSUPPORTED, "weight gradient: shape not taken by the tensor-core form (few rows, or N not a multiple of 4 or below 16)");
  if (workspace_bytes < p.total) return fail(SCN_ERR_WORKSPACE, "workspace smaller than scn_conv_nin_backward_weights_tc_bytes()");
  if (((uintptr_t)d_workspace | (uintptr_t)d_dout | (uintptr_t)d_dW) & 15) return fail(SCN_ERR_INVALID, "weight gradient: buffers must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  char *w = (char *)d_workspace;
  float *gatheredT = (float *)w;
  void *packed = w + p.gatheredBytes;
  void *split = p.splitBytes ? w + p.gatheredBytes + p.packedBytes : nullptr;
  float *zeroBias = (float *)(w + p.gatheredBytes + p.packedBytes + p.splitBytes);
  SCN_CUDA_TRY(cudaMemsetAsync(zeroBias, 0, sizeof(float) * N, s));
  k_gather_transpose<<<dim3(p.rowsP / GT_TILE, p.Kp / GT_TILE), dim3(32, 8), 0, s>>>(d_in, d_rules, rows, fs, nIn, p.K, p.rowsP, gatheredT);
  SCN_LAUNCH_CHECK("k_gather_transpose");
  int rc = tc_pack(d_dout, rows, N, SCN_PREC_3XTF32, packed, s);
  if (rc != SCN_OK) return rc;
  // "rows" = Kp input channels (whole tiles: no tile row is missing), one "input row" per channel of length rowsP
  float *product = p.outBytes ? (float *)(w + p.gatheredBytes + p.packedBytes + p.splitBytes + p.biasBytes) : d_dW;
  rc = tc_launch(gatheredT, nullptr, p.Kp, 1, p.rowsP, packed, zeroBias, nullptr, N, 1.0f, SCN_NOSIGMOID, SCN_PREC_3XTF32, product, split, p.splitBytes, s);
  if (rc == SCN_OK && p.outBytes) SCN_CUDA_TRY(cudaMemcpyAsync(d_dW, product, sizeof(float) * (size_t)p.K * N, cudaMemcpyDeviceToDevice, s));
  if (rc != SCN_OK) return rc;
  if (d_dB) {
    SCN_CUDA_TRY(cudaMemsetAsync(d_dB, 0, sizeof(float) * N, s));
    int chunks = std::max(1, std::min(4 * sm_count() / std::max(1, (N + 31) / 32), (rows + 255) / 256));
    const int rowsPerChunk = (rows + chunks - 1) / chunks;
    chunks = (rows + rowsPerChunk - 1) / rowsPerChunk;
    k_column_sums<<<dim3((N + 31) / 32, chunks), dim3(32, 8), 0, s>>>(d_dout, rows, N, rowsPerChunk, d_dB);
    SCN_LAUNCH_CHECK("k_column_sums");
  }
  return SCN_OK;
}

extern "C" int scn_transpose_weights(const float *d_W, int K, int N, float *d_Wt, scn_stream_t stream) {
  clear_error();
  if (K < 1 || N < 1 || !d_W || !d_Wt) return fail(SCN_ERR_INVALID, "bad transpose arguments");
  k_transpose<<<dim3((K + 31) / 32, (N + 31) / 32), dim3(32, 8), 0, (cudaStream_t)stream>>>(d_W, K, N, d_Wt);
  SCN_LAUNCH_CHECK("k_transpose");
  return SCN_OK;
}

extern "C" int scn_gather_backward(const float *d_dconv, const int *d_rules, long long count, int nIn, float *d_din, long long rows_in,
                                   scn_stream_t stream) {
  clear_error();
  if (count < 0 || nIn < 1 || rows_in < 0) return fail(SCN_ERR_INVALID, "bad gather sizes");
  cudaStream_t s = (cudaStream_t)stream;
  if (rows_in > 0) {
    if (!d_din) return fail(SCN_ERR_INVALID, "null pointer");
    SCN_CUDA_TRY(cudaMemsetAsync(d_din, 0, sizeof(float) * (size_t)rows_in * nIn, s));
  }
  if (count == 0) return SCN_OK;
  if (!d_dconv || !d_rules || !d_din) return fail(SCN_ERR_INVALID, "null pointer");
  k_gather_backward<<<grid_for(count * nIn, 256), 256, 0, s>>>(d_dconv, d_rules, count, nIn, d_din);
  SCN_LAUNCH_CHECK("k_gather_backward");
  return SCN_OK;
}

extern "C" int scn_maxpool_backward(const float *d_dout, const int *d_choices, long long n, float *d_din, long long n_in, scn_stream_t stream) {
  clear_error();
  if (n < 0 || n_in < 0) return fail(SCN_ERR_INVALID, "bad pooling sizes");
  cudaStream_t s = (cudaStream_t)stream;
  if (n_in > 0) {
    if (!d_din) return fail(SCN_ERR_INVALID, "null pointer");
    SCN_CUDA_TRY(cudaMemsetAsync(d_din, 0, sizeof(float) * (size_t)n_in, s));
  }
  if (n == 0) return SCN_OK;
  if (!d_dout || !d_choices || !d_din) return fail(SCN_ERR_INVALID, "null pointer");
  k_maxpool_backward<<<grid_for(n, 256), 256, 0, s>>>(d_dout, d_choices, n, d_din);
  SCN_LAUNCH_CHECK("k_maxpool_backward");
  return SCN_OK;
}

extern "C" int scn_terminal_pool_backward(const float *d_dout, const int *d_rules, int batch, int S, int C, float *d_din, long long rows_in,
                                          scn_stream_t stream) {
  clear_error();
  if (batch < 0 || S < 1 || C < 1 || rows_in < 0) return fail(SCN_ERR_INVALID, "bad terminal pooling sizes");
  cudaStream_t s = (cudaStream_t)stream;
  if (rows_in > 0) {
    if (!d_din) return fail(SCN_ERR_INVALID, "null pointer");
    SCN_CUDA_TRY(cudaMemsetAsync(d_din, 0, sizeof(float) * (size_t)rows_in * C, s));
  }
  if (batch == 0) return SCN_OK;
  if (!d_dout || !d_rules || !d_din) return fail(SCN_ERR_INVALID, "null pointer");
  k_terminal_pool_backward<<<batch, 128, 0, s>>>(d_dout, d_rules, S, C, d_din);
  SCN_LAUNCH_CHECK("k_terminal_pool_backward");
  return SCN_OK;
}

extern "C" int scn_sgd_update(float *d_w, float *d_momentum, const float *d_delta, long long n, float learningRate, float momentum,
                              int keep_positive, scn_stream_t stream) {
  clear_error();
  if (n < 0) return fail(SCN_ERR_INVALID, "bad size");
  if (n == 0) return SCN_OK;
  if (!d_w || !d_momentum || !d_delta) return fail(SCN_ERR_INVALID, "null pointer");
  k_sgd_update<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(d_w, d_momentum, d_delta, n, learningRate, momentum, keep_positive);
  SCN_LAUNCH_CHECK("k_sgd_update");
  return SCN_OK;
}


extern "C" int scn_mask_columns(float *d_x, long long rows, int N, const float *d_mask, scn_stream_t stream) {
  clear_error();
  if (rows < 0 || N < 1) return fail(SCN_ERR_INVALID, "bad mask sizes");
  if (rows == 0) return SCN_OK;
  if (!d_x || !d_mask) return fail(SCN_ERR_INVALID, "null pointer");
  k_mask_columns<<<grid_for(rows * N, 256), 256, 0, (cudaStream_t)stream>>>(d_x, rows * N, N, d_mask);
  SCN_LAUNCH_CHECK("k_mask_columns");
  return SCN_OK;
}

extern "C" int scn_sgd_update_masked(float *d_w, float *d_momentum, const float *d_delta, long long rows, int N, const float *d_row_mask,
                                     int row_period, const float *d_col_mask, float learningRate, float momentum, int keep_positive,
                                     scn_stream_t stream) {
  clear_error();
  if (rows < 0 || N < 1 || (d_row_mask && row_period < 1)) return fail(SCN_ERR_INVALID, "bad update sizes");
  if (rows == 0) return SCN_OK;
  if (!d_w || !d_momentum || !d_delta) return fail(SCN_ERR_INVALID, "null pointer");
  k_sgd_update_masked<<<grid_for(rows * N, 256), 256, 0, (cudaStream_t)stream>>>(d_w, d_momentum, d_delta, rows * N, N, d_row_mask,
                                                                                 d_row_mask ? row_period : 1, d_col_mask, learningRate, momentum,
                                                                                 keep_positive);
  SCN_LAUNCH_CHECK("k_sgd_update_masked");
  return SCN_OK;
}


extern "C" int scn_gather_columns(const float *d_W, int K, int N, const int *d_idx, int n, float *d_w, scn_stream_t stream) {
  clear_error();
  if (K < 1 || N < 1 || n < 0) return fail(SCN_ERR_INVALID, "bad column-gather sizes");
  if (n == 0) return SCN_OK;
  if (!d_W || !d_idx || !d_w) return fail(SCN_ERR_INVALID, "null pointer");
  k_gather_columns<<<grid_for((long long)K * n, 256), 256, 0, (cudaStream_t)stream>>>(d_W, K, N, d_idx, n, d_w);
  SCN_LAUNCH_CHECK("k_gather_columns");
  return SCN_OK;
}

extern "C" int scn_scatter_columns_axpy(float *d_W, int K, int N, const int *d_idx, int n, const float *d_delta, float alpha, scn_stream_t stream) {
  clear_error();
  if (K < 1 || N < 1 || n < 0) return fail(SCN_ERR_INVALID, "bad column-scatter sizes");
  if (n == 0) return SCN_OK;
  if (!d_W || !d_idx || !d_delta) return fail(SCN_ERR_INVALID, "null pointer");
  k_scatter_columns_axpy<<<grid_for((long long)K * n, 256), 256, 0, (cudaStream_t)stream>>>(d_W, K, N, d_idx, n, d_delta, alpha);
  SCN_LAUNCH_CHECK("k_scatter_columns_axpy");
  return SCN_OK;
}
