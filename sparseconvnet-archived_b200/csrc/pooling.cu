// Rule-driven pooling and the small row-wise kernels of the forward path.  All of them are
// HBM-bound: each input element is read once per rule that names it, every output element
// is written once, accesses are coalesced along the channel axis (float4 where C % 4 == 0).
#include "scn_common.cuh"
#include "conv_nin_tc.cuh"
#include <type_traits>

namespace scn {
namespace {

// Max pooling with argmax (MaxPoolingLayer.cu:9-35): negative rules are skipped, the first
// maximum wins (strict '<'), the choice is the flat input index rule*C + channel.
template <int VEC>
__global__ void k_maxpool(const float *__restrict__ in, const int *__restrict__ rules, int rowsOut, int sd, int C,
                          float *__restrict__ out, int *__restrict__ choice) {
  dependents_may_launch();
  wait_for_prior_grids(); // the features come from the kernel in front
  const int cv = C / VEC;
  const long long n = (long long)rowsOut * cv;
  for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < n; q += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(q / cv), j = (int)(q % cv) * VEC;
    float best[VEC];
    int idx[VEC];
    bool none = true;
#pragma unroll
    for (int v = 0; v < VEC; ++v) { best[v] = 0.f; idx[v] = -1; }
    if (VEC == 4 && sd <= 8) {
      // small windows: all rules, then all cells, are requested before the first comparison (two round trips to
      // memory instead of two per cell); a missing cell reads the row of a cell that is there and is skipped
      auto window = [&](auto widthC) {
        constexpr int WIDTH = decltype(widthC)::value;
        int rp[WIDTH], safe = -1;
#pragma unroll
        for (int p = 0; p < WIDTH; ++p) { rp[p] = p < sd ? __ldg(rules + (long long)r * sd + p) : -1; safe = max(safe, rp[p]); }
        if (safe < 0) return;
        float4 t[WIDTH];
#pragma unroll
        for (int p = 0; p < WIDTH; ++p) t[p] = *reinterpret_cast<const float4 *>(in + (long long)(rp[p] >= 0 ? rp[p] : safe) * C + j);
#pragma unroll
        for (int p = 0; p < WIDTH; ++p) {
          if (rp[p] < 0) continue;
          const float s[4] = {t[p].x, t[p].y, t[p].z, t[p].w};
          const long long base = (long long)rp[p] * C + j;
#pragma unroll
          for (int v = 0; v < 4; ++v)
            if (none || best[v % VEC] < s[v]) { best[v % VEC] = s[v]; idx[v % VEC] = (int)(base + v); }
          none = false;
        }
      };
      if (sd <= 4) window(std::integral_constant<int, 4>());
      else window(std::integral_constant<int, 8>());
    } else
    for (int p = 0; p < sd; ++p) {
      const int rp = __ldg(rules + (long long)r * sd + p);
      if (rp < 0) continue;
      float s[VEC];
      const long long base = (long long)rp * C + j;
      if (VEC == 4) { float4 t = *reinterpret_cast<const float4 *>(in + base); s[0] = t.x; s[1 % VEC] = t.y; s[2 % VEC] = t.z; s[3 % VEC] = t.w; }
      else { s[0] = in[base]; }
#pragma unroll
      for (int v = 0; v < VEC; ++v)
        if (none || best[v] < s[v]) { best[v] = s[v]; idx[v] = (int)(base + v); }
      none = false;
    }
    const long long o = (long long)r * C + j;
    if (VEC == 4) {
      *reinterpret_cast<float4 *>(out + o) = make_float4(best[0], best[1 % VEC], best[2 % VEC], best[3 % VEC]);
      *reinterpret_cast<int4 *>(choice + o) = make_int4(idx[0], idx[1 % VEC], idx[2 % VEC], idx[3 % VEC]);
    } else { out[o] = best[0]; choice[o] = idx[0]; }
  }
}

// Mean over each row's rules up to the first negative one (TerminalPoolingLayer.cu:22-34).
__global__ void k_terminal_pool(const float *__restrict__ in, const int *__restrict__ rules, int batch, int S, int C,
                                float *__restrict__ out) {
  const long long n = (long long)batch * C;
  for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < n; q += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(q / C), j = (int)(q % C);
    float t = 0.f;
    int p = 0;
    for (; p < S; ++p) {
      const int rp = __ldg(rules + (long long)b * S + p);
      if (rp < 0) break;
      t += in[(long long)rp * C + j];
    }
    out[q] = t / p;
  }
}

// propForwardToMatrixMultiply (ConvolutionalLayer.cu:12-31), a negative rule giving zeros.
__global__ void k_gather(const float *__restrict__ in, const int *__restrict__ rules, long long count, int nIn,
                         float *__restrict__ out) {
  const long long n = count * nIn;
  for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < n; q += (long long)gridDim.x * blockDim.x) {
    const long long c = q / nIn;
    const int j = (int)(q % nIn);
    const int r = __ldg(rules + c);
    out[q] = r >= 0 ? in[(long long)r * nIn + j] : 0.f;
  }
}

// vectorTopIndices (utilities.cu:35-56): descending values, equal values in index order.  One warp per
// row: every lane finds the best eligible entry of its stride, a shuffle reduction picks the largest value
// (the smaller index on a tie).
__global__ void k_top_indices(const float *__restrict__ probs, int rows, int nClasses, int nTop, int *__restrict__ top) {
  const int lane = threadIdx.x & 31;
  for (int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += gridDim.x * (blockDim.x >> 5)) {
    const float *v = probs + (long long)r * nClasses;
    float lastVal = 0.f;
    int lastIdx = -1;
    for (int t = 0; t < nTop; ++t) {
      int best = -1;
      float bv = 0.f;
      for (int i = lane; i < nClasses; i += 32) {
        const float x = v[i];
        const bool eligible = (lastIdx < 0) || x < lastVal || (x == lastVal && i > lastIdx);
        if (eligible && (best < 0 || x > bv)) { best = i; bv = x; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best, o);
        if (oi >= 0 && (best < 0 || ov > bv || (ov == bv && oi < best))) { best = oi; bv = ov; }
      }
      if (lane == 0) top[(long long)r * nTop + t] = best < 0 ? 0 : best;
      lastVal = bv; lastIdx = best;
    }
  }
}

// What the classifier's caller reads back, as one block: the probabilities, the nTop classes of every row and the
// error word of the tensor-core kernels (taken: the word is cleared).  Same selection as k_top_indices.
__global__ void k_classifier_result(const float *__restrict__ probs, int rows, int nClasses, int nTop, float *__restrict__ blockProbs,
                                    int *__restrict__ blockTop, int *__restrict__ blockFlag, int *tcError) {
  const int lane = threadIdx.x & 31;
  if (blockIdx.x == 0 && threadIdx.x == 0) *blockFlag = tcError ? atomicExch(tcError, 0) : 0;
  for (int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += gridDim.x * (blockDim.x >> 5)) {
    const float *v = probs + (long long)r * nClasses;
    for (int i = lane; i < nClasses; i += 32) blockProbs[(long long)r * nClasses + i] = v[i];
    float lastVal = 0.f;
    int lastIdx = -1;
    for (int t = 0; t < nTop; ++t) {
      int best = -1;
      float bv = 0.f;
      for (int i = lane; i < nClasses; i += 32) {
        const float x = v[i];
        const bool eligible = (lastIdx < 0) || x < lastVal || (x == lastVal && i > lastIdx);
        if (eligible && (best < 0 || x > bv)) { best = i; bv = x; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best, o);
        if (oi >= 0 && (best < 0 || ov > bv || (ov == bv && oi < best))) { best = oi; bv = ov; }
      }
      if (lane == 0) blockTop[(long long)r * nTop + t] = best < 0 ? 0 : best;
      lastVal = bv; lastIdx = best;
    }
  }
}

// Background row of each sample: the row whose key is negative (at most one per sample), -1 if
// none.  One warp per sample.
__global__ void k_background_rows(const int *__restrict__ keys, const int *__restrict__ off, int batch, int *__restrict__ bg) {
  const int lane = threadIdx.x & 31;
  for (int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); b < batch; b += gridDim.x * (blockDim.x >> 5)) {
    int found = -1;
    for (int r = off[b] + lane; r < off[b + 1]; r += 32)
      if (keys[r] < 0) found = r;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) found = max(found, __shfl_xor_sync(0xffffffffu, found, o));
    if (lane == 0) bg[b] = found;
  }
}

// applySigmoid as a stand-alone elementwise pass (SigmoidLayer.cu:187-222).
__global__ void k_activation(const float *__restrict__ in, float *__restrict__ out, long long n, int N, int act,
                             const float *__restrict__ prelu) {
  for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < n; q += (long long)gridDim.x * blockDim.x)
    out[q] = activate(in[q], act, prelu ? prelu[q % N] : 0.f);
}
// Row softmax (SigmoidLayer.cu:160-177), one thread per row.
__global__ void k_softmax(const float *__restrict__ in, float *__restrict__ out, int rows, int N) {
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += gridDim.x * blockDim.x) {
    const float *a = in + (long long)r * N;
    float *b = out + (long long)r * N;
    float mx = -10000.0f, acc = 0.0f;
    for (int k = 0; k < N; ++k) if (a[k] > mx) mx = a[k];
    for (int k = 0; k < N; ++k) { b[k] = expf(a[k] - mx); acc += b[k]; }
    for (int k = 0; k < N; ++k) b[k] /= acc;
  }
}

} // namespace
} // namespace scn

using namespace scn;

extern "C" int scn_background_rows(const int *d_keys, const int *d_off, int batch, int *d_bg, scn_stream_t stream) {
  clear_error();
  if (batch < 1 || !d_off || !d_bg) return fail(SCN_ERR_INVALID, "bad arguments");
  k_background_rows<<<grid_for((long long)batch * 32, 256), 256, 0, (cudaStream_t)stream>>>(d_keys, d_off, batch, d_bg);
  SCN_LAUNCH_CHECK("k_background_rows");
  return SCN_OK;
}

extern "C" int scn_activation_forward(const float *d_in, float *d_out, int rows, int N, int act, const float *d_prelu,
                                      scn_stream_t stream) {
  clear_error();
  if (rows < 0 || N < 1 || act < SCN_NOSIGMOID || act > SCN_SIGMOID) return fail(SCN_ERR_INVALID, "bad activation arguments");
  if (act == SCN_PRELU && !d_prelu) return fail(SCN_ERR_INVALID, "PReLU slopes missing");
  if (rows == 0) return SCN_OK;
  if (!d_in || !d_out) return fail(SCN_ERR_INVALID, "null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  if (act == SCN_SOFTMAX) k_softmax<<<grid_for(rows, 128), 128, 0, s>>>(d_in, d_out, rows, N);
  else k_activation<<<grid_for((long long)rows * N, 256), 256, 0, s>>>(d_in, d_out, (long long)rows * N, N, act, d_prelu);
  SCN_LAUNCH_CHECK("k_activation");
  return SCN_OK;
}

extern "C" int scn_maxpool_forward(const float *d_in, const int *d_rules, int rows_out, int sd, int C, float *d_out,
                                   int *d_choices, scn_stream_t stream) {
  clear_error();
  if (rows_out < 0 || sd < 1 || C < 1) return fail(SCN_ERR_INVALID, "bad max-pooling sizes");
  if (rows_out == 0) return SCN_OK;
  if (!d_in || !d_rules || !d_out || !d_choices) return fail(SCN_ERR_INVALID, "null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const bool vec = (C % 4 == 0) && ((uintptr_t)d_in % 16 == 0) && ((uintptr_t)d_out % 16 == 0) && ((uintptr_t)d_choices % 16 == 0);
  if (vec) (void)launch_dependent(k_maxpool<4>, dim3(grid_for((long long)rows_out * (C / 4), 256)), dim3(256), (size_t)0, s, d_in, d_rules, rows_out, sd, C, d_out, d_choices);
  else (void)launch_dependent(k_maxpool<1>, dim3(grid_for((long long)rows_out * C, 256)), dim3(256), (size_t)0, s, d_in, d_rules, rows_out, sd, C, d_out, d_choices);
  SCN_LAUNCH_CHECK("k_maxpool");
  return SCN_OK;
}

extern "C" int scn_terminal_pool_forward(const float *d_in, const int *d_rules, int batch, int S, int C, float *d_out,
                                         scn_stream_t stream) {
  clear_error();
  if (batch < 0 || S < 1 || C < 1) return fail(SCN_ERR_INVALID, "bad terminal-pooling sizes");
  if (batch == 0) return SCN_OK;
  if (!d_in || !d_rules || !d_out) return fail(SCN_ERR_INVALID, "null pointer");
  k_terminal_pool<<<grid_for((long long)batch * C, 128), 128, 0, (cudaStream_t)stream>>>(d_in, d_rules, batch, S, C, d_out);
  SCN_LAUNCH_CHECK("k_terminal_pool");
  return SCN_OK;
}

extern "C" int scn_gather_forward(const float *d_in, const int *d_rules, long long count, int nIn, float *d_out,
                                  scn_stream_t stream) {
  clear_error();
  if (count < 0 || nIn < 1) return fail(SCN_ERR_INVALID, "bad gather sizes");
  if (count == 0) return SCN_OK;
  if (!d_in || !d_rules || !d_out) return fail(SCN_ERR_INVALID, "null pointer");
  k_gather<<<grid_for(count * nIn, 256), 256, 0, (cudaStream_t)stream>>>(d_in, d_rules, count, nIn, d_out);
  SCN_LAUNCH_CHECK("k_gather");
  return SCN_OK;
}

extern "C" size_t scn_classifier_result_bytes(int rows, int nClasses, int nTop) {
  if (rows < 0 || nClasses < 1 || nTop < 1) return 0;
  return sizeof(float) * (size_t)rows * nClasses + sizeof(int) * (size_t)rows * nTop + sizeof(int);
}

extern "C" int scn_classifier_result(const float *d_probs, int rows, int nClasses, int nTop, void *d_block, scn_stream_t stream) {
  clear_error();
  if (rows < 1 || nClasses < 1 || nTop < 1 || nTop > nClasses) return fail(SCN_ERR_INVALID, "need rows >= 1 and 1 <= nTop <= nClasses");
  if (!d_probs || !d_block) return fail(SCN_ERR_INVALID, "null pointer");
  float *bp = (float *)d_block;
  int *bt = (int *)(bp + (size_t)rows * nClasses);
  k_classifier_result<<<grid_for((long long)rows * 32, 128), 128, 0, (cudaStream_t)stream>>>(d_probs, rows, nClasses, nTop, bp, bt, bt + (size_t)rows * nTop,
                                                                                             tc_error_word());
  SCN_LAUNCH_CHECK("k_classifier_result");
  return SCN_OK;
}

extern "C" int scn_top_indices(const float *d_probs, int rows, int nClasses, int nTop, int *d_top, scn_stream_t stream) {
  clear_error();
  if (rows < 0 || nClasses < 1 || nTop < 1 || nTop > nClasses) return fail(SCN_ERR_INVALID, "need 1 <= nTop <= nClasses");
  if (rows == 0) return SCN_OK;
  if (!d_probs || !d_top) return fail(SCN_ERR_INVALID, "null pointer");
  k_top_indices<<<grid_for((long long)rows * 32, 128), 128, 0, (cudaStream_t)stream>>>(d_probs, rows, nClasses, nTop, d_top);
  SCN_LAUNCH_CHECK("k_top_indices");
  return SCN_OK;
}
