#include "utilities.h"
#include "types.h"
#include <algorithm>
#include <cmath>
#include <cstring>

const char *batchTypeNames[] = {"TRAINBATCH", "TESTBATCH", "UNLABELEDBATCH", "RESCALEBATCH"};
const char *sigmoidNames[] = {"", "ReLU", "VeryLeakyReLU", "LeakyReLU", "tanh", "Softmax Classification", "PReLU", "Sigmoid"};
__int128_t multiplyAddCount = 0;

std::vector<int> range(int n) {
  std::vector<int> r(n);
  for (int i = 0; i < n; ++i) r[i] = i;
  return r;
}
int ipow(int base, int exp) {
  int r = 1;
  for (; exp; exp >>= 1, base *= base)
    if (exp & 1) r *= base;
  return r;
}
int triangleSize(int linearSize, int dimension) {
  int fs = 1;
  for (int i = 1; i <= dimension; ++i) fs = fs * (linearSize + dimension - i) / i;
  return fs;
}
int intRoundUp(int a, int d) { return ((a + d - 1) / d) * d; }
int intRound(int a, int d) { return (int)(std::round(a * 1.0 / d) * d); }

// Insertion top-k with strict comparisons: descending values, equal values keep index order.
template <typename t> std::vector<int> vectorTopIndices(std::vector<t> &test, int k) {
  std::vector<int> idx(k, 0);
  std::vector<t> best(k);
  int filled = 0;
  for (int i = 0; i < (int)test.size(); ++i) {
    int pos = filled;
    while (pos > 0 && test[i] > best[pos - 1]) --pos;
    if (pos >= k) continue;
    int last = std::min(filled, k - 1);
    for (int q = last; q > pos; --q) { best[q] = best[q - 1]; idx[q] = idx[q - 1]; }
    best[pos] = test[i]; idx[pos] = i;
    if (filled < k) ++filled;
  }
  return idx;
}
template std::vector<int> vectorTopIndices<float>(std::vector<float> &, int);

void scnCheckCuda(cudaError_t err, const char *file, int line) {
  if (err != cudaSuccess)
    throw ScnException(std::string("CUDA error: ") + cudaGetErrorString(err) + " at " + file + ":" + std::to_string(line));
}
void scnCheckStatus(int status, const char *file, int line) {
  if (status != SCN_OK)
    throw ScnException(std::string(scn_status_string(status)) + ": " + scn_last_error() + " at " + file + ":" + std::to_string(line));
}

int initializeGPU(int pciBusID) {
  int n = 0;
  cudaSafeCall(cudaGetDeviceCount(&n));
  int chosen = -1;
  for (int i = 0; i < n && chosen < 0; ++i) {
    int bus = 0;
    cudaSafeCall(cudaDeviceGetAttribute(&bus, cudaDevAttrPciBusId, i));
    if (pciBusID == -1 || bus == pciBusID) chosen = i;
  }
  if (chosen < 0) throw ScnException("no CUDA device with PCI bus id " + std::to_string(pciBusID));
  cudaSafeCall(cudaSetDevice(chosen));
  if (!scn_device_supported()) throw ScnException("this library runs on compute capability 10.x (B200) devices only");
  return chosen;
}

cudaMemStream::cudaMemStream() : pinnedMemorySize(1 << 20), pinnedMemory(nullptr), stream(nullptr), ownsStream(true) {
  cudaSafeCall(cudaMallocHost(&pinnedMemory, pinnedMemorySize));
  cudaSafeCall(cudaStreamCreate(&stream)); // a blocking stream: ordered against default-stream copies
}
cudaMemStream::cudaMemStream(cudaStream_t external)
    : pinnedMemorySize(1 << 20), pinnedMemory(nullptr), stream(external), ownsStream(false) {
  cudaSafeCall(cudaMallocHost(&pinnedMemory, pinnedMemorySize));
}
cudaMemStream::~cudaMemStream() {
  if (scratch || resultWords || chainBlock) cudaStreamSynchronize(stream);
  if (chainBlock) cudaFree(chainBlock);
  if (chainResident) scn_rules_chain_resident_destroy(chainResident);
  if (scratch) cudaFree(scratch);
  if (resultWords) cudaFree(resultWords);
  if (ownsStream && stream) cudaStreamDestroy(stream);
  if (pinnedMemory) cudaFreeHost(pinnedMemory);
}
void *cudaMemStream::deviceScratch(size_t bytes) {
  if (bytes > scratchBytes) {
    if (scratch) { cudaSafeCall(cudaStreamSynchronize(stream)); cudaSafeCall(cudaFree(scratch)); scratch = nullptr; scratchBytes = 0; }
    const size_t want = bytes + bytes / 4;
    cudaSafeCall(cudaMalloc(&scratch, want));
    scratchBytes = want;
  }
  return scratch;
}
void *cudaMemStream::chainWorkspace(size_t bytes) {
  if (bytes > chainBytes) {
    if (chainBlock) { cudaSafeCall(cudaStreamSynchronize(stream)); cudaSafeCall(cudaFree(chainBlock)); chainBlock = nullptr; chainBytes = 0; }
    const size_t want = bytes + bytes / 4;
    cudaSafeCall(cudaMalloc(&chainBlock, want));
    chainBytes = want;
    if (chainResident) scn_rules_chain_resident_invalidate(chainResident);
  }
  return chainBlock;
}
scn_chain_resident_t *cudaMemStream::chainState() {
  if (!chainResident) chainResident = scn_rules_chain_resident_create();
  if (!chainResident) throw ScnException("out of host memory");
  return chainResident;
}
int *cudaMemStream::deviceResult() {
  if (!resultWords) cudaSafeCall(cudaMalloc((void **)&resultWords, 4 * sizeof(int)));
  return resultWords;
}
void *cudaMemStream::staging(size_t bytes) {
  if (bytes > (size_t)pinnedMemorySize) {
    cudaSafeCall(cudaStreamSynchronize(stream)); // nothing may still be reading the old buffer
    cudaSafeCall(cudaFreeHost(pinnedMemory));
    pinnedMemory = nullptr;
    size_t want = std::max(bytes, (size_t)pinnedMemorySize * 2);
    if (want > (size_t)1 << 30) want = bytes;
    if (want > 0x7fffffffull) throw ScnException("staging buffer beyond 2 GiB");
    cudaSafeCall(cudaMallocHost(&pinnedMemory, want));
    pinnedMemorySize = (int)want;
  }
  return pinnedMemory;
}

// utilities.cu:132-169.  file / linenumber name the caller in the error message.
static void sgemmForm(bool ta, bool tb, float *A, float *B, float *C, int l, int m, int r, float alpha, float beta, const char *file, int line) {
  scnCheckStatus(scn_sgemm_rowmajor(ta, tb, A, B, C, l, m, r, alpha, beta, nullptr), file ? file : __FILE__, file ? line : __LINE__);
}
void d_rowMajorSGEMM_alphaAB_betaC(cublasHandle_t, float *A, float *B, float *C, int l, int m, int r, float alpha, float beta, const char *file, int line) {
  sgemmForm(false, false, A, B, C, l, m, r, alpha, beta, file, line);
}
void d_rowMajorSGEMM_alphaAtB_betaC(cublasHandle_t, float *A, float *B, float *C, int l, int m, int r, float alpha, float beta, const char *file, int line) {
  sgemmForm(true, false, A, B, C, l, m, r, alpha, beta, file, line);
}
void d_rowMajorSGEMM_alphaABt_betaC(cublasHandle_t, float *A, float *B, float *C, int l, int m, int r, float alpha, float beta, const char *file, int line) {
  sgemmForm(false, true, A, B, C, l, m, r, alpha, beta, file, line);
}
void d_rowMajorSGEMM_alphaAtBt_betaC(cublasHandle_t, float *A, float *B, float *C, int l, int m, int r, float alpha, float beta, const char *file, int line) {
  sgemmForm(true, true, A, B, C, l, m, r, alpha, beta, file, line);
}
