// Host helpers with the reference's names (utilities.h): integer arithmetic used by the
// builders, the pinned-staging stream object, top-k selection, error handling.
#pragma once
#include <cuda_runtime.h>
#include <stdexcept>
#include <string>
#include <vector>
#include "scn_b200.h"

// The reference's constructors take a cuBLAS handle (NetworkInNetworkLayer.h:24-28).  No
// cuBLAS is used here; the type is declared (identically to cublas_api.h) so the same
// signatures compile, and the handle is ignored.
struct cublasContext;
typedef struct cublasContext *cublasHandle_t;

// The reference's cuBLAS wrappers (utilities.h:82-102): C[l x r] = alpha * op(A) * op(B) + beta * C, row-major, op(A) l x m
// and op(B) m x r ("At": A is stored m x l, "Bt": B is stored r x m).  The handle is ignored; the product runs on the
// legacy default stream, which is ordered against the blocking streams the networks create.
void d_rowMajorSGEMM_alphaAB_betaC(cublasHandle_t handle, float *A, float *B, float *C, int l, int m, int r, float alpha, float beta,
                                   const char *file = 0, int linenumber = 0);
void d_rowMajorSGEMM_alphaAtB_betaC(cublasHandle_t handle, float *A, float *B, float *C, int l, int m, int r, float alpha, float beta,
                                    const char *file = 0, int linenumber = 0);
void d_rowMajorSGEMM_alphaABt_betaC(cublasHandle_t handle, float *A, float *B, float *C, int l, int m, int r, float alpha, float beta,
                                    const char *file = 0, int linenumber = 0);
void d_rowMajorSGEMM_alphaAtBt_betaC(cublasHandle_t handle, float *A, float *B, float *C, int l, int m, int r, float alpha, float beta,
                                     const char *file = 0, int linenumber = 0);

#define NTHREADS 512
#define KERNELBLOCKSIZE 32

std::vector<int> range(int n);                    // 0,1,...,n-1
int ipow(int base, int exp);                      // utilities.cu:14-26
int triangleSize(int linearSize, int dimension);  // utilities.cu:27-32
int intRound(int a, int d);                       // utilities.cu:103
int intRoundUp(int a, int d);                     // utilities.cu:102
template <typename t> std::vector<int> vectorTopIndices(std::vector<t> &test, int k); // utilities.cu:35-56

// Errors are C++ exceptions here; the reference prints and calls exit() (utilities.h:32-67).
struct ScnException : std::runtime_error {
  using std::runtime_error::runtime_error;
};
void scnCheckCuda(cudaError_t err, const char *file, int line);
void scnCheckStatus(int status, const char *file, int line);
#define cudaSafeCall(err) scnCheckCuda((err), __FILE__, __LINE__)
#define cudaCheckError() scnCheckCuda(cudaGetLastError(), __FILE__, __LINE__)
#define scnSafeCall(st) scnCheckStatus((st), __FILE__, __LINE__)

// Selects the device with this PCI bus id (-1: device 0) and returns its ordinal
// (utilities.cu:105-130).  Refuses devices that are not compute capability 10.x.
int initializeGPU(int pciBusID);

// A stream plus a pinned staging buffer (utilities.h:105-112).  The buffer grows on demand.
// With an external stream (the benchmark passes torch's current stream) the object does
// not own it.  It also owns the device scratch of this stream's rule builds (layer descriptors,
// per-sample counts, bitmaps, prefix sums): one per network, like every other buffer of a
// network, so that two networks on one device never share mutable state.
class cudaMemStream {
public:
  int pinnedMemorySize;
  void *pinnedMemory;
  cudaStream_t stream;
  cudaMemStream();
  explicit cudaMemStream(cudaStream_t external);
  ~cudaMemStream();
  void *staging(size_t bytes); // pinned buffer of at least `bytes`
  void *deviceScratch(size_t bytes); // device buffer of at least `bytes`; only work on `stream` may use it
  int *deviceResult();               // four device ints for a rule build whose counts nobody reads
  // Device block of the fused rule chain's resident build (scn_rules_chain_build_resident): nothing else writes it.
  void *chainWorkspace(size_t bytes);
  scn_chain_resident_t *chainState();
  cudaMemStream(const cudaMemStream &) = delete;
  cudaMemStream &operator=(const cudaMemStream &) = delete;

private:
  bool ownsStream;
  void *scratch = nullptr;
  size_t scratchBytes = 0;
  int *resultWords = nullptr;
  void *chainBlock = nullptr;
  size_t chainBytes = 0;
  scn_chain_resident_t *chainResident = nullptr;
};
