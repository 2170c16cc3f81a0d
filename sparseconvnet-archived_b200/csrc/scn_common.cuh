// Shared host/device helpers of libscn_b200.so (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
#include "scn_b200.h"

namespace scn {

// Thread-local message behind scn_last_error().
void set_error(const char *fmt, ...);
void clear_error();

// Kernels launched by this library in this process (every SCN_LAUNCH_CHECK counts one).
void count_launch();

// Number of SMs of the current device (cached per device); grids are sized in multiples of it.
int sm_count();

inline int fail(int status, const char *what) {
  set_error("%s", what);
  return status;
}

#define SCN_CUDA_TRY(expr)                                                                  \
  do {                                                                                      \
    cudaError_t e__ = (expr);                                                               \
    if (e__ != cudaSuccess) {                                                               \
      scn::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, __LINE__); \
      return SCN_ERR_CUDA;                                                                  \
    }                                                                                       \
  } while (0)

#define SCN_LAUNCH_CHECK(name)                                                              \
  do {                                                                                      \
    scn::count_launch();                                                                    \
    cudaError_t e__ = cudaGetLastError();                                                   \
    if (e__ != cudaSuccess) {                                                               \
      scn::set_error("launch of %s failed: %s", name, cudaGetErrorString(e__));             \
      return SCN_ERR_CUDA;                                                                  \
    }                                                                                       \
  } while (0)

// Programmatic dependent launch.  A kernel launched through launch_dependent() may start while the kernel
// in front of it in the stream is still running, once all of that kernel's CTAs have called
// dependents_may_launch() or exited; it must call wait_for_prior_grids() before it reads or writes any global
// memory that an earlier kernel of the stream touches (the wait returns when the earlier grids have finished
// and their writes are visible).  What runs before the wait (barrier and tensor-memory set-up, block scheduling)
// overlaps the earlier kernel's last wave.  SCN_DEPENDENT_LAUNCH=0 in the environment gives plain launches.
bool dependent_launch_enabled();
__device__ __forceinline__ void dependents_may_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void wait_for_prior_grids() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
template <class... KArgs, class... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = dependent_launch_enabled() ? 1 : 0;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Grid size for a grid-stride kernel over n items: enough CTAs to cover n, capped at
// `waves` CTAs per SM so a launch never exceeds a few resident waves.
inline int grid_for(long long n, int block, int waves = 8) {
  long long need = (n + block - 1) / block;
  long long cap = (long long)sm_count() * waves;
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ActivationFunction semantics of the reference (SigmoidLayer.cu:9, 46, 83, 121, 204-213;
// NetworkInNetworkPReLULayer.cu:12-13).  SOFTMAX is handled by the callers.
__device__ __forceinline__ float activate(float v, int act, float slope) {
  switch (act) {
  case SCN_RELU: return v > 0.f ? v : 0.f;
  case SCN_VLEAKYRELU: return v > 0.f ? v : v * 0.333f;
  case SCN_LEAKYRELU: return v > 0.f ? v : v * 0.01f;
  case SCN_TANH: return tanhf(v);
  case SCN_SIGMOID: return 1.0f / (1.0f + expf(-v));
  case SCN_PRELU: return v > 0.f ? v : v * slope;
  default: return v;
  }
}

// The same with the activation fixed at compile time: inner loops must not carry the switch
// (the tanh/exp branches cost hundreds of instructions per element when the compiler keeps
// them on the path).  SCN_DISPATCH_ACT(act, F) calls F<ACT>() for the run-time value.
template <int ACT> __device__ __forceinline__ float activate_t(float v, float slope) {
  if (ACT == SCN_RELU) return v > 0.f ? v : 0.f;
  if (ACT == SCN_VLEAKYRELU) return v > 0.f ? v : v * 0.333f;
  if (ACT == SCN_LEAKYRELU) return v > 0.f ? v : v * 0.01f;
  if (ACT == SCN_TANH) return tanhf(v);
  if (ACT == SCN_SIGMOID) return 1.0f / (1.0f + expf(-v));
  if (ACT == SCN_PRELU) return v > 0.f ? v : v * slope;
  return v;
}
#define SCN_DISPATCH_ACT(act, CALL)                                                          \
  switch (act) {                                                                            \
  case SCN_RELU: { constexpr int ACT = SCN_RELU; CALL; } break;                             \
  case SCN_VLEAKYRELU: { constexpr int ACT = SCN_VLEAKYRELU; CALL; } break;                 \
  case SCN_LEAKYRELU: { constexpr int ACT = SCN_LEAKYRELU; CALL; } break;                   \
  case SCN_TANH: { constexpr int ACT = SCN_TANH; CALL; } break;                             \
  case SCN_SIGMOID: { constexpr int ACT = SCN_SIGMOID; CALL; } break;                       \
  case SCN_PRELU: { constexpr int ACT = SCN_PRELU; CALL; } break;                           \
  default: { constexpr int ACT = SCN_NOSIGMOID; CALL; } break;                              \
  }

} // namespace scn
