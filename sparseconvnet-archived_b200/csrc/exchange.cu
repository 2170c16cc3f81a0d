// Exchange of classifier results between the GPUs of one node, over peer memory.
//
// The forward path shards by sample: every rank builds its own rulebooks and runs its own layers; the one thing the
// ranks ever tell each other is the [rows x nClasses] block of probabilities at the end of a step.  That block is a
// few KB, so what it costs is not bandwidth but the host work and the stream synchronisation of a library collective
// in every step.  Here a rank instead STORES its block straight into a buffer of every peer (plain peer stores over
// NVLink, then a system-scope release store of the step number), and a peer picks the blocks of a step up with a
// kernel that waits -- for a bounded time -- until every source's step number has arrived.  Both kernels run on the
// rank's own stream in front of the copy that brings the step's results to the host, so a step has no host-side
// collective call and no second synchronisation.
//
// Buffer of a rank (scn_exchange_buffer_bytes): a header {step, rows, floats}[SLOTS][MAX_RANKS], then
// float data[SLOTS][world][cap_floats].  Step s lives in slot s % SLOTS.  A source may overwrite a slot only after it
// has collected a later step from the owner, which the owner publishes after (in stream order) its own read of that
// slot: see scn_exchange_collect.  The waits are bounded: a rank that never publishes makes the collectors record
// its bit in their status word after the time limit and return; nothing spins forever.
#include <cstring>
#include "scn_common.cuh"

namespace {
constexpr int SLOTS = 4;
constexpr int MAX_RANKS = 16;
constexpr size_t HEADER_BYTES = 1024;
struct Header {
  unsigned step[SLOTS][MAX_RANKS];
  int rows[SLOTS][MAX_RANKS];
  int floats[SLOTS][MAX_RANKS];
};
static_assert(sizeof(Header) <= HEADER_BYTES, "header grows beyond its page");

unsigned long long g_timeout_ns = 2000ull * 1000 * 1000;

__host__ __device__ inline size_t cap_aligned(int capFloats) { return ((size_t)capFloats + 3) / 4 * 4; }
__device__ inline float *slot_data(char *base, int world, int capFloats, int slot, int source) {
  return (float *)(base + HEADER_BYTES) + ((size_t)slot * world + source) * cap_aligned(capFloats);
}
__device__ inline void store_release_sys(unsigned *p, unsigned v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ inline unsigned load_acquire_sys(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ inline unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

struct StepParams {
  void *peer[MAX_RANKS]; // publish: every rank's buffer (own included)
  const float *block;
  int floats, rows, world, rank, capFloats;
  unsigned publishStep; // 0: nothing to publish
  char *local;          // collect: this rank's buffer
  unsigned collectStep; // 0: nothing to collect
  float *out;
  int *rowsOut, *status;
  unsigned long long timeoutNs;
};

// CTA d of the publishing half copies this rank's block into rank d's buffer (d == rank: its own), then announces it.
__device__ void publish_block(const StepParams &p, int d) {
  char *base = (char *)p.peer[d];
  const int slot = p.publishStep % SLOTS;
  float *dst = slot_data(base, p.world, p.capFloats, slot, p.rank);
  const bool vec = (((uintptr_t)p.block) & 15) == 0;
  if (vec) {
    const int n4 = p.floats >> 2;
    const float4 *s4 = (const float4 *)p.block;
    float4 *d4 = (float4 *)dst;
    for (int i = threadIdx.x; i < n4; i += blockDim.x) d4[i] = s4[i];
    for (int i = (n4 << 2) + threadIdx.x; i < p.floats; i += blockDim.x) dst[i] = p.block[i];
  } else {
    for (int i = threadIdx.x; i < p.floats; i += blockDim.x) dst[i] = p.block[i];
  }
  __threadfence_system(); // every thread's stores are ordered before ...
  __syncthreads();
  if (threadIdx.x == 0) { // ... the announcement
    Header *h = (Header *)base;
    h->rows[slot][p.rank] = p.rows;
    h->floats[slot][p.rank] = p.floats;
    store_release_sys(&h->step[slot][p.rank], p.publishStep);
  }
}

// CTA r of the collecting half waits until source r's block of the step has arrived in this rank's buffer and copies it
// to out + r * capFloats; rowsOut[r] = its row count.  A source that does not arrive within the time limit sets bit r
// of *status (its block and row count are left untouched).
__device__ void collect_block(const StepParams &p, int r) {
  const int slot = p.collectStep % SLOTS;
  Header *h = (Header *)p.local;
  __shared__ int arrived;
  if (threadIdx.x == 0) {
    const unsigned long long t0 = now_ns();
    int ok = 1;
    while (load_acquire_sys(&h->step[slot][r]) != p.collectStep) {
      if (now_ns() - t0 > p.timeoutNs) { ok = 0; break; }
      __nanosleep(100);
    }
    if (!ok) atomicOr(p.status, 1 << r);
    arrived = ok;
  }
  __syncthreads();
  if (!arrived) return;
  const int floats = min(h->floats[slot][r], p.capFloats);
  if (threadIdx.x == 0 && p.rowsOut) p.rowsOut[r] = h->rows[slot][r];
  const float *src = slot_data(p.local, p.world, p.capFloats, slot, r);
  float *dst = p.out + (size_t)r * p.capFloats;
  if (((((uintptr_t)dst) | ((size_t)p.capFloats * 4)) & 15) == 0) {
    const int n4 = floats >> 2;
    for (int i = threadIdx.x; i < n4; i += blockDim.x) ((float4 *)dst)[i] = ((const float4 *)src)[i];
    for (int i = (n4 << 2) + threadIdx.x; i < floats; i += blockDim.x) dst[i] = src[i];
  } else {
    for (int i = threadIdx.x; i < floats; i += blockDim.x) dst[i] = src[i];
  }
}

// One launch does both halves of a step: CTAs [0, world) collect (if there is a step to collect), the CTAs behind them
// publish.  The collected step is an earlier one than the published one, and a collecting CTA waits only for stores of
// OTHER launches (the peers' publishing halves, on their own GPUs), never for a CTA of this grid.
__global__ void __launch_bounds__(256) k_exchange_step(const __grid_constant__ StepParams p) {
  scn::wait_for_prior_grids(); // the block to publish is the result of the kernel in front
  const int nCollect = p.collectStep ? p.world : 0;
  if ((int)blockIdx.x < nCollect) collect_block(p, blockIdx.x);
  else publish_block(p, blockIdx.x - nCollect);
}
} // namespace

extern "C" {

size_t scn_exchange_buffer_bytes(int world, int cap_floats) {
  if (world < 1 || world > MAX_RANKS || cap_floats < 1) return 0;
  return HEADER_BYTES + sizeof(float) * SLOTS * (size_t)world * cap_aligned(cap_floats);
}

void scn_exchange_set_timeout_ms(int ms) { g_timeout_ns = (unsigned long long)(ms < 1 ? 1 : ms) * 1000 * 1000; }

int scn_exchange_alloc(size_t bytes, void **d_buffer, unsigned char *ipc_handle) {
  scn::clear_error();
  if (!bytes || !d_buffer) return scn::fail(SCN_ERR_INVALID, "bad exchange buffer arguments");
  void *p = nullptr;
  SCN_CUDA_TRY(cudaMalloc(&p, bytes));
  cudaError_t e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e == cudaSuccess && ipc_handle) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, p);
    if (e == cudaSuccess) memcpy(ipc_handle, &h, sizeof(h));
  }
  if (e != cudaSuccess) {
    cudaFree(p);
    scn::set_error("exchange buffer set-up failed: %s", cudaGetErrorString(e));
    return SCN_ERR_CUDA;
  }
  *d_buffer = p;
  return SCN_OK;
}

int scn_exchange_free(void *d_buffer) {
  scn::clear_error();
  if (d_buffer) SCN_CUDA_TRY(cudaFree(d_buffer));
  return SCN_OK;
}

int scn_exchange_open(const unsigned char *ipc_handle, void **d_peer) {
  scn::clear_error();
  if (!ipc_handle || !d_peer) return scn::fail(SCN_ERR_INVALID, "bad exchange handle arguments");
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle, sizeof(h));
  SCN_CUDA_TRY(cudaIpcOpenMemHandle(d_peer, h, cudaIpcMemLazyEnablePeerAccess));
  return SCN_OK;
}

int scn_exchange_close(void *d_peer) {
  scn::clear_error();
  if (d_peer) SCN_CUDA_TRY(cudaIpcCloseMemHandle(d_peer));
  return SCN_OK;
}

static int launch_step(StepParams &p, scn_stream_t stream) {
  const int ctas = (p.collectStep ? p.world : 0) + (p.publishStep ? p.world : 0);
  if (!ctas) return SCN_OK;
  p.timeoutNs = g_timeout_ns;
  cudaError_t e = scn::launch_dependent(k_exchange_step, dim3(ctas), dim3(256), 0, (cudaStream_t)stream, p);
  if (e != cudaSuccess) {
    scn::set_error("launch of k_exchange_step failed: %s", cudaGetErrorString(e));
    return SCN_ERR_CUDA;
  }
  SCN_LAUNCH_CHECK("k_exchange_step");
  return SCN_OK;
}
static int fill_publish(StepParams &p, const float *d_block, int floats, int rows, void *const *peers, int world, int rank, int cap_floats,
                        unsigned step) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || cap_floats < 1 || floats < 0 || floats > cap_floats || !peers || step == 0)
    return scn::fail(SCN_ERR_INVALID, "bad exchange publish arguments (1..16 ranks, floats <= cap_floats, steps count from 1)");
  if (floats && !d_block) return scn::fail(SCN_ERR_INVALID, "null pointer");
  for (int r = 0; r < world; ++r) {
    if (!peers[r]) return scn::fail(SCN_ERR_INVALID, "a peer buffer is missing");
    p.peer[r] = peers[r];
  }
  p.block = d_block; p.floats = floats; p.rows = rows; p.world = world; p.rank = rank; p.capFloats = cap_floats; p.publishStep = step;
  return SCN_OK;
}
static int fill_collect(StepParams &p, void *d_local, int world, int cap_floats, unsigned step, float *d_out, int *d_rows, int *d_status) {
  if (world < 1 || world > MAX_RANKS || cap_floats < 1 || !d_local || !d_out || !d_status || step == 0)
    return scn::fail(SCN_ERR_INVALID, "bad exchange collect arguments");
  p.local = (char *)d_local; p.world = world; p.capFloats = cap_floats; p.collectStep = step; p.out = d_out; p.rowsOut = d_rows; p.status = d_status;
  return SCN_OK;
}

int scn_exchange_publish(const float *d_block, int floats, int rows, void *const *peers, int world, int rank, int cap_floats, unsigned step,
                         scn_stream_t stream) {
  scn::clear_error();
  StepParams p = {};
  int rc = fill_publish(p, d_block, floats, rows, peers, world, rank, cap_floats, step);
  return rc ? rc : launch_step(p, stream);
}

int scn_exchange_collect(void *d_local, int world, int cap_floats, unsigned step, float *d_out, int *d_rows, int *d_status, scn_stream_t stream) {
  scn::clear_error();
  StepParams p = {};
  int rc = fill_collect(p, d_local, world, cap_floats, step, d_out, d_rows, d_status);
  return rc ? rc : launch_step(p, stream);
}

int scn_exchange_step(void *d_local, unsigned collect_step, float *d_out, int *d_rows, int *d_status, const float *d_block, int floats, int rows,
                      void *const *peers, int world, int rank, int cap_floats, unsigned publish_step, scn_stream_t stream) {
  scn::clear_error();
  if (collect_step && publish_step && collect_step >= publish_step)
    return scn::fail(SCN_ERR_INVALID, "one launch collects an earlier step than the one it publishes");
  StepParams p = {};
  int rc = SCN_OK;
  if (collect_step) rc = fill_collect(p, d_local, world, cap_floats, collect_step, d_out, d_rows, d_status);
  if (!rc && publish_step) rc = fill_publish(p, d_block, floats, rows, peers, world, rank, cap_floats, publish_step);
  return rc ? rc : launch_step(p, stream);
}

} // extern "C"
