// Fused rule-gather + NetworkInNetwork forward on the 5th-generation tensor cores
// (tcgen05.mma with the accumulator in tensor memory), sm_100a only.
//
//   out[r][n] = act( p * sum_k A[r][k] * W[k][n] + p * B[n] ),   A[r][f*nIn + c] = in[rules[r*fs+f]][c]
//
// A persistent CTA (one per SM) walks 128-row x BN-column output tiles.  The K axis is walked in
// slabs of 32 fp32 values (128 bytes, one 128B-swizzle row).  14 warps, by role:
//
//   warps 0-3   epilogue of tile i while the main loop already runs tile i+1 (two accumulators in
//               tensor memory): tcgen05.ld of 32 columns -> padded shared slice -> coalesced row
//               stores with p*acc + p*bias and the activation.
//   warps 4-7   gather: asynchronous copies (cp.async, zero fill for a negative rule or a row past
//               the end) of the rows the rules name, straight into the canonical K-major
//               SWIZZLE_128B tile; completion arrives on the stage's "raw" barrier, so several
//               slabs are in flight.  nIn % 32 == 0: a slab lies inside one filter cell and a row of
//               it is 128 contiguous bytes (16-byte copies).  Any other nIn (3 input channels, say):
//               4-byte copies, lane = position in the slab, so that the lanes of one instruction
//               read neighbouring words of the few source rows one output row names.  The tile's rules are staged in shared memory, the next tile's prefetched
//               meanwhile.
//   warps 8-11  split: once a raw tile has landed it already serves as the tf32 "hi" operand (the
//               tensor core reads the upper 19 bits of each fp32); these warps write lo = x - hi
//               into the second image, fence to the async proxy and arrive on the "full" barrier.
//   warp 12     one thread issues a cp.async.bulk per slab for the weight tile (hi and lo images,
//               pre-split, pre-transposed and pre-swizzled once by tc_pack, so the copy is a plain
//               contiguous block into this CTA's own shared memory; no tensor map is needed).
//   warp 13     allocates tensor memory; one thread issues, per slab, 3 x 4 tcgen05.mma
//               (kind::tf32, M=128, N=BN, K=8): A_lo*B_hi + A_hi*B_lo + A_hi*B_hi, which restores
//               fp32-grade accuracy from tf32 products ("3xTF32"), then tcgen05.commit onto the
//               stage's "empty" barrier.
//
// The gathered matrix never exists in global memory (the reference writes and re-reads it,
// ConvolutionalLayer.cu:124-133).  Every mbarrier wait has a time limit: on expiry the kernel
// records an error code in g_tc_error and carries on to its normal exit, so tensor memory is
// always released and the context stays usable.
#include "conv_nin_tc.cuh"
#include <cstdlib>
#include <type_traits>
#include <cuda_bf16.h>

namespace scn {

__device__ int g_tc_error = 0;

// Source of the 16-byte gather for a missing row (negative rule, row past the end): zeros.  Copying
// from here instead of predicating each copy keeps the gather loop at three instructions per copy.
constexpr int ZERO_ROW_FLOATS = 16384;
__device__ __align__(128) float g_zero_row[ZERO_ROW_FLOATS];
__device__ int g_no_row = -1; // what a load of a missing rule reads: loads stay unconditional, nothing selects on their values

namespace {

constexpr int BM = 128;          // rows per CTA tile (UMMA M)
constexpr int SLAB = 32;         // fp32 values of K per pipeline stage
constexpr int ROW_BYTES = 128;   // bytes of one smem row (SLAB * 4)
constexpr int A_HALF = BM * ROW_BYTES; // 16 KB: one of A_hi / A_lo
constexpr int NUM_THREADS = 448;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull; // 2 s

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait: false (and an error code) if the phase did not complete in time.
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int code) {
  unsigned long long start = 0;
  for (uint32_t i = 0;; ++i) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    if ((i & 63) == 63) {
      if (*(volatile int *)&g_tc_error != 0) return false; // another wait already gave up: do not wait again
      const unsigned long long now = global_ns();
      if (start == 0) start = now;
      else if (now - start > WAIT_LIMIT_NS) break;
    }
  }
  atomicCAS(&g_tc_error, 0, code);
  return false;
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// Shared-memory matrix descriptor, K-major, SWIZZLE_128B: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3fff);
  d |= (uint64_t)1 << 16;             // leading byte offset (unused for swizzled K-major): 1
  d |= (uint64_t)(1024 >> 4) << 32;   // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;             // descriptor version of this architecture
  d |= (uint64_t)2 << 61;             // SWIZZLE_128B
  return d;
}
// The same for a tile whose rows are 64 bytes long (32 bf16 values of K), SWIZZLE_64B: 8-row groups 512 bytes apart.
__device__ __forceinline__ uint64_t smem_desc64(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3fff);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(512 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)4 << 61;             // SWIZZLE_64B
  return d;
}
// bf16 operands (kind::f16), A in tensor memory: lane = row, each 32-bit column holds two consecutive values of K
__device__ __forceinline__ void mma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
               ::"r"(d_tmem), "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// A operand in tensor memory (lane = row, one tf32 per column)
__device__ __forceinline__ void mma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
               ::"r"(d_tmem), "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ float to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

struct Params {
  const float *in; const int *rules; int rows, fs, nIn;
  const unsigned char *packed; const float *bias; const float *prelu;
  int N, BN, nTiles, nSlabs, stages, tmemCols, rulesBytes; float p; int act; float *out; uint32_t idesc;
  int mTiles, accStride, K, generic, epi2, rulesDouble, rawEntries, nStages64, atmem, aBase, bf16; const int *rowsPtr; const int *poolRules; int *choices; int poolCells; int kSplit; float *partial; // K split over kSplit CTAs per tile: raw partial sums go to partial[split][row][col]
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t srcBytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(srcBytes) : "memory");
}
__device__ __forceinline__ void cp_async16_full(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void *src, uint32_t srcBytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(srcBytes) : "memory");
}
// The barrier receives one arrival once all cp.async issued so far by this thread have landed.
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// Position in a ring of n buffers and the parity of the current pass over it (no division per step).
struct Ring {
  int idx = 0, phase = 0, n;
  __device__ explicit Ring(int n_) : n(n_) {}
  __device__ __forceinline__ void next() { if (++idx == n) { idx = 0; phase ^= 1; } }
};

constexpr int MAX_STAGES = 6;
constexpr int EPI_COLS = 32;                      // accumulator columns staged per epilogue step
constexpr int EPI_LD = EPI_COLS + 4;              // padded row stride (floats) of the staging slice
constexpr int EPI_BYTES = BM * EPI_LD * 4;        // 18 KB

// Epilogue role (warps 0-3 of both tensor-core kernels): drains accumulator n & 1 of work item n
// while the main loop fills the other one.
// POOL: a non-overlapping max-pooling layer behind this layer is applied here (MaxPoolingLayer.cu:9-35).  The
// tile's 128 rows are 128/cells pooling windows x cells; tile row i is the layer-output row poolRules[row0 + i]
// (negative: skipped, as maxPool skips it).  Only the pooled rows and their choices are written.
// Two groups (four warps each) may share the work: group g takes the work items n = g, g + 2, ... of this CTA,
// i.e. always accumulator g; each has its own staging slice, pooling-row table and named barrier.
// The CTA's LAST work item has no main loop behind it to hide under, so the producer warps, idle by then, help:
// with tailShare = 3 the owner (tailRank 0) takes every third 32-column slice of that item and the gather and split
// warps (tailRank 1, 2: they run this function for that one item, staging through tailEpi, a pipeline stage that is
// free once the item's MMAs have completed) take the others.
template <bool SPLIT, int ACT, bool POOL = false>
__device__ __forceinline__ void epilogue_role(const Params &P, float *epiBase, uint32_t tmem, uint32_t accFullBar, uint32_t accEmptyBar,
                                              int nItems, int kSplit, int rows, int group = 0, int nGroups = 1, int tailShare = 0,
                                              int tailRank = 0, float *tailEpi = nullptr) {
  __shared__ int poolRow0[BM]; // POOL: this tile's layer-output row per tile row (the second group's table follows its staging slice)
  int *poolRow = tailRank ? reinterpret_cast<int *>(tailEpi + EPI_BYTES / 4) : group ? reinterpret_cast<int *>(epiBase + 2 * (EPI_BYTES / 4)) : poolRow0;
  float *epi = tailRank ? tailEpi : epiBase + (size_t)group * (EPI_BYTES / 4);
  const int barId = tailRank ? 3 + tailRank : group ? 3 : 1;
  const int t = threadIdx.x & 127; // thread of the group; its warp reads tensor-memory lanes 32 * (warp % 4)...
  const int warp = t >> 5;
  const uint32_t laneAddr = tmem + ((uint32_t)(warp * 32) << 16);
  float *myRow = epi + (size_t)t * EPI_LD;
  const int c4 = t & 7, rsub = t >> 3; // store phase: 8 threads per row, 16 rows per pass
  int n = group, firstItem = blockIdx.x + group * gridDim.x;
  if (tailRank) { // a helper: this CTA's last item only
    const int count = (nItems - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    if (nItems <= (int)blockIdx.x || count <= 0) return;
    n = count - 1;
    firstItem = blockIdx.x + n * gridDim.x;
  }
  for (int item = firstItem; item < nItems; item += nGroups * gridDim.x, n += nGroups) {
    const bool shared = tailShare > 1 && item + nGroups * (int)gridDim.x >= nItems;
    const int sliceFirst = shared ? tailRank * EPI_COLS : 0, sliceStep = shared ? tailShare * EPI_COLS : EPI_COLS;
    const int tileId = SPLIT ? item / kSplit : item, split = SPLIT ? item - tileId * kSplit : 0;
    const int tileN = tileId % P.nTiles, tileM = tileId / P.nTiles;
    const int ab = n & 1;
    mbar_wait(accFullBar + 8 * ab, (n >> 1) & 1, 2);
    tc_fence_after();
    const int row0 = tileM * BM, col0 = tileN * P.BN;
    if (POOL) { // read before the first slice's barrier, used after it
      const long long gr = (long long)row0 + t;
      poolRow[t] = gr < rows ? __ldg(P.poolRules + gr) : -1;
    }
    for (int c = sliceFirst; c < P.BN; c += sliceStep) {
      const int width = min(EPI_COLS, P.BN - c); // 32, or 16 for the last slice when BN % 32 == 16
      uint32_t a[32];
      const uint32_t addr = laneAddr + (uint32_t)(ab * P.accStride + c);
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                   : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]), "=r"(a[4]), "=r"(a[5]), "=r"(a[6]), "=r"(a[7]),
                     "=r"(a[8]), "=r"(a[9]), "=r"(a[10]), "=r"(a[11]), "=r"(a[12]), "=r"(a[13]), "=r"(a[14]), "=r"(a[15])
                   : "r"(addr));
      if (width > 16)
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                     : "=r"(a[16]), "=r"(a[17]), "=r"(a[18]), "=r"(a[19]), "=r"(a[20]), "=r"(a[21]), "=r"(a[22]), "=r"(a[23]),
                       "=r"(a[24]), "=r"(a[25]), "=r"(a[26]), "=r"(a[27]), "=r"(a[28]), "=r"(a[29]), "=r"(a[30]), "=r"(a[31])
                     : "r"(addr + 16));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int q = 0; q < 32; q += 4)
        if (q < width)
          *reinterpret_cast<float4 *>(myRow + q) = make_float4(__uint_as_float(a[q]), __uint_as_float(a[q + 1]), __uint_as_float(a[q + 2]), __uint_as_float(a[q + 3]));
      asm volatile("bar.sync %0, 128;" ::"r"(barId) : "memory");
      // coalesced: 8 threads cover one row's 128 bytes, a warp covers 4 rows per instruction
      const int col = col0 + c + c4 * 4;
      const bool colOk = c4 * 4 < width && col < P.N; // N % 4 == 0: a float4 is in or out as a whole
      float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f), s4 = b4;
      if (colOk && !SPLIT) {
        b4 = __ldg(reinterpret_cast<const float4 *>(P.bias + col));
        if (ACT == SCN_PRELU) s4 = __ldg(reinterpret_cast<const float4 *>(P.prelu + col));
      }
      if (POOL) {
        // the window's cells are read together (independent shared-memory loads), then compared in order
        auto pool_windows = [&](auto cellsC, auto batchC) {
          constexpr int CELLSC = decltype(cellsC)::value, CH = decltype(batchC)::value; // CELLSC == 0: any power of two
          constexpr bool ACT_LAST = ACT == SCN_NOSIGMOID || ACT == SCN_VLEAKYRELU || ACT == SCN_LEAKYRELU; // strictly increasing
          const int CELLS = CELLSC ? CELLSC : P.poolCells, WINDOWS = BM / CELLS;
#pragma unroll
          for (int pr = rsub; pr < WINDOWS; pr += 16) { // (WINDOWS < 16: rows rsub >= WINDOWS have no window)
            const long long w = (long long)tileM * WINDOWS + pr; // pooled row
            if (!colOk || w * CELLS >= rows) continue;
            float best[4] = {0.f, 0.f, 0.f, 0.f};
            int idx[4] = {-1, -1, -1, -1};
            bool none = true;
#pragma unroll 1
            for (int cell0 = 0; cell0 < CELLS; cell0 += CH) {
              int from[CH];
              float4 v[CH];
#pragma unroll
              for (int j = 0; j < CH; ++j) {
                from[j] = poolRow[pr * CELLS + cell0 + j];
                v[j] = *reinterpret_cast<const float4 *>(epi + (size_t)(pr * CELLS + cell0 + j) * EPI_LD + c4 * 4);
              }
#pragma unroll
              for (int j = 0; j < CH; ++j) {
                if (from[j] < 0) continue;
                // ACT_LAST: p * v + p * b and the activation do not decrease in v, so the cells are compared on the raw
                // sums and only the winner is finished (where two different sums round to one output, this picks the
                // larger sum and the reference the earlier cell: the pooled value is the same)
                const float o[4] = {ACT_LAST ? v[j].x : activate_t<ACT>(P.p * v[j].x + P.p * b4.x, s4.x),
                                    ACT_LAST ? v[j].y : activate_t<ACT>(P.p * v[j].y + P.p * b4.y, s4.y),
                                    ACT_LAST ? v[j].z : activate_t<ACT>(P.p * v[j].z + P.p * b4.z, s4.z),
                                    ACT_LAST ? v[j].w : activate_t<ACT>(P.p * v[j].w + P.p * b4.w, s4.w)};
                const int base = from[j] * P.N + col;
#pragma unroll
                for (int k = 0; k < 4; ++k)
                  if (none || best[k] < o[k]) { best[k] = o[k]; idx[k] = base + k; } // the first maximum wins
                none = false;
              }
            }
            if (ACT_LAST && !none) {
              best[0] = activate_t<ACT>(P.p * best[0] + P.p * b4.x, s4.x); best[1] = activate_t<ACT>(P.p * best[1] + P.p * b4.y, s4.y);
              best[2] = activate_t<ACT>(P.p * best[2] + P.p * b4.z, s4.z); best[3] = activate_t<ACT>(P.p * best[3] + P.p * b4.w, s4.w);
            }
            *reinterpret_cast<float4 *>(P.out + w * P.N + col) = make_float4(best[0], best[1], best[2], best[3]);
            *reinterpret_cast<int4 *>(P.choices + w * P.N + col) = make_int4(idx[0], idx[1], idx[2], idx[3]);
          }
        };
        switch (P.poolCells) { // 2 x 2 and 2 x 2 x 2 windows unrolled; 2, 16 and 32 cells in batches of two
        case 4: pool_windows(std::integral_constant<int, 4>(), std::integral_constant<int, 4>()); break;
        case 8: pool_windows(std::integral_constant<int, 8>(), std::integral_constant<int, 8>()); break;
        default: pool_windows(std::integral_constant<int, 0>(), std::integral_constant<int, 2>()); break;
        }
      } else
#pragma unroll
      for (int pass = 0; pass < BM / 16; ++pass) {
        const int rl = pass * 16 + rsub, r = row0 + rl;
        if (!colOk || r >= rows) continue;
        const float4 v = *reinterpret_cast<const float4 *>(epi + (size_t)rl * EPI_LD + c4 * 4);
        if (SPLIT) {
          *reinterpret_cast<float4 *>(P.partial + ((long long)split * rows + r) * P.N + col) = v;
        } else {
          float4 o;
          // NetworkInNetworkLayer.cu:187-195: alpha = beta = p over a bias-filled output
          o.x = activate_t<ACT>(P.p * v.x + P.p * b4.x, s4.x); o.y = activate_t<ACT>(P.p * v.y + P.p * b4.y, s4.y);
          o.z = activate_t<ACT>(P.p * v.z + P.p * b4.z, s4.z); o.w = activate_t<ACT>(P.p * v.w + P.p * b4.w, s4.w);
          *reinterpret_cast<float4 *>(P.out + (long long)r * P.N + col) = o;
        }
      }
      asm volatile("bar.sync %0, 128;" ::"r"(barId) : "memory"); // the slice is free again
    }
    if (tailRank) break; // (nothing waits for the last item's accumulator)
    tc_fence_before();
    mbar_arrive(accEmptyBar + 8 * ab); // this accumulator may be overwritten
  }
}

// Work items are output tiles, or (tile, K range) pairs when K is split over several CTAs.
// ATMEM: the A operand is fed from tensor memory.  The split warps store the hi (raw) and lo images of
// a slab straight into one of two 64-column tensor-memory slots (tcgen05.st, thread = row) and the MMAs
// read A from there: the lo image is never written to shared memory and the tensor core reads no A tile
// from it, which takes about 30 % off the shared-memory data pipe, the resource that bounds this
// kernel (second convolution of the benchmark 81 -> 66 us, third 72 -> 64 us).  Needs 2 accumulators + 128
// columns <= 512, i.e. BN <= 192; a shared-memory stage then holds the raw A tile and the weight images only.
template <bool SPLIT, int ACT, bool ATMEM, bool POOL = false>
__global__ void __launch_bounds__(NUM_THREADS, 1) k_conv_nin_tc(const Params P) {
  extern __shared__ unsigned char smem_raw[];
  int *rulesS = reinterpret_cast<int *>(smem_raw); // [128 x fs] rule tile of the current item (when it fits)
  // 1024-byte alignment: the swizzle pattern is a function of absolute shared-memory address bits
  unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + (P.rulesDouble ? 2 : 1) * P.rulesBytes + 1023) & ~(uintptr_t)1023);
  const int bHalf = P.BN * ((ATMEM && P.bf16) ? ROW_BYTES / 2 : ROW_BYTES); // one of B_hi / B_lo: 32 values of K per row, tf32 or bf16
  const int aBytes = ATMEM ? A_HALF : 2 * A_HALF;  // A raw (= hi) [, A_lo]
  const int stageBytes = aBytes + 2 * bHalf;       // then B_hi, B_lo
  float *epi = reinterpret_cast<float *>(smem + (size_t)P.stages * stageBytes);
  __shared__ __align__(8) uint64_t bars[3 * MAX_STAGES + 8];
  __shared__ uint32_t tmemBase;
  const uint32_t rawBar = smem_u32(&bars[0]), fullBar = smem_u32(&bars[MAX_STAGES]), emptyBar = smem_u32(&bars[2 * MAX_STAGES]),
                 accFullBar = smem_u32(&bars[3 * MAX_STAGES]), accEmptyBar = smem_u32(&bars[3 * MAX_STAGES + 2]),
                 aFullBar = smem_u32(&bars[3 * MAX_STAGES + 4]), aEmptyBar = smem_u32(&bars[3 * MAX_STAGES + 6]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P.stages; ++s) {
      mbar_init(rawBar + 8 * s, 128);      // the gather threads' cp.async completions
      mbar_init(fullBar + 8 * s, ATMEM ? 1 : 128 + 1); // [the split threads +] the weight copy
      mbar_init(emptyBar + 8 * s, 1);      // tcgen05.commit
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(accFullBar + 8 * a, 1); mbar_init(accEmptyBar + 8 * a, 128);
      mbar_init(aFullBar + 8 * a, 128); mbar_init(aEmptyBar + 8 * a, 1); // tensor-memory A slots (ATMEM)
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 13) { // tensor memory: two 128 x BN fp32 accumulators
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmemBase)), "r"((uint32_t)P.tmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmemBase;
  // The next kernel's CTAs may take over SMs as this grid's CTAs leave them.  Said only now that this CTA holds its
  // tensor-memory columns: a dependent CTA that shared the SM could otherwise allocate first and then sit in its own
  // wait for this grid while this CTA waits for columns (tcgen05.alloc has no time limit).
  scn::dependents_may_launch();
  scn::wait_for_prior_grids(); // everything above overlapped the kernel in front; its results are read from here on
  // the row count may still be on its way to the host when this kernel is launched: read it from device memory
  // (POOL: rows counts tile rows = pooled rows x cells, and the device-side count is in pooled rows)
  const int rows = P.rowsPtr ? min(max(*(const volatile int *)P.rowsPtr, 0) * (POOL ? P.poolCells : 1), P.rows) : P.rows;
  const int mTiles = P.rowsPtr ? (rows + BM - 1) / BM : P.mTiles;
  const int kSplit = SPLIT ? P.kSplit : 1;
  const int nItems = mTiles * P.nTiles * kSplit;

  // decode a work item
  auto itemTile = [&](int item, int &tileM, int &tileN, int &slab0, int &nLoc) {
    const int tileId = SPLIT ? item / kSplit : item, split = SPLIT ? item - tileId * kSplit : 0;
    tileN = tileId % P.nTiles; tileM = tileId / P.nTiles;
    slab0 = SPLIT ? split * P.nSlabs / kSplit : 0;
    nLoc = SPLIT ? (split + 1) * P.nSlabs / kSplit - slab0 : P.nSlabs;
    return split;
  };

  const bool epi2 = !SPLIT && !ATMEM && P.epi2;
  // the producer warps share the epilogue of the CTA's last item (two free pipeline stages serve as their staging slices)
  const int tailShare = (!epi2 && P.stages >= 2 && stageBytes >= EPI_BYTES + BM * 4) ? 3 : 0;
  if (warp < 4) {
    epilogue_role<SPLIT, ACT, POOL>(P, epi, tmem, accFullBar, accEmptyBar, nItems, kSplit, rows, 0, epi2 ? 2 : 1, tailShare);
  } else if (warp < 8) {
    // ------------------------------------------------------------ gather: asynchronous 16-byte copies
    const int t = threadIdx.x - 128, chunk = t & 7, rbase = t >> 3;
    // this thread's 16-byte chunk sits at the same offset in each of its 8 rows (16 rows apart)
    const uint32_t rowOff = (rbase >> 3) * 1024 + (rbase & 7) * ROW_BYTES + ((chunk ^ (rbase & 7)) << 4);
    int nItem = 0;
    Ring ring(P.stages);
    // 16-byte asynchronous copies of one tile's [128 x fs] rules (the tile starts 512*fs bytes into
    // the array, so chunks are aligned); bytes past the end of the array are not read.
    auto stage_rules_async = [&](int item, int buf) {
      int tileM, tileN, slab0, nLoc;
      itemTile(item, tileM, tileN, slab0, nLoc);
      const long long first = (long long)tileM * BM * P.fs, total = (long long)rows * P.fs;
      const uint32_t dst = smem_u32(rulesS) + buf * P.rulesBytes;
      for (int ch = t; ch < BM * P.fs / 4; ch += 128) {
        const long long left = total - (first + ch * 4);
        const uint32_t bytes = left >= 4 ? 16u : left > 0 ? (uint32_t)left * 4u : 0u;
        cp_async16(dst + ch * 16, bytes ? (const void *)(P.rules + first + ch * 4) : (const void *)P.rules, bytes);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // POOL: tile row t is the layer-output row poolRules[first tile row + t]; its fs rules are copied from there
    // (4-byte copies), the row id itself goes behind them ([128 x fs] rules, then 128 row ids per buffer)
    auto pool_row_of = [&](int item) {
      int tileM, tileN, slab0, nLoc;
      itemTile(item, tileM, tileN, slab0, nLoc);
      const long long gr = (long long)tileM * BM + t;
      return __ldg(gr < rows ? P.poolRules + gr : &g_no_row);
    };
    auto stage_rules_pool = [&](int buf, int from) {
      int *base = rulesS + buf * (P.rulesBytes >> 2);
      const uint32_t dst = smem_u32(base) + t * P.fs * 4;
      if (!P.generic) // (the word-by-word gather reads its rules from global memory, see there)
        for (int f = 0; f < P.fs; ++f)
          cp_async4(dst + 4 * f, from >= 0 ? (const void *)(P.rules + (long long)from * P.fs + f) : (const void *)P.rules, from >= 0 ? 4u : 0u);
      base[BM * P.fs + t] = from;
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    int fromNext = -1; // POOL: this thread's row id of the tile after the next staged one
    if (POOL) {
      if ((int)blockIdx.x < nItems) stage_rules_pool(0, pool_row_of(blockIdx.x));
      if ((int)(blockIdx.x + gridDim.x) < nItems) fromNext = pool_row_of(blockIdx.x + gridDim.x);
    } else if (P.rulesDouble && (int)blockIdx.x < nItems) stage_rules_async(blockIdx.x, 0);
    for (int item = blockIdx.x; item < nItems; item += gridDim.x, ++nItem) {
      int tileM, tileN, slab0, nLoc;
      itemTile(item, tileM, tileN, slab0, nLoc);
      const int row0 = tileM * BM;
      const int *rulesT = rulesS; // this tile's staged rules
      const int *fromT = nullptr; // POOL: this tile's layer-output row per tile row
      if (POOL) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        asm volatile("bar.sync 2, 128;" ::: "memory");
        rulesT = rulesS + (nItem & 1) * (P.rulesBytes >> 2);
        fromT = rulesT + BM * P.fs;
        if (item + (int)gridDim.x < nItems) {
          stage_rules_pool((nItem + 1) & 1, fromNext);
          fromNext = item + 2 * (int)gridDim.x < nItems ? pool_row_of(item + 2 * gridDim.x) : -1;
        }
      } else if (P.rulesDouble) {
        // the rules of this tile were prefetched while the previous tile's copies were issued
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        asm volatile("bar.sync 2, 128;" ::: "memory"); // all chunks landed; everyone is done with the other buffer
        rulesT = rulesS + (nItem & 1) * (P.rulesBytes >> 2);
        if (item + (int)gridDim.x < nItems) stage_rules_async(item + gridDim.x, (nItem + 1) & 1);
      } else if (P.rulesBytes > 0) { // synchronous staging (rule pointer not 16-byte aligned, or no room for two buffers)
        asm volatile("bar.sync 2, 128;" ::: "memory"); // everyone has issued the previous item's copies
        const int nr = BM * P.fs;
        for (int e = t; e < nr; e += 128) rulesS[e] = __ldg(P.rules + min((long long)row0 * P.fs + e, (long long)rows * P.fs - 1));
        asm volatile("bar.sync 2, 128;" ::: "memory");
      }
      if (epi2) {
        // Few input channels, one slab (a first layer): lane = tile row.  A lane reads its row's fs rules, then
        // the fs x nIn words they name (every load unconditional: a missing rule reads a -1 word, a missing
        // row the zero row), computes lo = x - tf32(x) and stores both images of its row as 16-byte chunks
        // (rows r..r+7 fall on eight different chunk columns of the swizzled tile: no bank conflict).
        // About 250 instructions per warp and tile where the lane-per-word form and the split warps need 700.
        auto gather_rows = [&](auto ninC) {
          constexpr int NIN = decltype(ninC)::value, FMAX = SLAB / NIN;
          const int st = ring.idx;
          int from;
          if (POOL) from = fromT[t];
          else from = row0 + t < rows ? row0 + t : -1;
          int rule[FMAX];
#pragma unroll
          for (int f = 0; f < FMAX; ++f)
            rule[f] = __ldg(f < P.fs && from >= 0 ? P.rules + (long long)from * P.fs + f : &g_no_row);
          float v[SLAB];
#pragma unroll
          for (int k = 0; k < SLAB; ++k) v[k] = 0.f;
#pragma unroll
          for (int f = 0; f < FMAX; ++f)
#pragma unroll
            for (int c = 0; c < NIN; ++c)
              v[f * NIN + c] = __ldg(rule[f] >= 0 ? P.in + (long long)rule[f] * NIN + c : g_zero_row);
          mbar_wait(emptyBar + 8 * st, ring.phase ^ 1, 1);
          unsigned char *rowp = smem + (size_t)st * stageBytes + (t >> 3) * 1024 + (t & 7) * ROW_BYTES;
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
            float4 hi = make_float4(v[4 * ch], v[4 * ch + 1], v[4 * ch + 2], v[4 * ch + 3]), lo;
            lo.x = hi.x - __uint_as_float(__float_as_uint(hi.x) & 0xffffe000u);
            lo.y = hi.y - __uint_as_float(__float_as_uint(hi.y) & 0xffffe000u);
            lo.z = hi.z - __uint_as_float(__float_as_uint(hi.z) & 0xffffe000u);
            lo.w = hi.w - __uint_as_float(__float_as_uint(hi.w) & 0xffffe000u);
            const int off = (ch ^ (t & 7)) << 4;
            *reinterpret_cast<float4 *>(rowp + off) = hi;
            *reinterpret_cast<float4 *>(rowp + A_HALF + off) = lo;
          }
          fence_async_smem(); // the tensor core reads the tile through the asynchronous proxy
          mbar_arrive(fullBar + 8 * st);
          ring.next();
        };
        switch (P.nIn) { // (one slab: nLoc == 1)
        case 1: gather_rows(std::integral_constant<int, 1>()); break;
        case 2: gather_rows(std::integral_constant<int, 2>()); break;
        case 3: gather_rows(std::integral_constant<int, 3>()); break;
        default: gather_rows(std::integral_constant<int, 4>()); break;
        }
        continue;
      }
      if (P.generic) {
        // nIn is not a multiple of 32 (e.g. 3 input channels): a slab spans several filter cells, so
        // the tile is gathered word by word.  Lane = position in the slab: its filter cell f and channel c
        // are fixed per slab, and the 32 lanes of one load read neighbouring words of the few source rows
        // that one output row names (9 sectors instead of 32 for a 3-channel 3x3 filter).  Each warp covers
        // 32 rows with 32 independent loads held in registers, then stores them to the swizzled tile:
        // one round trip to L2 per slab.  (4-byte asynchronous copies cost the load/store unit about a
        // cycle per element, 4096 per slab, and starved the epilogue's loads and stores: the first
        // convolution of the benchmark took 8700 cycles per tile in both roles.)  k >= K (padding up to a
        // multiple of 32) and missing rows are zero.
        const int wq = warp - 4;
        for (int q = 0; q < nLoc; ++q, ring.next()) {
          const int s = slab0 + q, st = ring.idx;
          const int k = s * SLAB + lane;
          const bool kOk = k < P.K;
          const int f = kOk ? k / P.nIn : 0, c = k - f * P.nIn;
          // every load is unconditional (a safe address for a missing row): a select on a loaded value would
          // make the loads wait for one another
          int src[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int rl = wq * 32 + j, r = row0 + rl;
            if (POOL) { // the rules of the row that this tile row stands for, straight from global memory
              const int from = fromT[rl];
              src[j] = __ldg(kOk && from >= 0 ? P.rules + (long long)from * P.fs + f : &g_no_row);
            } else {
              src[j] = -1;
              if (kOk && r < rows) {
                if (P.rulesBytes > 0) src[j] = rulesT[rl * P.fs + f];
                else if (P.rules) src[j] = __ldg(P.rules + (long long)r * P.fs + f);
                else src[j] = r;
              }
            }
          }
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __ldg(src[j] >= 0 ? P.in + (long long)src[j] * P.nIn + c : g_zero_row);
          mbar_wait(emptyBar + 8 * st, ring.phase ^ 1, 1);
          unsigned char *dst0 = smem + (size_t)st * stageBytes + wq * 4096 + (lane & 3) * 4;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            *reinterpret_cast<float *>(dst0 + (j >> 3) * 1024 + (j & 7) * ROW_BYTES + (((lane >> 2) ^ (j & 7)) << 4)) = v[j];
          fence_async_smem(); // the tensor core reads the tile through the asynchronous proxy
          mbar_arrive(rawBar + 8 * st);
        }
        continue;
      }
      const float *rowPtr[8]; // start of the current filter cell's source row (nullptr: no row -> zero fill)
      int curF = -1;
      int f = slab0 * SLAB / P.nIn, c0 = slab0 * SLAB - f * P.nIn; // filter cell and channel offset of the slab, kept incrementally
      for (int q = 0; q < nLoc; ++q, ring.next(), c0 += SLAB) {
        const int st = ring.idx;
        if (c0 == P.nIn) { c0 = 0; ++f; }
        if (f != curF) { // the rule column changes every nIn/32 slabs
          curF = f;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rl = rbase + 16 * i, r = row0 + rl;
            int src = -1;
            if (POOL) { if (fromT[rl] >= 0) src = rulesT[rl * P.fs + f]; }
            else if (r < rows) {
              if (P.rulesBytes > 0) src = rulesT[rl * P.fs + f];
              else if (P.rules) src = __ldg(P.rules + (long long)r * P.fs + f);
              else src = r;
            }
            // a negative rule (or a row past the end) reads zeros
            rowPtr[i] = (src >= 0 ? P.in + (long long)src * P.nIn : g_zero_row) + chunk * 4;
          }
        }
        mbar_wait(emptyBar + 8 * st, ring.phase ^ 1, 1);
        const uint32_t dst = smem_u32(smem + (size_t)st * stageBytes) + rowOff;
#pragma unroll
        for (int i = 0; i < 8; ++i) cp_async16_full(dst + i * 2048, rowPtr[i] + c0);
        cp_async_arrive(rawBar + 8 * st);
      }
    }
    if (tailShare)
      epilogue_role<SPLIT, ACT, POOL>(P, epi, tmem, accFullBar, accEmptyBar, nItems, kSplit, rows, 0, 1, tailShare, 1, reinterpret_cast<float *>(smem));
  } else if (warp < 12 && epi2) {
    // the gather writes both images itself: these warps drain every second accumulator instead
    if (!SPLIT && !ATMEM) epilogue_role<false, ACT, POOL>(P, epi, tmem, accFullBar, accEmptyBar, nItems, kSplit, rows, 1, 2);
  } else if (warp < 12) {
    // ------------------------------------------------------------ split: lo = x - tf32(x)
    const int t = threadIdx.x - 256;
    Ring ring(P.stages), slot(P.atmem ? P.atmem : 1);
    for (int item = blockIdx.x; item < nItems; item += gridDim.x) {
      int tileM, tileN, slab0, nLoc;
      itemTile(item, tileM, tileN, slab0, nLoc);
      for (int q = 0; q < nLoc; ++q, ring.next()) {
        const int st = ring.idx;
        mbar_wait(rawBar + 8 * st, ring.phase, 5);
        unsigned char *aHi = smem + (size_t)st * stageBytes, *aLo = aHi + A_HALF;
        if (ATMEM) {
          // thread = row: its 32 values, 8 swizzled 16-byte chunks (rows r..r+7 of a quarter warp read 8
          // different chunk columns: no bank conflict)
          const unsigned char *rowp = aHi + (t >> 3) * 1024 + (t & 7) * ROW_BYTES;
          uint32_t v[32];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint4 x = *reinterpret_cast<const uint4 *>(rowp + ((c ^ (t & 7)) << 4));
            v[4 * c] = x.x; v[4 * c + 1] = x.y; v[4 * c + 2] = x.z; v[4 * c + 3] = x.w;
          }
          // bf16 operands: x = hi + lo with hi = bf16(x), lo = bf16(x - hi); two consecutive values of K share a 32-bit
          // column (the lower one in the lower half).  Converted BEFORE the wait for the slot, so that only the stores
          // to tensor memory stand between the MMAs that free the slot and the MMAs that read it next.
          uint32_t w16[32];
          if (P.bf16) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float a = __uint_as_float(v[2 * j]), b = __uint_as_float(v[2 * j + 1]);
              const __nv_bfloat162 hi2 = __floats2bfloat162_rn(a, b);
              const __nv_bfloat162 lo2 = __floats2bfloat162_rn(a - __low2float(hi2), b - __high2float(hi2));
              w16[j] = *reinterpret_cast<const uint32_t *>(&hi2);
              w16[16 + j] = *reinterpret_cast<const uint32_t *>(&lo2);
            }
          }
          mbar_wait(aEmptyBar + 8 * slot.idx, slot.phase ^ 1, 8); // the MMAs that read this slot have finished
          tc_fence_after();
          if (P.bf16) {
            // hi image at columns +0..15 of the slot, lo at +16..31
            const uint32_t taddr16 = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(P.aBase + slot.idx * 32);
#pragma unroll
            for (int g16 = 0; g16 < 2; ++g16)
              asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                           ::"r"(taddr16 + g16 * 16), "r"(w16[16 * g16]), "r"(w16[16 * g16 + 1]), "r"(w16[16 * g16 + 2]), "r"(w16[16 * g16 + 3]),
                             "r"(w16[16 * g16 + 4]), "r"(w16[16 * g16 + 5]), "r"(w16[16 * g16 + 6]), "r"(w16[16 * g16 + 7]), "r"(w16[16 * g16 + 8]),
                             "r"(w16[16 * g16 + 9]), "r"(w16[16 * g16 + 10]), "r"(w16[16 * g16 + 11]), "r"(w16[16 * g16 + 12]), "r"(w16[16 * g16 + 13]),
                             "r"(w16[16 * g16 + 14]), "r"(w16[16 * g16 + 15]) : "memory");
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            mbar_arrive(aFullBar + 8 * slot.idx);
            slot.next();
            continue;
          }
          // lanes 32*(warp % 4)..+31 belong to this warp; hi image at columns +0..31, lo at +32..63
          const uint32_t taddr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(P.aBase + slot.idx * 64);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t w[32];
#pragma unroll
            for (int k = 0; k < 32; ++k)
              w[k] = h == 0 ? v[k] : __float_as_uint(__uint_as_float(v[k]) - __uint_as_float(v[k] & 0xffffe000u));
#pragma unroll
            for (int g16 = 0; g16 < 2; ++g16)
              asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                           ::"r"(taddr + h * 32 + g16 * 16), "r"(w[16 * g16]), "r"(w[16 * g16 + 1]), "r"(w[16 * g16 + 2]), "r"(w[16 * g16 + 3]),
                             "r"(w[16 * g16 + 4]), "r"(w[16 * g16 + 5]), "r"(w[16 * g16 + 6]), "r"(w[16 * g16 + 7]), "r"(w[16 * g16 + 8]),
                             "r"(w[16 * g16 + 9]), "r"(w[16 * g16 + 10]), "r"(w[16 * g16 + 11]), "r"(w[16 * g16 + 12]), "r"(w[16 * g16 + 13]),
                             "r"(w[16 * g16 + 14]), "r"(w[16 * g16 + 15]) : "memory");
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          tc_fence_before();
          mbar_arrive(aFullBar + 8 * slot.idx);
          slot.next();
          continue;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int off = t * 16 + i * 2048; // the swizzle is the same in both images: work on raw offsets
          const float4 v = *reinterpret_cast<const float4 *>(aHi + off);
          // kind::tf32 reads the upper 19 bits of each fp32 (sign, exponent, 10 mantissa bits), so
          // the raw tile already is the "hi" operand; lo = x - hi is exact in fp32 and is cut to
          // tf32 the same way when it is read.
          float4 lo;
          lo.x = v.x - __uint_as_float(__float_as_uint(v.x) & 0xffffe000u);
          lo.y = v.y - __uint_as_float(__float_as_uint(v.y) & 0xffffe000u);
          lo.z = v.z - __uint_as_float(__float_as_uint(v.z) & 0xffffe000u);
          lo.w = v.w - __uint_as_float(__float_as_uint(v.w) & 0xffffe000u);
          *reinterpret_cast<float4 *>(aLo + off) = lo;
        }
        fence_async_smem(); // make the generic-proxy stores visible to the tensor core's reads
        mbar_arrive(fullBar + 8 * st);
      }
    }
    if (tailShare)
      epilogue_role<SPLIT, ACT, POOL>(P, epi, tmem, accFullBar, accEmptyBar, nItems, kSplit, rows, 0, 1, tailShare, 2,
                                      reinterpret_cast<float *>(smem + stageBytes));
  } else if (warp == 12) {
    // ------------------------------------------------------------ weight tiles by bulk copy
    if (lane == 0) {
      const uint32_t bytes = 2 * bHalf;
      Ring ring(P.stages);
      for (int item = blockIdx.x; item < nItems; item += gridDim.x) {
        int tileM, tileN, slab0, nLoc;
        itemTile(item, tileM, tileN, slab0, nLoc);
        const unsigned char *srcBase = P.packed + ((size_t)tileN * P.nSlabs + slab0) * bytes;
        for (int q = 0; q < nLoc; ++q, ring.next()) {
          const int st = ring.idx;
          mbar_wait(emptyBar + 8 * st, ring.phase ^ 1, 3);
          mbar_arrive_expect_tx(fullBar + 8 * st, bytes);
          bulk_g2s(smem_u32(smem + (size_t)st * stageBytes + aBytes), srcBase + (size_t)q * bytes, bytes, fullBar + 8 * st);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ MMA issue
    if (lane == 0) {
      int n = 0;
      Ring ring(P.stages), slot(P.atmem ? P.atmem : 1);
      for (int item = blockIdx.x; item < nItems; item += gridDim.x, ++n) {
        int tileM, tileN, slab0, nLoc;
        itemTile(item, tileM, tileN, slab0, nLoc);
        const int ab = n & 1;
        mbar_wait(accEmptyBar + 8 * ab, ((n >> 1) & 1) ^ 1, 6); // the epilogue has drained this accumulator
        tc_fence_after();
        const uint32_t acc = tmem + (uint32_t)(ab * P.accStride);
        for (int q = 0; q < nLoc; ++q, ring.next()) {
          const int st = ring.idx;
          mbar_wait(fullBar + 8 * st, ring.phase, 4);
          tc_fence_after();
          const uint32_t aHi = smem_u32(smem + (size_t)st * stageBytes), aLo = aHi + A_HALF;
          const uint32_t bHi = aHi + aBytes, bLo = bHi + bHalf;
          const uint64_t dAhi = smem_desc(aHi), dAlo = smem_desc(aLo), dBhi = smem_desc(bHi), dBlo = smem_desc(bLo);
          if (ATMEM) {
            mbar_wait(aFullBar + 8 * slot.idx, slot.phase, 9);
            tc_fence_after();
            if (P.bf16) { // two K = 16 steps per slab and product; A advances 8 columns, B 32 bytes per step
              const uint32_t t16Hi = tmem + (uint32_t)(P.aBase + slot.idx * 32), t16Lo = t16Hi + 16;
              const uint64_t eBhi = smem_desc64(bHi), eBlo = smem_desc64(bLo);
#pragma unroll
              for (int k = 0; k < 2; ++k) mma_bf16_ts(acc, t16Lo + 8 * k, eBhi + 2 * k, P.idesc, (q | k) != 0);
#pragma unroll
              for (int k = 0; k < 2; ++k) mma_bf16_ts(acc, t16Hi + 8 * k, eBlo + 2 * k, P.idesc, 1);
#pragma unroll
              for (int k = 0; k < 2; ++k) mma_bf16_ts(acc, t16Hi + 8 * k, eBhi + 2 * k, P.idesc, 1);
              mma_commit(emptyBar + 8 * st);
              mma_commit(aEmptyBar + 8 * slot.idx);
              slot.next();
              continue;
            }
            const uint32_t tHi = tmem + (uint32_t)(P.aBase + slot.idx * 64), tLo = tHi + 32;
#pragma unroll
            for (int k = 0; k < 4; ++k) mma_tf32_ts(acc, tLo + 8 * k, dBhi + 2 * k, P.idesc, (q | k) != 0);
#pragma unroll
            for (int k = 0; k < 4; ++k) mma_tf32_ts(acc, tHi + 8 * k, dBlo + 2 * k, P.idesc, 1);
#pragma unroll
            for (int k = 0; k < 4; ++k) mma_tf32_ts(acc, tHi + 8 * k, dBhi + 2 * k, P.idesc, 1);
            mma_commit(emptyBar + 8 * st);
            mma_commit(aEmptyBar + 8 * slot.idx);
            slot.next();
            continue;
          }
          // small cross terms first, the dominant hi*hi product last
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_tf32(acc, dAlo + 2 * k, dBhi + 2 * k, P.idesc, (q | k) != 0);
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_tf32(acc, dAhi + 2 * k, dBlo + 2 * k, P.idesc, 1);
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_tf32(acc, dAhi + 2 * k, dBhi + 2 * k, P.idesc, 1);
          mma_commit(emptyBar + 8 * st); // frees the stage once these MMAs have read it
        }
        mma_commit(accFullBar + 8 * ab);
      }
    }
  }
  __syncwarp(); // the single-thread roles rejoin their warps before the block-wide barrier
  __syncthreads();
  if (warp == 13) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)P.tmemCols) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------
// bf16 operands (kind::f16), fp32 accumulation.  PASSES == 3: x = hi + lo with hi = bf16(x),
// lo = bf16(x - hi) for both operands and A_lo*B_hi + A_hi*B_lo + A_hi*B_hi ("3xBF16": products
// carry 16 mantissa bits, relative error about 2^-16 per product, half the tensor-pipe time and
// 5/8 of the operand bytes of 3xTF32).  PASSES == 1: plain bf16 (A_hi*B_hi only).
//
// Same roles as k_conv_nin_tc, but the gather lands in a ring of raw fp32 entries (128 rows x 32
// values) that is separate from the operand stages (128 rows x 64 bf16 = two raw entries), so
// gathers stay in flight while earlier slabs are converted and multiplied:
//   warps 4-7   gather into raw entry e: wait rawEmpty[e], cp.async, arrival on rawFull[e]
//   warps 8-15  convert: wait empty[stage] once, then per half: wait rawFull[e], read fp32,
//               write the bf16 hi (and lo) 16-byte chunks of the K-major SWIZZLE_128B operand
//               rows, arrive on rawEmpty[e]; after both halves fence to the async proxy and
//               arrive on full[stage]
//   warp 16     weight block of the stage (hi [and lo] image, packed by tc_pack) by bulk copy
//   warp 17     per stage PASSES x 4 tcgen05.mma (M=128, N=BN, K=16), commit onto empty[stage]
constexpr int MAX_RAW = 8;
constexpr int CONVERT_THREADS = 256;                       // warps 8-15
constexpr int MMA_WARP16 = 8 + CONVERT_THREADS / 32 + 1;   // then the weight warp, then the MMA warp
constexpr int NUM_THREADS16 = (MMA_WARP16 + 1) * 32;

__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) { // a at the lower address
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t *>(&v);
}
__device__ __forceinline__ float bf16_hi(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

template <bool SPLIT, int ACT, int PASSES>
__global__ void __launch_bounds__(NUM_THREADS16, 1) k_conv_nin_tc16(const Params P) {
  extern __shared__ unsigned char smem_raw[];
  int *rulesS = reinterpret_cast<int *>(smem_raw);
  unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + (P.rulesDouble ? 2 : 1) * P.rulesBytes + 1023) & ~(uintptr_t)1023);
  const int bImg = P.BN * ROW_BYTES;                       // one weight image: BN rows x 64 bf16
  const int aBytes = (PASSES == 3 ? 2 : 1) * A_HALF;       // A_hi [, A_lo]
  const int stageBytes = aBytes + (PASSES == 3 ? 2 : 1) * bImg;
  unsigned char *rawRing = smem;                           // rawEntries x 16 KB
  unsigned char *stageRing = smem + (size_t)P.rawEntries * A_HALF;
  float *epi = reinterpret_cast<float *>(stageRing + (size_t)P.stages * stageBytes);
  __shared__ __align__(8) uint64_t bars[2 * MAX_RAW + 2 * MAX_STAGES + 4];
  __shared__ uint32_t tmemBase;
  const uint32_t rawFullBar = smem_u32(&bars[0]), rawEmptyBar = smem_u32(&bars[MAX_RAW]), fullBar = smem_u32(&bars[2 * MAX_RAW]),
                 emptyBar = smem_u32(&bars[2 * MAX_RAW + MAX_STAGES]), accFullBar = smem_u32(&bars[2 * MAX_RAW + 2 * MAX_STAGES]),
                 accEmptyBar = smem_u32(&bars[2 * MAX_RAW + 2 * MAX_STAGES + 2]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kSplit = SPLIT ? P.kSplit : 1;
  const int nItems = P.mTiles * P.nTiles * kSplit;

  if (threadIdx.x == 0) {
    for (int e = 0; e < P.rawEntries; ++e) { mbar_init(rawFullBar + 8 * e, 128); mbar_init(rawEmptyBar + 8 * e, CONVERT_THREADS); }
    for (int st = 0; st < P.stages; ++st) {
      mbar_init(fullBar + 8 * st, CONVERT_THREADS + 1); // the convert threads + the weight copy
      mbar_init(emptyBar + 8 * st, 1);      // tcgen05.commit
    }
    for (int a = 0; a < 2; ++a) { mbar_init(accFullBar + 8 * a, 1); mbar_init(accEmptyBar + 8 * a, 128); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP16) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmemBase)), "r"((uint32_t)P.tmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmemBase;

  // work item -> tile and its range of 64-wide K stages
  auto itemTile = [&](int item, int &tileM, int &tileN, int &stage0, int &nLoc) {
    const int tileId = SPLIT ? item / kSplit : item, split = SPLIT ? item - tileId * kSplit : 0;
    tileN = tileId % P.nTiles; tileM = tileId / P.nTiles;
    stage0 = SPLIT ? split * P.nStages64 / kSplit : 0;
    nLoc = SPLIT ? (split + 1) * P.nStages64 / kSplit - stage0 : P.nStages64;
  };

  if (warp < 4) {
    epilogue_role<SPLIT, ACT>(P, epi, tmem, accFullBar, accEmptyBar, nItems, kSplit, P.rows);
  } else if (warp < 8) {
    // ------------------------------------------------------------ gather into the raw ring
    const int t = threadIdx.x - 128, chunk = t & 7, rbase = t >> 3;
    const uint32_t rowOff = (rbase >> 3) * 1024 + (rbase & 7) * ROW_BYTES + ((chunk ^ (rbase & 7)) << 4);
    int nItem = 0;
    Ring raw(P.rawEntries); // raw entries: 32 values of K each
    auto stage_rules_async = [&](int item, int buf) {
      int tileM, tileN, stage0, nLoc;
      itemTile(item, tileM, tileN, stage0, nLoc);
      const long long first = (long long)tileM * BM * P.fs, total = (long long)P.rows * P.fs;
      const uint32_t dst = smem_u32(rulesS) + buf * P.rulesBytes;
      for (int ch = t; ch < BM * P.fs / 4; ch += 128) {
        const long long left = total - (first + ch * 4);
        const uint32_t bytes = left >= 4 ? 16u : left > 0 ? (uint32_t)left * 4u : 0u;
        cp_async16(dst + ch * 16, bytes ? (const void *)(P.rules + first + ch * 4) : (const void *)P.rules, bytes);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (P.rulesDouble && (int)blockIdx.x < nItems) stage_rules_async(blockIdx.x, 0);
    for (int item = blockIdx.x; item < nItems; item += gridDim.x, ++nItem) {
      int tileM, tileN, stage0, nLoc;
      itemTile(item, tileM, tileN, stage0, nLoc);
      const int row0 = tileM * BM;
      const int *rulesT = rulesS;
      if (P.rulesDouble) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        asm volatile("bar.sync 2, 128;" ::: "memory");
        rulesT = rulesS + (nItem & 1) * (P.rulesBytes >> 2);
        if (item + (int)gridDim.x < nItems) stage_rules_async(item + gridDim.x, (nItem + 1) & 1);
      } else if (P.rulesBytes > 0) {
        asm volatile("bar.sync 2, 128;" ::: "memory");
        const int nr = BM * P.fs;
        for (int e = t; e < nr; e += 128) rulesS[e] = __ldg(P.rules + min((long long)row0 * P.fs + e, (long long)P.rows * P.fs - 1));
        asm volatile("bar.sync 2, 128;" ::: "memory");
      }
      const float *rowPtr[8];
      int curF = -1;
      const int wq = warp - 4;
      int f16 = 2 * stage0 * SLAB / P.nIn, c0 = 2 * stage0 * SLAB - f16 * P.nIn - SLAB; // 16-byte path: cell and channel offset, kept incrementally
      for (int q = 0; q < 2 * nLoc; ++q) {
        const int s = 2 * stage0 + q, e = raw.idx; // s: 32-wide slab of K
        if (s >= P.nSlabs) break; // the second half of the last stage lies past K: the convert warps write zeros
        c0 += SLAB;
        if (c0 >= P.nIn) { c0 -= P.nIn; ++f16; }
        mbar_wait(rawEmptyBar + 8 * e, raw.phase ^ 1, 1);
        const uint32_t entry = smem_u32(rawRing + (size_t)e * A_HALF);
        if (P.generic) { // any nIn: 4-byte copies, lane = position in the slab (see k_conv_nin_tc)
          const int k = s * SLAB + lane;
          const bool kOk = k < P.K;
          const int f = kOk ? k / P.nIn : 0, c = k - f * P.nIn;
          const uint32_t dst0 = entry + (uint32_t)wq * 4096 + (lane & 3) * 4;
#pragma unroll 1
          for (int i0 = 0; i0 < 32; i0 += 8) {
            int src[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int rl = wq * 32 + i0 + j, r = row0 + rl;
              src[j] = -1;
              if (kOk && r < P.rows) {
                if (P.rulesBytes > 0) src[j] = rulesT[rl * P.fs + f];
                else if (P.rules) src[j] = __ldg(P.rules + (long long)r * P.fs + f);
                else src[j] = r;
              }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t dst = dst0 + (i0 >> 3) * 1024 + j * ROW_BYTES + (((lane >> 2) ^ j) << 4);
              cp_async4(dst, src[j] >= 0 ? (const void *)(P.in + (long long)src[j] * P.nIn + c) : (const void *)P.in, src[j] >= 0 ? 4u : 0u);
            }
          }
        } else {
          // (one 128-byte bulk copy per row and slab instead of these per-lane copies was measured 1.4-1.8x
          // slower: the copy engine retires a small bulk copy about every 25 cycles per SM)
          const int f = f16;
          if (f != curF) { // the rule column changes every nIn/32 slabs
            curF = f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rl = rbase + 16 * i, r = row0 + rl;
              int src = -1;
              if (r < P.rows) {
                if (P.rulesBytes > 0) src = rulesT[rl * P.fs + f];
                else if (P.rules) src = __ldg(P.rules + (long long)r * P.fs + f);
                else src = r;
              }
              rowPtr[i] = (src >= 0 ? P.in + (long long)src * P.nIn : g_zero_row) + chunk * 4;
            }
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) cp_async16_full(entry + rowOff + i * 2048, rowPtr[i] + c0);
        }
        cp_async_arrive(rawFullBar + 8 * e);
        raw.next();
      }
    }
  } else if (warp < 8 + CONVERT_THREADS / 32) {
    // ------------------------------------------------------------ convert fp32 -> bf16 hi [, lo]
    const int t = threadIdx.x - 256;
    // 8 consecutive threads take the four 8-value groups of rows r and r + 4: their 16-byte stores
    // hit eight different chunks (the swizzle term differs in bit 2), and the second row reads its
    // two fp32 chunks in the opposite order, so loads and stores are free of bank conflicts
    const int kg = t & 3, hiRow = (t >> 2) & 1, qd = (t >> 3) & 15, part = t >> 7;
    Ring raw(P.rawEntries), ring(P.stages); // raw entries, operand stages
    for (int item = blockIdx.x; item < nItems; item += gridDim.x) {
      int tileM, tileN, stage0, nLoc;
      itemTile(item, tileM, tileN, stage0, nLoc);
      for (int q = 0; q < nLoc; ++q, ring.next()) {
        const int st = ring.idx;
        mbar_wait(emptyBar + 8 * st, ring.phase ^ 1, 7); // the tensor core has finished with this stage
        unsigned char *aHi = stageRing + (size_t)st * stageBytes, *aLo = aHi + A_HALF;
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          if (2 * (stage0 + q) + h >= P.nSlabs) { // K ends inside this stage: the upper half of the operand rows is zero
#pragma unroll
            for (int ii = 0; ii < 512 / CONVERT_THREADS; ++ii) {
              const int i = part * (512 / CONVERT_THREADS) + ii;
              const int r = (qd >> 2) * 32 + i * 8 + (qd & 3) + 4 * hiRow;
              const int off = (r >> 3) * 1024 + (r & 7) * ROW_BYTES + (((h * 4 + kg) ^ (r & 7)) << 4);
              *reinterpret_cast<uint4 *>(aHi + off) = make_uint4(0u, 0u, 0u, 0u);
              if (PASSES == 3) *reinterpret_cast<uint4 *>(aLo + off) = make_uint4(0u, 0u, 0u, 0u);
            }
            continue;
          }
          const int e = raw.idx;
          mbar_wait(rawFullBar + 8 * e, raw.phase, 5);
          const unsigned char *rawp = rawRing + (size_t)e * A_HALF;
#pragma unroll
          for (int ii = 0; ii < 512 / CONVERT_THREADS; ++ii) {
            // a group = 8 consecutive values of K of one row: two 16-byte fp32 chunks in, one 16-byte
            // bf16 chunk out (per image)
            const int i = part * (512 / CONVERT_THREADS) + ii;
            const int r = (qd >> 2) * 32 + i * 8 + (qd & 3) + 4 * hiRow;
            const unsigned char *rowp = rawp + (r >> 3) * 1024 + (r & 7) * ROW_BYTES;
            const float4 va = *reinterpret_cast<const float4 *>(rowp + (((2 * kg + hiRow) ^ (r & 7)) << 4));
            const float4 vb = *reinterpret_cast<const float4 *>(rowp + (((2 * kg + 1 - hiRow) ^ (r & 7)) << 4));
            const float4 v0 = hiRow ? vb : va, v1 = hiRow ? va : vb;
            const int off = (r >> 3) * 1024 + (r & 7) * ROW_BYTES + (((h * 4 + kg) ^ (r & 7)) << 4);
            const float h0 = bf16_hi(v0.x), h1 = bf16_hi(v0.y), h2 = bf16_hi(v0.z), h3 = bf16_hi(v0.w);
            const float h4 = bf16_hi(v1.x), h5 = bf16_hi(v1.y), h6 = bf16_hi(v1.z), h7 = bf16_hi(v1.w);
            *reinterpret_cast<uint4 *>(aHi + off) = make_uint4(pack_bf16(h0, h1), pack_bf16(h2, h3), pack_bf16(h4, h5), pack_bf16(h6, h7));
            if (PASSES == 3)
              *reinterpret_cast<uint4 *>(aLo + off) = make_uint4(pack_bf16(v0.x - h0, v0.y - h1), pack_bf16(v0.z - h2, v0.w - h3),
                                                                 pack_bf16(v1.x - h4, v1.y - h5), pack_bf16(v1.z - h6, v1.w - h7));
          }
          mbar_arrive(rawEmptyBar + 8 * e); // the raw entry may be overwritten
          raw.next();
        }
        fence_async_smem(); // make the generic-proxy stores visible to the tensor core's reads
        mbar_arrive(fullBar + 8 * st);
      }
    }
  } else if (warp == MMA_WARP16 - 1) {
    // ------------------------------------------------------------ weight blocks by bulk copy
    if (lane == 0) {
      const uint32_t bytes = (PASSES == 3 ? 2 : 1) * bImg;
      Ring ring(P.stages);
      for (int item = blockIdx.x; item < nItems; item += gridDim.x) {
        int tileM, tileN, stage0, nLoc;
        itemTile(item, tileM, tileN, stage0, nLoc);
        const unsigned char *srcBase = P.packed + ((size_t)tileN * P.nStages64 + stage0) * bytes;
        for (int q = 0; q < nLoc; ++q, ring.next()) {
          const int st = ring.idx;
          mbar_wait(emptyBar + 8 * st, ring.phase ^ 1, 3);
          mbar_arrive_expect_tx(fullBar + 8 * st, bytes);
          bulk_g2s(smem_u32(stageRing + (size_t)st * stageBytes + aBytes), srcBase + (size_t)q * bytes, bytes, fullBar + 8 * st);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ MMA issue
    if (lane == 0) {
      int n = 0;
      Ring ring(P.stages);
      for (int item = blockIdx.x; item < nItems; item += gridDim.x, ++n) {
        int tileM, tileN, stage0, nLoc;
        itemTile(item, tileM, tileN, stage0, nLoc);
        const int ab = n & 1;
        mbar_wait(accEmptyBar + 8 * ab, ((n >> 1) & 1) ^ 1, 6);
        tc_fence_after();
        const uint32_t acc = tmem + (uint32_t)(ab * P.accStride);
        for (int q = 0; q < nLoc; ++q, ring.next()) {
          const int st = ring.idx;
          mbar_wait(fullBar + 8 * st, ring.phase, 4);
          tc_fence_after();
          const uint32_t aHi = smem_u32(stageRing + (size_t)st * stageBytes), aLo = aHi + A_HALF;
          const uint32_t bHi = aHi + aBytes, bLo = bHi + bImg;
          const uint64_t dAhi = smem_desc(aHi), dAlo = smem_desc(aLo), dBhi = smem_desc(bHi), dBlo = smem_desc(bLo);
          if (PASSES == 3) { // small cross terms first, the dominant hi*hi product last
#pragma unroll
            for (int k = 0; k < 4; ++k) mma_bf16(acc, dAlo + 2 * k, dBhi + 2 * k, P.idesc, (q | k) != 0);
#pragma unroll
            for (int k = 0; k < 4; ++k) mma_bf16(acc, dAhi + 2 * k, dBlo + 2 * k, P.idesc, 1);
#pragma unroll
            for (int k = 0; k < 4; ++k) mma_bf16(acc, dAhi + 2 * k, dBhi + 2 * k, P.idesc, 1);
          } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) mma_bf16(acc, dAhi + 2 * k, dBhi + 2 * k, P.idesc, (q | k) != 0);
          }
          mma_commit(emptyBar + 8 * st);
        }
        mma_commit(accFullBar + 8 * ab);
      }
    }
  }
  __syncwarp();
  __syncthreads();
  if (warp == MMA_WARP16) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)P.tmemCols) : "memory");
  }
}

// W[K x N] row-major -> per (column tile, 64-wide K stage) one contiguous block: the bf16 hi image
// [BN x 64] (K-major, SWIZZLE_128B order), then for three passes the lo image.
__global__ void k_pack_bf16(const float *__restrict__ W, int K, int N, int BN, int nTiles, int nStages64, int passes,
                            unsigned short *__restrict__ packed) {
  const long long total = (long long)nTiles * nStages64 * BN * 64;
  const int images = passes == 3 ? 2 : 1;
  for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < total; q += (long long)gridDim.x * blockDim.x) {
    const int kl = (int)(q % 64);
    const int nl = (int)((q / 64) % BN);
    const long long blk = q / (64LL * BN);
    const int stage = (int)(blk % nStages64), tile = (int)(blk / nStages64);
    const int k = stage * 64 + kl, n = tile * BN + nl;
    const float w = (k < K && n < N) ? W[(long long)k * N + n] : 0.f;
    const __nv_bfloat16 hi = __float2bfloat16_rn(w), lo = __float2bfloat16_rn(w - __bfloat162float(hi));
    const int off = (nl >> 3) * 1024 + (nl & 7) * ROW_BYTES + ((((kl >> 3) ^ (nl & 7))) << 4) + (kl & 7) * 2;
    unsigned short *base = packed + blk * ((long long)images * BN * 64);
    base[off >> 1] = *reinterpret_cast<const unsigned short *>(&hi);
    if (images == 2) base[BN * 64 + (off >> 1)] = *reinterpret_cast<const unsigned short *>(&lo);
  }
}

// W[K x N] row-major -> per (column tile, 32-wide K slab) one contiguous block: the bf16 hi image [BN x 32] (K-major rows of
// 64 bytes in SWIZZLE_64B order: 16-byte chunk c of row n sits at chunk c ^ ((n >> 1) & 3)), then the lo image.
__global__ void k_pack_bf16_slab(const float *__restrict__ W, int K, int N, int BN, int nTiles, int nSlabs, unsigned short *__restrict__ packed) {
  const long long total = (long long)nTiles * nSlabs * BN * SLAB;
  for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < total; q += (long long)gridDim.x * blockDim.x) {
    const int kl = (int)(q % SLAB);
    const int nl = (int)((q / SLAB) % BN);
    const long long blk = q / ((long long)SLAB * BN);
    const int slab = (int)(blk % nSlabs), tile = (int)(blk / nSlabs);
    const int k = slab * SLAB + kl, n = tile * BN + nl;
    const float w = (k < K && n < N) ? W[(long long)k * N + n] : 0.f;
    const __nv_bfloat16 hi = __float2bfloat16_rn(w), lo = __float2bfloat16_rn(w - __bfloat162float(hi));
    const int off = (nl >> 3) * 512 + (nl & 7) * 64 + ((((kl >> 3) ^ ((nl >> 1) & 3))) << 4) + (kl & 7) * 2;
    unsigned short *base = packed + blk * (2LL * BN * SLAB);
    base[off >> 1] = *reinterpret_cast<const unsigned short *>(&hi);
    base[BN * SLAB + (off >> 1)] = *reinterpret_cast<const unsigned short *>(&lo);
  }
}

// W[K x N] row-major -> per (column tile, K slab) one contiguous block: the hi image then the lo
// image of the [BN x 32] K-major tile, already in the SWIZZLE_128B shared-memory order.
__global__ void k_pack_tf32(const float *__restrict__ W, int K, int N, int BN, int nTiles, int nSlabs, float *__restrict__ packed) {
  const long long total = (long long)nTiles * nSlabs * BN * SLAB;
  for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < total; q += (long long)gridDim.x * blockDim.x) {
    const int kl = (int)(q % SLAB);
    const int nl = (int)((q / SLAB) % BN);
    const long long blk = q / ((long long)SLAB * BN);
    const int slab = (int)(blk % nSlabs), tile = (int)(blk / nSlabs);
    const int k = slab * SLAB + kl, n = tile * BN + nl;
    const float w = (k < K && n < N) ? W[(long long)k * N + n] : 0.f;
    const float hi = to_tf32(w), lo = to_tf32(w - hi);
    const int off = (nl >> 3) * 1024 + (nl & 7) * ROW_BYTES + ((((kl >> 2) ^ (nl & 7))) << 4) + (kl & 3) * 4;
    float *base = packed + blk * (2LL * BN * SLAB);
    base[off >> 2] = hi;
    base[BN * SLAB + (off >> 2)] = lo;
  }
}

// Sum the K-split partials in split order (deterministic), then bias, dropout scale, activation.
template <int ACT>
__global__ void k_splitk_finish(const float *__restrict__ partial, int kSplit, long long rows, int N, const float *__restrict__ bias,
                                const float *__restrict__ prelu, float p, float *__restrict__ out) {
  dependents_may_launch();
  wait_for_prior_grids(); // the partial sums come from the kernel in front
  const long long n4 = rows * N / 4;
  const int nv = N >> 2;
  for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < n4; q += (long long)gridDim.x * blockDim.x) {
    float4 a = reinterpret_cast<const float4 *>(partial)[q];
    for (int s = 1; s < kSplit; ++s) {
      const float4 b = reinterpret_cast<const float4 *>(partial)[(long long)s * n4 + q];
      a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    }
    const int v = (int)(q % nv);
    const float4 b4 = __ldg(reinterpret_cast<const float4 *>(bias) + v);
    float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (prelu) s4 = __ldg(reinterpret_cast<const float4 *>(prelu) + v);
    float4 o;
    o.x = activate_t<ACT>(p * a.x + p * b4.x, s4.x); o.y = activate_t<ACT>(p * a.y + p * b4.y, s4.y);
    o.z = activate_t<ACT>(p * a.z + p * b4.z, s4.z); o.w = activate_t<ACT>(p * a.w + p * b4.w, s4.w);
    reinterpret_cast<float4 *>(out)[q] = o;
  }
}

// The same with a non-overlapping max pooling applied on the way (MaxPoolingLayer.cu:9-35): one thread per pooled
// row and four columns; every cell's partial sums are added in split order and finished exactly as above, the
// first maximum wins, the choice is the flat index row * N + column of the learnt layer's (unwritten) output.
template <int ACT>
__global__ void k_splitk_finish_pool(const float *__restrict__ partial, int kSplit, long long rows, int N, const float *__restrict__ bias,
                                     const float *__restrict__ prelu, float p, const int *__restrict__ poolRules, int cells, int rowsPool,
                                     float *__restrict__ out, int *__restrict__ choices) {
  dependents_may_launch();
  wait_for_prior_grids(); // the partial sums come from the kernel in front
  const int nv = N >> 2;
  const long long n4 = rows * nv, total = (long long)rowsPool * nv;
  for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < total; q += (long long)gridDim.x * blockDim.x) {
    const int w = (int)(q / nv), v = (int)(q - (long long)w * nv);
    const float4 b4 = __ldg(reinterpret_cast<const float4 *>(bias) + v);
    float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (prelu) s4 = __ldg(reinterpret_cast<const float4 *>(prelu) + v);
    float best[4] = {0.f, 0.f, 0.f, 0.f};
    int idx[4] = {-1, -1, -1, -1};
    bool none = true;
    for (int c = 0; c < cells; ++c) {
      const int from = __ldg(poolRules + (long long)w * cells + c);
      if (from < 0) continue;
      const long long src = (long long)from * nv + v;
      float4 a = reinterpret_cast<const float4 *>(partial)[src];
      for (int sp = 1; sp < kSplit; ++sp) {
        const float4 b = reinterpret_cast<const float4 *>(partial)[(long long)sp * n4 + src];
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
      }
      const float o[4] = {activate_t<ACT>(p * a.x + p * b4.x, s4.x), activate_t<ACT>(p * a.y + p * b4.y, s4.y),
                          activate_t<ACT>(p * a.z + p * b4.z, s4.z), activate_t<ACT>(p * a.w + p * b4.w, s4.w)};
      const int base = from * N + 4 * v;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (none || best[k] < o[k]) { best[k] = o[k]; idx[k] = base + k; }
      none = false;
    }
    reinterpret_cast<float4 *>(out)[q] = make_float4(best[0], best[1], best[2], best[3]);
    reinterpret_cast<int4 *>(choices)[q] = make_int4(idx[0], idx[1], idx[2], idx[3]);
  }
}

// The K-split finish of a layer of few rows with the small learnt layer behind it (the classifier of a network:
// NetworkInNetworkLayer.cu:187-201 twice, SigmoidLayer.cu:160-177 for its softmax) applied on the way: one CTA per
// row adds the partial sums in split order, finishes the row exactly as k_splitk_finish does (and writes it), keeps
// it in shared memory and multiplies it with W2[N x N2], N2 <= 16, in fp32 on the CUDA cores.
template <int ACT>
__global__ void __launch_bounds__(256)
k_splitk_finish_nin(const float *__restrict__ partial, int kSplit, long long rows, int N, const float *__restrict__ bias,
                    const float *__restrict__ prelu, float p, float *__restrict__ mid, const float *__restrict__ W2,
                    const float *__restrict__ B2, const float *__restrict__ prelu2, int N2, float p2, int act2, float *__restrict__ out2) {
  extern __shared__ float xS[]; // the finished row, then 8 x 16 partial dot products
  float *red = xS + N;
  dependents_may_launch();
  wait_for_prior_grids(); // the partial sums come from the kernel in front
  const int nv = N >> 2, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long n4 = rows * nv;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    __syncthreads();
    for (int v = threadIdx.x; v < nv; v += 256) {
      const long long q = row * nv + v;
      // eight partial sums are requested at a time (independent loads), then added in split order
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int sp0 = 0; sp0 < kSplit; sp0 += 8) {
        float4 t[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) t[u] = reinterpret_cast<const float4 *>(partial)[(long long)min(sp0 + u, kSplit - 1) * n4 + q];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (sp0 + u == 0) a = t[u];
          else if (sp0 + u < kSplit) { a.x += t[u].x; a.y += t[u].y; a.z += t[u].z; a.w += t[u].w; }
        }
      }
      const float4 b4 = __ldg(reinterpret_cast<const float4 *>(bias) + v);
      float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
      if (prelu) s4 = __ldg(reinterpret_cast<const float4 *>(prelu) + v);
      float4 o;
      o.x = activate_t<ACT>(p * a.x + p * b4.x, s4.x); o.y = activate_t<ACT>(p * a.y + p * b4.y, s4.y);
      o.z = activate_t<ACT>(p * a.z + p * b4.z, s4.z); o.w = activate_t<ACT>(p * a.w + p * b4.w, s4.w);
      if (mid) reinterpret_cast<float4 *>(mid)[q] = o;
      reinterpret_cast<float4 *>(xS)[v] = o;
    }
    __syncthreads();
    float acc[16];
#pragma unroll
    for (int n = 0; n < 16; ++n) acc[n] = 0.f;
    for (int k0 = threadIdx.x; k0 < N; k0 += 256 * 3) { // three rows of W2 requested at a time
      float w[3][16];
#pragma unroll
      for (int u = 0; u < 3; ++u) {
        const float *wr = W2 + (long long)min(k0 + 256 * u, N - 1) * N2;
#pragma unroll
        for (int n = 0; n < 16; ++n) w[u][n] = __ldg(wr + (n < N2 ? n : 0));
      }
#pragma unroll
      for (int u = 0; u < 3; ++u) {
        const float x = k0 + 256 * u < N ? xS[k0 + 256 * u] : 0.f;
#pragma unroll
        for (int n = 0; n < 16; ++n) acc[n] = fmaf(x, w[u][n], acc[n]);
      }
    }
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      float v = acc[n];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) red[warp * 16 + n] = v;
    }
    __syncthreads();
    if (warp == 0) {
      const bool valid = lane < N2;
      float s = 0.f;
      if (valid)
        for (int w = 0; w < 8; ++w) s += red[w * 16 + lane];
      float v = valid ? p2 * s + p2 * __ldg(B2 + lane) : -10000.0f;
      if (act2 == SCN_SOFTMAX) { // SigmoidLayer.cu:160-177: running maximum from -10000
        float mx = fmaxf(v, -10000.0f);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float e = valid ? expf(v - mx) : 0.f, sum = e;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        v = e / sum;
      } else if (valid) {
        v = activate(v, act2, prelu2 ? __ldg(prelu2 + lane) : 0.f);
      }
      if (valid) out2[row * N2 + lane] = v;
    }
  }
}

// How many CTAs share one output tile's K range: only when the tiles alone leave most SMs idle.
int choose_ksplit(int tiles, int nSlabs, long long rows, int N, size_t wsBytes) {
  const int sms = sm_count();
  if (tiles * 2 > sms || nSlabs < 8) return 1;
  int k = sms / tiles;
  if (k > nSlabs / 4) k = nSlabs / 4;
  if (k > 128) k = 128;
  while (k > 1 && (size_t)k * rows * N * sizeof(float) > wsBytes) --k;
  return k < 2 ? 1 : k;
}

struct Tiling { int BN, nTiles, nSlabs, stages, tmemCols, rulesBytes, rulesDouble, accStride, atmem, aBase, bf16; size_t smemBytes; };

// Word-wise gathers of at most this many input channels use the row-per-lane form with two epilogue groups
constexpr int ROWWISE_MAX_NIN = 4;

// Operand format of the three-product split (x = hi + lo for both operands, lo*lo dropped).  tf32 (SCN_PREC_3XTF32): 21
// mantissa bits per product.  SCN_PREC_SPLIT chooses per layer: bf16 operands (16 bits per product: measured 1.0-2.4e-5
// against fp64 on the benchmark networks, bound 1e-4; half the tensor-pipe time and half the weight bytes in shared
// memory) where the A operand is fed from tensor memory (K >= 128: four slabs or more), tf32 elsewhere.  The choice
// depends on K and N only, because the weights are packed for it before any batch is seen.
bool is_split(int precision) { return precision == SCN_PREC_3XTF32 || precision == SCN_PREC_SPLIT; }

// oneItem: no CTA gets more than one work item, so the second accumulator is never used and its columns can
// hold the A slots: the tensor-memory A path then reaches BN = 256.
bool make_tiling(int K, int N, int fs, bool haveRules, Tiling *t, bool allowBf16, bool oneItem = false, bool pool = false, bool epi2 = false) {
  if (K < 1 || N < 16) return false;
  t->nSlabs = (K + SLAB - 1) / SLAB; // the last slab is zero-padded
  t->bf16 = (allowBf16 && t->nSlabs >= 4 && !epi2) ? 1 : 0;
  const int epiBytes = epi2 ? 2 * EPI_BYTES + BM * 4 : EPI_BYTES;
  t->rulesBytes = (haveRules && fs <= 32 && !(epi2 && !pool)) ? BM * fs * 4 : 0; // (the row-per-lane gather reads rules from global memory)
  if (pool) { // fused max-pooling: staged rules are mandatory, two buffers, each followed by the tile's 128 row ids
    if (!t->rulesBytes) return false;
    t->rulesBytes += BM * 4;
  }
  // tf32: narrower tiles (so that every layer could use the tensor-memory A path) were measured slower: A is gathered once
  // per column tile.  bf16: two accumulators and two 32-column A slots must fit in 512 columns: tiles of at most 224.
  t->nTiles = t->bf16 ? (N + 223) / 224 : (N + 255) / 256;
  t->BN = ((N + t->nTiles - 1) / t->nTiles + 15) / 16 * 16;
  t->accStride = (t->BN + 31) / 32 * 32;
  // 64-column A slots in tensor memory beside the two accumulators: two (BN <= 192) or none, A then stays in
  // shared memory (a single slot serialises split and MMA and was measured slower); short K gains nothing
  t->aBase = (oneItem ? 1 : 2) * t->accStride;
  t->atmem = (t->nSlabs >= 4 && t->aBase + (t->bf16 ? 64 : 128) <= 512) ? 2 : 0;
  if (t->bf16 && !t->atmem) return false; // (cannot happen: BN <= 224)
  const int stageBytes = (t->atmem ? 1 : 2) * A_HALF + 2 * t->BN * (t->bf16 ? ROW_BYTES / 2 : ROW_BYTES);
  auto stagesWith = [&](int ruleBufs) {
    const int n = (int)((226 * 1024 - 1024 - ruleBufs * t->rulesBytes - epiBytes) / stageBytes);
    return n > MAX_STAGES ? MAX_STAGES : n;
  };
  const int stages = stagesWith(pool ? 2 : 1);
  if (stages < 2) return false;
  t->stages = stages;
  t->rulesDouble = (pool || (t->rulesBytes > 0 && stagesWith(2) == stages)) ? 1 : 0; // prefetch the next tile's rules if that costs no stage
  int cols = 32;
  while (cols < (t->atmem ? t->aBase + (t->bf16 ? 64 : 128) : 2 * t->accStride)) cols *= 2; // the accumulators [+ the A slots], at most 512 columns
  t->tmemCols = cols;
  t->smemBytes = (size_t)stages * stageBytes + 1024 + (size_t)(1 + t->rulesDouble) * t->rulesBytes + epiBytes;
  return true;
}

// bf16 kernels: operand stage = A images (16 KB each) + weight images (BN x 128 B each) for 64 values
// of K; the raw ring takes what is left (at least two entries = one stage's worth of gather).
// The column tiling depends on N and the number of passes only (weights are packed once, before any
// rulebook is known): the fewest column tiles for which two stages, two raw entries and 4 KB of
// staged rules (two buffers of a 2^2 filter) fit.  Stages, raw entries and rule buffers are then chosen per launch.
bool make_tiling16(int K, int N, int fs, bool haveRules, int passes, Tiling *t, int *rawEntries, int *nStages64) {
  if (K < 1 || N < 16) return false;
  const int images = passes == 3 ? 2 : 1;
  const int avail = 226 * 1024 - 1024 - EPI_BYTES;
  t->nSlabs = (K + SLAB - 1) / SLAB;
  *nStages64 = (t->nSlabs + 1) / 2;
  int nTiles = (N + 255) / 256, BN = 0, stageBytes = 0;
  for (;; ++nTiles) {
    BN = ((N + nTiles - 1) / nTiles + 15) / 16 * 16;
    stageBytes = images * (A_HALF + BN * ROW_BYTES);
    if (2 * stageBytes + 2 * A_HALF + 4 * 1024 <= avail) break;
    if (BN == 16) return false;
  }
  t->nTiles = nTiles; t->BN = BN;
  const int oneRules = (haveRules && fs <= 32) ? BM * fs * 4 : 0;
  int ruleBufs = oneRules ? 2 : 0;
  while (ruleBufs > 0 && 2 * stageBytes + 2 * A_HALF + ruleBufs * oneRules > avail) --ruleBufs;
  t->rulesBytes = ruleBufs ? oneRules : 0; // 0: the gather reads its rules from global memory
  t->rulesDouble = ruleBufs == 2 ? 1 : 0;
  const int room = avail - ruleBufs * oneRules;
  int stages = 3, raw = (room - 3 * stageBytes) / A_HALF; // three stages when two raw entries still fit
  if (raw < 2) { stages = 2; raw = (room - 2 * stageBytes) / A_HALF; }
  if (raw > MAX_RAW) raw = MAX_RAW;
  t->stages = stages; *rawEntries = raw;
  t->accStride = (BN + 31) / 32 * 32;
  int cols = 32;
  while (cols < 2 * t->accStride) cols *= 2;
  t->tmemCols = cols;
  t->smemBytes = (size_t)stages * stageBytes + (size_t)raw * A_HALF + 1024 + (size_t)ruleBufs * oneRules + EPI_BYTES;
  return true;
}

int passes_of(int precision) { return precision == SCN_PREC_3XBF16 ? 3 : precision == SCN_PREC_BF16 ? 1 : 0; }

} // namespace

bool tc_shape_ok(int fs, int nIn, int N, int precision) {
  Tiling t;
  if (nIn % SLAB == 0 && nIn > ZERO_ROW_FLOATS) return false; // the 16-byte gather reads missing rows from g_zero_row
  int raw, st64;
  if (passes_of(precision)) return N % 4 == 0 && make_tiling16(fs * nIn, N, fs, true, passes_of(precision), &t, &raw, &st64);
  if (!is_split(precision)) return false;
  return N % 4 == 0 && make_tiling(fs * nIn, N, fs, true, &t, precision == SCN_PREC_SPLIT);
}

size_t tc_packed_bytes(int K, int N, int precision) {
  Tiling t;
  if (const int passes = passes_of(precision)) {
    int raw, st64;
    if (!make_tiling16(K, N, 1, false, passes, &t, &raw, &st64)) return 0;
    return (size_t)t.nTiles * st64 * (passes == 3 ? 2 : 1) * t.BN * ROW_BYTES;
  }
  if (!is_split(precision)) return 0;
  if (!make_tiling(K, N, 1, false, &t, precision == SCN_PREC_SPLIT)) return 0;
  return (size_t)t.nTiles * t.nSlabs * 2 * t.BN * (t.bf16 ? ROW_BYTES / 2 : ROW_BYTES);
}

int tc_pack(const float *d_W, int K, int N, int precision, void *d_packed, cudaStream_t s) {
  Tiling t;
  if (const int passes = passes_of(precision)) {
    int raw, st64;
    if (!make_tiling16(K, N, 1, false, passes, &t, &raw, &st64)) return fail(SCN_ERR_UNSUPPORTED, "no tensor-core layout for this shape/precision");
    const long long total = (long long)t.nTiles * st64 * t.BN * 64;
    k_pack_bf16<<<grid_for(total, 256), 256, 0, s>>>(d_W, K, N, t.BN, t.nTiles, st64, passes, (unsigned short *)d_packed);
    SCN_LAUNCH_CHECK("k_pack_bf16");
    return SCN_OK;
  }
  if (!is_split(precision) || !make_tiling(K, N, 1, false, &t, precision == SCN_PREC_SPLIT)) return fail(SCN_ERR_UNSUPPORTED, "no tensor-core layout for this shape/precision");
  const long long total = (long long)t.nTiles * t.nSlabs * t.BN * SLAB;
  if (t.bf16) {
    k_pack_bf16_slab<<<grid_for(total, 256), 256, 0, s>>>(d_W, K, N, t.BN, t.nTiles, t.nSlabs, (unsigned short *)d_packed);
    SCN_LAUNCH_CHECK("k_pack_bf16_slab");
    return SCN_OK;
  }
  k_pack_tf32<<<grid_for(total, 256), 256, 0, s>>>(d_W, K, N, t.BN, t.nTiles, t.nSlabs, (float *)d_packed);
  SCN_LAUNCH_CHECK("k_pack_tf32");
  return SCN_OK;
}

size_t tc_workspace_bytes(int rows, int fs, int nIn, int N, int precision) {
  Tiling t;
  if (const int passes = passes_of(precision)) {
    int raw, st64;
    if (N % 4 != 0 || !make_tiling16(fs * nIn, N, fs, true, passes, &t, &raw, &st64)) return 0;
    const int k = choose_ksplit(((rows + BM - 1) / BM) * t.nTiles, st64 * 2, rows, N, (size_t)-1);
    return k > 1 ? (size_t)k * rows * N * sizeof(float) : 0;
  }
  if (!is_split(precision) || N % 4 != 0 || !make_tiling(fs * nIn, N, fs, true, &t, precision == SCN_PREC_SPLIT)) return 0;
  const int tiles = ((rows + BM - 1) / BM) * t.nTiles;
  const int k = choose_ksplit(tiles, t.nSlabs, rows, N, (size_t)-1);
  return k > 1 ? (size_t)k * rows * N * sizeof(float) : 0;
}

int tc_launch(const float *d_in, const int *d_rules, int rows, int fs, int nIn, const void *d_packed, const float *d_B,
              const float *d_prelu, int N, float p, int act, int precision, float *d_out, void *d_ws, size_t wsBytes,
              cudaStream_t s, const int *d_rows, const int *d_pool_rules, int pool_cells, int *d_choices, int rows_unpooled,
              const FinishPool *finish_pool, const FinishNin *finish_nin) {
  Tiling t;
  const int passes = passes_of(precision);
  int rawEntries = 0, nStages64 = 0;
  const bool pool = d_pool_rules != nullptr;
  // pooled: `rows` counts pooled rows; the kernel's row space is pooled rows x cells (a tile = 128 / cells windows)
  if (pool && (passes || !d_rules || !d_choices || pool_cells < 2 || pool_cells > 32 || (pool_cells & (pool_cells - 1)) || (long long)rows * pool_cells > INT_MAX))
    return fail(SCN_ERR_UNSUPPORTED, "fused max-pooling needs the split (tf32 / bf16 operand) kernel, rules, and 2, 4, 8, 16 or 32 cells per window");
  // Where the layer alone would split K (few tiles) the fused row space is not used: the plain kernel writes its
  // partial sums over the layer's own rows and the pooling happens in the finishing kernel.
  if (pool && !passes && rows_unpooled > 0 && d_ws && !d_rows && N % 4 == 0 && ((uintptr_t)d_ws & 15) == 0 &&
      is_split(precision) && make_tiling(fs * nIn, N, fs, true, &t, precision == SCN_PREC_SPLIT)) {
    const int plainTiles = ((rows_unpooled + BM - 1) / BM) * t.nTiles;
    if (choose_ksplit(plainTiles, t.nSlabs, rows_unpooled, N, wsBytes) > 1) {
      FinishPool fp = {d_pool_rules, pool_cells, rows, d_choices};
      return tc_launch(d_in, d_rules, rows_unpooled, fs, nIn, d_packed, d_B, d_prelu, N, p, act, precision, d_out, d_ws, wsBytes, s,
                       nullptr, nullptr, 0, nullptr, 0, &fp);
    }
  }
  if (pool) rows *= pool_cells;
  const bool ok = N % 4 == 0 && (passes ? make_tiling16(fs * nIn, N, fs, d_rules != nullptr, passes, &t, &rawEntries, &nStages64)
                                        : is_split(precision) && make_tiling(fs * nIn, N, fs, d_rules != nullptr, &t, precision == SCN_PREC_SPLIT, false, pool));
  // (a row longer than the zero row is fine where no tile row can be missing: no rules and whole tiles of real rows)
  const bool noMissingRows = !d_rules && !pool && !d_rows && rows % BM == 0;
  if (!ok || (nIn % SLAB == 0 && nIn > ZERO_ROW_FLOATS && !noMissingRows)) return fail(SCN_ERR_UNSUPPORTED, "shape not supported by the tensor-core kernel");
  if (((uintptr_t)d_in | (uintptr_t)d_out | (uintptr_t)d_packed) & 15) return fail(SCN_ERR_INVALID, "tensor-core path needs 16-byte aligned buffers");
  Params P;
  const int mTiles = (rows + BM - 1) / BM;
  int kSplit = (d_ws && ((uintptr_t)d_ws & 15) == 0) ? choose_ksplit(mTiles * t.nTiles, passes ? 2 * nStages64 : t.nSlabs, rows, N, wsBytes) : 1;
  if (pool && kSplit > 1) return fail(SCN_ERR_UNSUPPORTED, "fused max-pooling is not combined with a K split");
  if (finish_nin && (kSplit <= 1 || passes || pool)) return fail(SCN_ERR_UNSUPPORTED, "the second learnt layer rides on the K-split finish only");
  if (pool && rows_unpooled > 0) {
    // The window-major row space repeats rows that several windows name (background rows) and pads ragged
    // windows: do not fuse where that costs a wave of tiles, or where the layer alone would split K.
    const int plainTiles = ((rows_unpooled + BM - 1) / BM) * t.nTiles, sms = sm_count();
    if (choose_ksplit(plainTiles, t.nSlabs, rows_unpooled, N, (size_t)-1) > 1 ||
        (mTiles * t.nTiles + sms - 1) / sms > (plainTiles + sms - 1) / sms)
      return fail(SCN_ERR_UNSUPPORTED, "fused max-pooling would not pay for this shape");
  }
  const bool oneItem = !passes && !t.atmem && mTiles * t.nTiles * kSplit <= sm_count();
  // few input channels and one slab (a first layer): row-per-lane gather that also writes the lo image, and the
  // four warps that would split become a second epilogue group
  const bool epi2 = !passes && d_rules && nIn % SLAB != 0 && nIn <= ROWWISE_MAX_NIN && t.nSlabs == 1 && kSplit == 1 && !t.atmem;
  if (oneItem || epi2) make_tiling(fs * nIn, N, fs, d_rules != nullptr, &t, precision == SCN_PREC_SPLIT, oneItem, pool, epi2);
  P.epi2 = epi2 ? 1 : 0;
  P.rawEntries = rawEntries; P.nStages64 = nStages64; P.atmem = passes ? 0 : t.atmem; P.aBase = t.aBase;
  P.bf16 = (!passes && t.bf16 && t.atmem) ? 1 : 0;
  if (d_rows && (passes || kSplit > 1)) return fail(SCN_ERR_UNSUPPORTED, "a device-side row count needs the split (tf32 / bf16 operand) kernel without K split");
  P.rowsPtr = d_rows; P.poolRules = d_pool_rules; P.poolCells = pool_cells; P.choices = d_choices;
  P.in = d_in; P.rules = d_rules; P.rows = rows; P.fs = fs; P.nIn = nIn;
  P.packed = (const unsigned char *)d_packed; P.bias = d_B; P.prelu = d_prelu;
  P.N = N; P.BN = t.BN; P.nTiles = t.nTiles; P.nSlabs = t.nSlabs; P.stages = t.stages; P.tmemCols = t.tmemCols; P.rulesBytes = t.rulesBytes;
  P.p = p; P.act = act; P.out = d_out;
  // instruction descriptor: D = fp32, A = B = tf32 (2) or bf16 (1), both K-major, N = BN, M = 128
  const uint32_t fmt = (passes || P.bf16) ? 1u : 2u;
  P.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(t.BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  P.kSplit = kSplit;
  P.partial = (float *)d_ws;
  P.mTiles = mTiles; P.accStride = t.accStride;
  P.K = fs * nIn; P.generic = (nIn % SLAB != 0) ? 1 : 0;
  P.rulesDouble = (t.rulesDouble && (pool || ((uintptr_t)d_rules & 15) == 0)) ? 1 : 0;
  const int items = mTiles * t.nTiles * P.kSplit;
  const int grid = items < sm_count() ? items : sm_count(); // persistent: one CTA per SM
#define SCN_TC16_LAUNCH(PASSES)                                                                                                          \
  do {                                                                                                                                  \
    if (P.kSplit > 1) {                                                                                                                 \
      SCN_CUDA_TRY(cudaFuncSetAttribute(k_conv_nin_tc16<true, SCN_NOSIGMOID, PASSES>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024)); \
      k_conv_nin_tc16<true, SCN_NOSIGMOID, PASSES><<<grid, NUM_THREADS16, t.smemBytes, s>>>(P);                                          \
    } else {                                                                                                                            \
      SCN_DISPATCH_ACT(act, SCN_CUDA_TRY(cudaFuncSetAttribute(k_conv_nin_tc16<false, ACT, PASSES>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024)); \
                       (k_conv_nin_tc16<false, ACT, PASSES><<<grid, NUM_THREADS16, t.smemBytes, s>>>(P)));                               \
    }                                                                                                                                   \
  } while (0)
  if (passes == 3) SCN_TC16_LAUNCH(3);
  else if (passes == 1) SCN_TC16_LAUNCH(1);
  else if (pool && P.atmem) {
    SCN_DISPATCH_ACT(act, SCN_CUDA_TRY(cudaFuncSetAttribute(k_conv_nin_tc<false, ACT, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
                     (void)launch_dependent(k_conv_nin_tc<false, ACT, true, true>, dim3(grid), dim3(NUM_THREADS), (size_t)t.smemBytes, s, P));
  } else if (pool) {
    SCN_DISPATCH_ACT(act, SCN_CUDA_TRY(cudaFuncSetAttribute(k_conv_nin_tc<false, ACT, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
                     (void)launch_dependent(k_conv_nin_tc<false, ACT, false, true>, dim3(grid), dim3(NUM_THREADS), (size_t)t.smemBytes, s, P));
  } else if (P.atmem && P.kSplit > 1) {
    SCN_CUDA_TRY(cudaFuncSetAttribute(k_conv_nin_tc<true, SCN_NOSIGMOID, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
    (void)launch_dependent(k_conv_nin_tc<true, SCN_NOSIGMOID, true>, dim3(grid), dim3(NUM_THREADS), (size_t)t.smemBytes, s, P);
  } else if (P.atmem) {
    SCN_DISPATCH_ACT(act, SCN_CUDA_TRY(cudaFuncSetAttribute(k_conv_nin_tc<false, ACT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
                     (void)launch_dependent(k_conv_nin_tc<false, ACT, true>, dim3(grid), dim3(NUM_THREADS), (size_t)t.smemBytes, s, P));
  } else if (P.kSplit > 1) {
    SCN_CUDA_TRY(cudaFuncSetAttribute(k_conv_nin_tc<true, SCN_NOSIGMOID, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
    (void)launch_dependent(k_conv_nin_tc<true, SCN_NOSIGMOID, false>, dim3(grid), dim3(NUM_THREADS), (size_t)t.smemBytes, s, P);
  } else {
    SCN_DISPATCH_ACT(act, SCN_CUDA_TRY(cudaFuncSetAttribute(k_conv_nin_tc<false, ACT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
                     (void)launch_dependent(k_conv_nin_tc<false, ACT, false>, dim3(grid), dim3(NUM_THREADS), (size_t)t.smemBytes, s, P));
  }
#undef SCN_TC16_LAUNCH
  SCN_LAUNCH_CHECK("k_conv_nin_tc");
  if (P.kSplit > 1 && finish_nin) {
    const FinishNin &fn2 = *finish_nin;
    const int blocks = rows < 8 * sm_count() ? rows : 8 * sm_count();
    SCN_DISPATCH_ACT(act, (void)launch_dependent(k_splitk_finish_nin<ACT>, dim3(blocks), dim3(256), (size_t)(N + 128) * sizeof(float), s, (const float *)P.partial,
                                                 P.kSplit, (long long)rows, N, d_B, d_prelu, p, d_out, fn2.W2, fn2.B2, fn2.prelu2, fn2.N2, fn2.p2, fn2.act2,
                                                 fn2.out2));
    SCN_LAUNCH_CHECK("k_splitk_finish_nin");
  } else if (P.kSplit > 1 && finish_pool) {
    const FinishPool &fp = *finish_pool;
    SCN_DISPATCH_ACT(act, (void)launch_dependent(k_splitk_finish_pool<ACT>, dim3(grid_for((long long)fp.rowsPool * N / 4, 256)), dim3(256), (size_t)0, s,
                                                 (const float *)P.partial, P.kSplit, (long long)rows, N, d_B, d_prelu, p, fp.poolRules, fp.cells, fp.rowsPool,
                                                 d_out, fp.choices));
    SCN_LAUNCH_CHECK("k_splitk_finish_pool");
  } else if (P.kSplit > 1) {
    SCN_DISPATCH_ACT(act, (void)launch_dependent(k_splitk_finish<ACT>, dim3(grid_for((long long)rows * N / 4, 256)), dim3(256), (size_t)0, s, (const float *)P.partial, P.kSplit, rows, N, d_B, d_prelu, p, d_out));
    SCN_LAUNCH_CHECK("k_splitk_finish");
  }
  return SCN_OK;
}

int *tc_error_word() {
  static int *cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!cached[dev]) {
    void *p = nullptr;
    if (cudaGetSymbolAddress(&p, g_tc_error) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    cached[dev] = (int *)p;
  }
  return cached[dev];
}

int tc_take_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
  return v;
}

} // namespace scn
