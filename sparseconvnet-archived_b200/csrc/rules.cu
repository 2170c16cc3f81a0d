// Rule construction on the GPU: the device replacement of the reference's per-sample
// SparseGrid maps (SparseGrid.h, vectorHash.cpp) and gridRules builders (Regions.cu).
//
// Data structure.  A sample's grid is an occupancy bitmap over its nIn^dim cells with a rank
// directory: word w of sample b is {bits, number of active cells in earlier words}.  This is
// the reference's vectorHash (a dense key-indexed array, vectorHash.h:6-23) at 1/16 of its
// size, and it answers both questions the builders ask: "is cell k active" (one bit) and
// "which row is cell k" (rank of k among the active cells -> sortedRow[]).  The rank is also
// the position of k in ascending-key order, which is the order the reference's vectorHash
// backend iterates in and therefore the order that fixes output row numbers.
//
// Row numbering.  The reference visits input sites in ascending key and, for each, the
// output sites it touches in ascending output key; an output site gets the next free row id
// the first time it is touched (Regions.cu:566-573).  So an output site is "created" by the
// smallest active key in its receptive field, and its id is
//     (#sites created by smaller input keys) + (its rank among the sites this key creates).
// Kernels: mark bits -> rank directory -> per input site, flag the outputs it creates ->
// exclusive scan of the per-site counts -> per sample offsets and background rows -> assign
// output keys -> fill rule cells.  All pure integer, HBM/L2-bound work; no host
// synchronisation: every size the kernels need is read from device memory.
#include "scn_common.cuh"
#include <algorithm>
#include <cstring>
#include <new>
#include <mutex>
#include <vector>

namespace scn {
namespace {

constexpr int MAX_CUBE = 256; // size^dim cells of a receptive field

struct Regions {
  int lattice, dim, nIn, nOut, size, stride, minActive;
  int sd, cube, Tax, T, W, cells, fullSize;
  float rNIn, rNOut, rSize, rSd, rT, rTax, rStride; // reciprocals for the float-assisted divisions below
  signed char ord[MAX_CUBE];         // cube cell -> rule column, -1 outside a triangular filter
  unsigned char cellOfCol[MAX_CUBE]; // rule column -> cube cell
  // Fractional max-pooling (FractionalPoolingRegions, Regions.cu:127-157): region bounds come from per
  // sample, per axis tick tables instead of size/stride.  fmp: 0 regular regions, 1 overlapping
  // (every region spans `size` cells per axis), 2 non-overlapping (regions of size-1 or size cells;
  // rule cells outside a region hold -1, Regions.cu:201-215).
  int fmp, tickStride;
  const int *ticks; // [(b*dim + axis) * tickStride]: inputL[nOut], inputR[nOut], outputL[nIn], outputR[nIn]
};

__device__ __forceinline__ const int *tick_axis(const Regions &R, int b, int a) { return R.ticks + ((size_t)b * R.dim + a) * R.tickStride; }

__host__ __device__ inline long long ipowll(long long b, int e) {
  long long r = 1;
  while (e-- > 0) r *= b;
  return r;
}

// Largest b with off[b] <= row (samples own contiguous row blocks).
__device__ __forceinline__ int find_sample(const int *__restrict__ off, int batch, int row) {
  int lo = 0, hi = batch;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (__ldg(off + mid) <= row) lo = mid; else hi = mid;
  }
  return lo;
}

__device__ __forceinline__ void decode(int key, int n, int dim, int *c) {
  for (int a = dim - 1; a >= 0; --a) { c[a] = key % n; key /= n; }
}
__device__ __forceinline__ int encode(const int *c, int n, int dim) {
  int k = 0;
  for (int a = 0; a < dim; ++a) k = k * n + c[a];
  return k;
}

__global__ void k_mark(Regions R, int batch, const int *__restrict__ keys, const int *__restrict__ off,
                       uint2 *dir, int *result) {
  const int n = off[batch];
  for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < n; row += gridDim.x * blockDim.x) {
    int key = keys[row];
    if (key < 0) continue; // background row
    if (key >= R.cells) { atomicOr(result + 2, SCN_DEV_ERR_KEY); continue; }
    int b = find_sample(off, batch, row);
    unsigned bit = 1u << (key & 31);
    unsigned old = atomicOr(&dir[(size_t)b * R.W + (key >> 5)].x, bit);
    if (old & bit) atomicOr(result + 2, SCN_DEV_ERR_DUPLICATE);
  }
}

// One CTA per sample: exclusive scan of the word popcounts.
__global__ void k_rank(Regions R, int batch, uint2 *dir, int *nSites) {
  __shared__ int warpSum[32];
  __shared__ int carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nWarps = blockDim.x >> 5;
  for (int b = blockIdx.x; b < batch; b += gridDim.x) {
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    uint2 *d = dir + (size_t)b * R.W;
    for (int w0 = 0; w0 < R.W; w0 += blockDim.x) {
      int w = w0 + threadIdx.x;
      int c = (w < R.W) ? __popc(d[w].x) : 0;
      int incl = c;
      for (int o = 1; o < 32; o <<= 1) { int v = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += v; }
      if (lane == 31) warpSum[warp] = incl;
      __syncthreads();
      if (warp == 0) {
        int v = (lane < nWarps) ? warpSum[lane] : 0;
        for (int o = 1; o < 32; o <<= 1) { int u = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += u; }
        warpSum[lane] = v; // inclusive over warps
      }
      __syncthreads();
      int base = carry + (warp ? warpSum[warp - 1] : 0);
      if (w < R.W) d[w].y = base + incl - c;
      __syncthreads();
      if (threadIdx.x == 0) carry += warpSum[nWarps - 1];
      __syncthreads();
    }
    if (threadIdx.x == 0) nSites[b] = carry;
    __syncthreads();
  }
}

__device__ __forceinline__ bool cell_active(const uint2 *__restrict__ d, int key) {
  return (d[key >> 5].x >> (key & 31)) & 1u;
}
__device__ __forceinline__ int cell_rank(const uint2 *__restrict__ d, int key) {
  uint2 e = d[key >> 5];
  return e.y + __popc(e.x & ((1u << (key & 31)) - 1u));
}

// Output coordinates of the t-th output site input site i can touch (mixed radix over the
// axes, so ascending t = ascending output key); false if t names none.
__device__ __forceinline__ bool touched_output(const Regions &R, int b, const int *i, int t, int *j) {
  if (R.fmp) { // outputL/outputR tables (Regions.cu:45-51)
    for (int a = R.dim - 1; a >= 0; --a) {
      const int ta = t % R.Tax; t /= R.Tax;
      const int *tk = tick_axis(R, b, a) + 2 * R.nOut;
      j[a] = __ldg(tk + i[a]) + ta;
      if (j[a] >= __ldg(tk + R.nIn + i[a])) return false;
    }
    return true;
  }
  if (R.minActive == -1) { // 'valid': the site centred on i (Regions.cu:691-696)
    bool ok = true;
    for (int a = 0; a < R.dim; ++a) { ok = ok && i[a] >= 1 && i[a] <= R.nOut; j[a] = i[a] - 1; }
    return ok;
  }
  int sum = 0;
  for (int a = R.dim - 1; a >= 0; --a) {
    int ta = t % R.Tax; t /= R.Tax;
    int lo = max(0, (i[a] - R.size + R.stride) / R.stride);
    int hi = min(i[a] / R.stride + 1, R.nOut);
    j[a] = lo + ta;
    if (j[a] >= hi) return false;
    sum += j[a];
  }
  if (R.lattice == SCN_LATTICE_TRIANGULAR && sum >= R.nOut) return false;
  return true;
}

// Does input site i (active) create output site j: is i the first active cell of j's cube
// field in lexicographic (= key) order, and does the field hold enough active inputs?
__device__ bool creates(const Regions &R, int b, const uint2 *__restrict__ d, const int *i, const int *j) {
  if (R.minActive == -1) return true;
  int cc[4] = {0, 0, 0, 0}, ii[4];
  int active = 0;
  if (R.fmp) { // the field of j is [inputL(j), inputR(j)) per axis; first active cell in key order wins
    int lo[4], ext[4];
    for (int a = 0; a < R.dim; ++a) {
      const int *tk = tick_axis(R, b, a);
      lo[a] = __ldg(tk + j[a]);
      ext[a] = __ldg(tk + R.nOut + j[a]) - lo[a];
    }
    for (;;) {
      bool self = true;
      for (int a = 0; a < R.dim; ++a) { ii[a] = lo[a] + cc[a]; self = self && ii[a] == i[a]; }
      if (self) return true;
      if (cell_active(d, encode(ii, R.nIn, R.dim))) return false;
      int a = R.dim - 1;
      while (a >= 0 && ++cc[a] >= ext[a]) { cc[a] = 0; --a; }
      if (a < 0) return false;
    }
  }
  for (int cell = 0; cell < R.cube; ++cell) {
    bool self = true;
    for (int a = 0; a < R.dim; ++a) { ii[a] = j[a] * R.stride + cc[a]; self = self && ii[a] == i[a]; }
    if (self) {
      if (R.minActive <= 1) return true;
      active += (R.ord[cell] >= 0);
      // keep counting the rest of the field
      for (int c2 = cell + 1; c2 < R.cube; ++c2) {
        int a = R.dim - 1;
        while (a >= 0 && ++cc[a] >= R.size) { cc[a] = 0; --a; }
        if (R.ord[c2] < 0) continue;
        for (int q = 0; q < R.dim; ++q) ii[q] = j[q] * R.stride + cc[q];
        active += cell_active(d, encode(ii, R.nIn, R.dim));
      }
      return active >= R.minActive;
    }
    if (cell_active(d, encode(ii, R.nIn, R.dim))) return false; // an earlier key got there first
    int a = R.dim - 1;
    while (a >= 0 && ++cc[a] >= R.size) { cc[a] = 0; --a; }
  }
  return false;
}

// Division of 0 <= x < 2^24 by n with a float reciprocal (quotient off by at most one, then fixed).
__device__ __forceinline__ int fdiv(int x, int n, float rn, int *rem) {
  int q = __float2int_rz(__int2float_rn(x) * rn);
  int r = x - q * n;
  if (r < 0) { --q; r += n; } else if (r >= n) { ++q; r -= n; }
  *rem = r;
  return q;
}
template <int DIM> __device__ __forceinline__ void decode_f(int key, int n, float rn, int *c) {
#pragma unroll
  for (int a = DIM - 1; a > 0; --a) key = fdiv(key, n, rn, &c[a]);
  c[0] = key;
}
template <int DIM> __device__ __forceinline__ int encode_f(const int *c, int n) {
  int k = c[0];
#pragma unroll
  for (int a = 1; a < DIM; ++a) k = k * n + c[a];
  return k;
}
template <int DIM> __device__ __forceinline__ bool touched_output_f(const Regions &R, const int *i, int t, int *j) {
  if (R.minActive == -1) {
    bool ok = true;
#pragma unroll
    for (int a = 0; a < DIM; ++a) { ok = ok && i[a] >= 1 && i[a] <= R.nOut; j[a] = i[a] - 1; }
    return ok;
  }
  int sum = 0;
  bool ok = true;
#pragma unroll
  for (int a = DIM - 1; a >= 0; --a) {
    int ta;
    t = fdiv(t, R.Tax, R.rTax, &ta);
    int rem;
    const int num = i[a] - R.size + R.stride; // outputL = max(0, num / stride): a non-positive num gives 0
    const int lo = num <= 0 ? 0 : fdiv(num, R.stride, R.rStride, &rem);
    const int hi = min(fdiv(i[a], R.stride, R.rStride, &rem) + 1, R.nOut);
    j[a] = lo + ta;
    ok = ok && j[a] < hi;
    sum += j[a];
  }
  if (R.lattice == SCN_LATTICE_TRIANGULAR && sum >= R.nOut) return false;
  return ok;
}
// Any active cell among the keys k0 .. k0 + n - 1 (1 <= n <= 32): they are neighbouring bits of the bitmap.
__device__ __forceinline__ bool range_any(const uint2 *d, int k0, int n) {
  const int w = k0 >> 5, sh = k0 & 31;
  unsigned bits = d[w].x >> sh;
  if (sh + n > 32) bits |= d[w + 1].x << (32 - sh);
  return (bits & (n == 32 ? 0xffffffffu : (1u << n) - 1u)) != 0u;
}
// The cells k0 .. k0 + n - 1 (1 <= n <= 32) as the low n bits of a word.
__device__ __forceinline__ unsigned range_bits(const uint2 *d, int k0, int n) {
  const int w = k0 >> 5, sh = k0 & 31;
  unsigned bits = d[w].x >> sh;
  if (sh + n > 32) bits |= d[w + 1].x << (32 - sh);
  return bits & (n == 32 ? 0xffffffffu : (1u << n) - 1u);
}
template <int DIM> __device__ bool creates_f(const Regions &R, const uint2 *d, const int *i, const int *j) {
  if (R.minActive == -1) return true;
  if (R.minActive <= 1 && R.size <= 32) {
    // Site i creates output j iff no cell of j's field with a smaller key is active.  Along the last axis the
    // field's cells are neighbouring keys, so each line of the field in front of i is one masked look at the
    // bitmap (a 3 x 3 field: at most 3 looks instead of 8 cell probes).
    int co[DIM > 1 ? DIM - 1 : 1];
#pragma unroll
    for (int a = 0; a < DIM - 1; ++a) co[a] = 0;
    const int x0 = j[DIM - 1] * R.stride, selfIn = i[DIM - 1] - x0;
    for (int line = 0; line < R.cube; ++line) {
      int key0 = 0;
      bool same = true;
#pragma unroll
      for (int a = 0; a < DIM - 1; ++a) {
        const int ia = j[a] * R.stride + co[a];
        key0 = key0 * R.nIn + ia;
        same = same && ia == i[a];
      }
      key0 = key0 * R.nIn + x0;
      if (same) return selfIn == 0 || !range_any(d, key0, selfIn);
      if (range_any(d, key0, R.size)) return false;
#pragma unroll
      for (int a = DIM - 2; a >= 0; --a) { if (++co[a] < R.size) break; co[a] = 0; }
    }
    return false;
  }
  int cc[DIM], ii[DIM];
#pragma unroll
  for (int a = 0; a < DIM; ++a) cc[a] = 0;
  int active = 0;
  bool seenSelf = false;
  for (int cell = 0; cell < R.cube; ++cell) {
    bool self = true;
#pragma unroll
    for (int a = 0; a < DIM; ++a) { ii[a] = j[a] * R.stride + cc[a]; self = self && ii[a] == i[a]; }
    if (self) {
      if (R.minActive <= 1) return true;
      seenSelf = true;
      active += (R.ord[cell] >= 0);
    } else {
      const bool on = cell_active(d, encode_f<DIM>(ii, R.nIn));
      if (!seenSelf) { if (on) return false; } // an earlier key got there first
      else if (R.ord[cell] >= 0) active += on;
    }
#pragma unroll
    for (int a = DIM - 1; a >= 0; --a) { if (++cc[a] < R.size) break; cc[a] = 0; }
  }
  return seenSelf && active >= R.minActive;
}


// Per input row: its slot in ascending-key order, the outputs it creates, and their count.
__global__ void k_flags(Regions R, int batch, const int *__restrict__ keys, const int *__restrict__ off,
                        const uint2 *__restrict__ dir, int *sortedRow, unsigned char *flags, int *cnt,
                        bool withFlags) {
  const int n = off[batch];
  for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < n; row += gridDim.x * blockDim.x) {
    int key = keys[row];
    if (key < 0 || key >= R.cells) continue;
    int b = find_sample(off, batch, row);
    const uint2 *d = dir + (size_t)b * R.W;
    int slot = off[b] + cell_rank(d, key);
    sortedRow[slot] = row;
    if (!withFlags) continue;
    int i[4], j[4];
    decode(key, R.nIn, R.dim, i);
    int c = 0;
    for (int t = 0; t < R.T; ++t) {
      bool f = touched_output(R, b, i, t, j) && creates(R, b, d, i, j);
      flags[(size_t)slot * R.T + t] = f;
      c += f;
    }
    cnt[slot] = c;
  }
}

// ---- exclusive scan of cnt[0..n) in place, total at cnt[n]; n read from the device.
constexpr int SCAN_THREADS = 256, SCAN_ITEMS = 8, SCAN_CHUNK = SCAN_THREADS * SCAN_ITEMS;

__device__ __forceinline__ int block_exclusive_scan(int v, int *total) {
  __shared__ int ws[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nWarps = blockDim.x >> 5;
  int incl = v;
  for (int o = 1; o < 32; o <<= 1) { int u = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += u; }
  __syncthreads(); // ws may still be read by a previous call
  if (lane == 31) ws[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int s = (lane < nWarps) ? ws[lane] : 0;
    for (int o = 1; o < 32; o <<= 1) { int u = __shfl_up_sync(0xffffffffu, s, o); if (lane >= o) s += u; }
    ws[lane] = s;
  }
  __syncthreads();
  *total = ws[nWarps - 1];
  return (warp ? ws[warp - 1] : 0) + incl - v;
}

__global__ void k_scan_reduce(const int *__restrict__ cnt, const int *__restrict__ off, int batch, int *partial) {
  const int n = off[batch];
  const int nChunks = (n + SCAN_CHUNK - 1) / SCAN_CHUNK;
  for (int c = blockIdx.x; c < nChunks; c += gridDim.x) {
    int s = 0;
    for (int k = 0; k < SCAN_ITEMS; ++k) {
      int idx = c * SCAN_CHUNK + k * SCAN_THREADS + threadIdx.x;
      if (idx < n) s += cnt[idx];
    }
    int total;
    block_exclusive_scan(s, &total);
    if (threadIdx.x == 0) partial[c] = total;
  }
}
__global__ void k_scan_partials(const int *__restrict__ off, int batch, int *partial) {
  const int n = off[batch];
  const int nChunks = (n + SCAN_CHUNK - 1) / SCAN_CHUNK;
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int c0 = 0; c0 < nChunks; c0 += blockDim.x) {
    int c = c0 + threadIdx.x;
    int v = (c < nChunks) ? partial[c] : 0;
    int total;
    int ex = block_exclusive_scan(v, &total);
    if (c < nChunks) partial[c] = carry + ex;
    __syncthreads();
    if (threadIdx.x == 0) carry += total;
    __syncthreads();
  }
  if (threadIdx.x == 0) partial[nChunks] = carry;
}
__global__ void k_scan_apply(int *cnt, const int *__restrict__ off, int batch, const int *__restrict__ partial) {
  const int n = off[batch];
  const int nChunks = (n + SCAN_CHUNK - 1) / SCAN_CHUNK;
  for (int c = blockIdx.x; c < nChunks; c += gridDim.x) {
    int v[SCAN_ITEMS], s = 0;
    const int base = c * SCAN_CHUNK + threadIdx.x * SCAN_ITEMS;
    for (int k = 0; k < SCAN_ITEMS; ++k) { v[k] = (base + k < n) ? cnt[base + k] : 0; s += v[k]; }
    int total;
    int ex = block_exclusive_scan(s, &total) + partial[c];
    for (int k = 0; k < SCAN_ITEMS; ++k) { if (base + k < n) cnt[base + k] = ex; ex += v[k]; }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) cnt[n] = partial[nChunks];
}

// Per sample: output row offsets, background rows, totals.  One CTA.
__global__ void k_samples(Regions R, int batch, const int *__restrict__ inOff, const int *__restrict__ P,
                          int *outOff, int *outBg, int *outKeys, int capacity, int *result) {
  __shared__ int carry, maxSites;
  if (threadIdx.x == 0) { carry = 0; maxSites = 0; }
  __syncthreads();
  for (int b0 = 0; b0 < batch; b0 += blockDim.x) {
    int b = b0 + threadIdx.x;
    int sites = 0, need = 0, before = 0;
    if (b < batch) {
      before = P[inOff[b]];
      sites = P[inOff[b + 1]] - before;
      need = sites < R.fullSize; // e.g. Regions.cu:647-652
    }
    int total;
    int ex = block_exclusive_scan(need, &total);
    if (b < batch) {
      int first = before + carry + ex;
      outOff[b] = first;
      int bgRow = need ? first + sites : -1;
      outBg[b] = bgRow;
      if (need && bgRow < capacity) outKeys[bgRow] = -1;
      atomicMax(&maxSites, sites);
    }
    __syncthreads();
    if (threadIdx.x == 0) carry += total;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    int sitesTotal = P[inOff[batch]];
    int rows = sitesTotal + carry;
    outOff[batch] = rows;
    result[0] = rows;
    result[1] = sitesTotal;
    result[3] = maxSites;
    if (rows > capacity) atomicOr(result + 2, SCN_DEV_ERR_CAPACITY);
  }
}

// Per (input slot, touched output) pair that creates a site: the site's row id and key.
__global__ void k_assign(Regions R, int batch, const int *__restrict__ keys, const int *__restrict__ inOff,
                         const int *__restrict__ sortedRow, const unsigned char *__restrict__ flags,
                         const int *__restrict__ P, const int *__restrict__ outOff, int *outKeys, int capacity) {
  const long long n = (long long)inOff[batch] * R.T;
  for (long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x; p < n; p += (long long)gridDim.x * blockDim.x) {
    if (!flags[p]) continue;
    int slot = (int)(p / R.T), t = (int)(p % R.T);
    int rank = 0;
    for (int q = 0; q < t; ++q) rank += flags[(size_t)slot * R.T + q];
    int b = find_sample(inOff, batch, slot);
    int outRow = outOff[b] + (P[slot] - P[inOff[b]]) + rank;
    if (outRow >= capacity) continue;
    int i[4], j[4];
    decode(keys[sortedRow[slot]], R.nIn, R.dim, i);
    touched_output(R, b, i, t, j);
    outKeys[outRow] = encode(j, R.nOut, R.dim);
  }
}

// One thread per rule cell: rules[row*sd + col], coalesced.
__global__ void k_fill(Regions R, int batch, const int *__restrict__ inOff, const int *__restrict__ inBg,
                       const uint2 *__restrict__ dir, const int *__restrict__ sortedRow,
                       const int *__restrict__ outOff, const int *__restrict__ outKeys, int *rules,
                       int capacity, const int *__restrict__ result) {
  const long long n = (long long)min(result[0], capacity) * R.sd;
  for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < n; q += (long long)gridDim.x * blockDim.x) {
    int r = (int)(q / R.sd), col = (int)(q % R.sd);
    int b = find_sample(outOff, batch, r);
    int key = outKeys[r];
    int v = inBg[b];
    if (key >= 0) {
      int j[4], cc[4], ii[4];
      decode(key, R.nOut, R.dim, j);
      decode(R.cellOfCol[col], R.size, R.dim, cc);
      bool inside = true;
      if (R.fmp) {
        for (int a = 0; a < R.dim; ++a) {
          const int *tk = tick_axis(R, b, a);
          const int lo = __ldg(tk + j[a]);
          ii[a] = lo + cc[a];
          inside = inside && ii[a] < __ldg(tk + R.nOut + j[a]);
        }
      } else {
        for (int a = 0; a < R.dim; ++a) ii[a] = j[a] * R.stride + cc[a];
      }
      if (!inside) v = -1; // a cell beyond a short non-overlapping region (Regions.cu:201-203)
      else {
        int ck = encode(ii, R.nIn, R.dim);
        const uint2 *d = dir + (size_t)b * R.W;
        uint2 e = d[ck >> 5];
        if ((e.x >> (ck & 31)) & 1u) v = sortedRow[inOff[b] + e.y + __popc(e.x & ((1u << (ck & 31)) - 1u))];
      }
    }
    rules[q] = v;
  }
}


// ---- the same three kernels with the dimension fixed at compile time and float-assisted
// divisions, used whenever every cell index is below 2^24 (all benchmark grids are)
template <int DIM>
__global__ void k_flags_t(Regions R, int batch, const int *__restrict__ keys, const int *__restrict__ off,
                          const uint2 *__restrict__ dir, int *sortedRow, unsigned char *flags, int *cnt) {
  const int n = off[batch];
  for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < n; row += gridDim.x * blockDim.x) {
    const int key = keys[row];
    if (key < 0 || key >= R.cells) continue;
    const int b = find_sample(off, batch, row);
    const uint2 *d = dir + (size_t)b * R.W;
    const int slot = off[b] + cell_rank(d, key);
    sortedRow[slot] = row;
    int i[DIM], j[DIM];
    decode_f<DIM>(key, R.nIn, R.rNIn, i);
    int c = 0;
    for (int t = 0; t < R.T; ++t) {
      const bool f = touched_output_f<DIM>(R, i, t, j) && creates_f<DIM>(R, d, i, j);
      flags[(size_t)slot * R.T + t] = f;
      c += f;
    }
    cnt[slot] = c;
  }
}
template <int DIM>
__global__ void k_assign_t(Regions R, int batch, const int *__restrict__ keys, const int *__restrict__ inOff,
                           const int *__restrict__ sortedRow, const unsigned char *__restrict__ flags,
                           const int *__restrict__ P, const int *__restrict__ outOff, int *outKeys, int capacity) {
  const long long n = (long long)inOff[batch] * R.T;
  for (long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x; p < n; p += (long long)gridDim.x * blockDim.x) {
    if (!flags[p]) continue;
    const int slot = (int)(p / R.T), t = (int)(p - (long long)slot * R.T);
    int rank = 0;
    for (int q = 0; q < t; ++q) rank += flags[(size_t)slot * R.T + q];
    const int b = find_sample(inOff, batch, slot);
    const int outRow = outOff[b] + (P[slot] - P[inOff[b]]) + rank;
    if (outRow >= capacity) continue;
    int i[DIM], j[DIM];
    decode_f<DIM>(keys[sortedRow[slot]], R.nIn, R.rNIn, i);
    touched_output_f<DIM>(R, i, t, j);
    outKeys[outRow] = encode_f<DIM>(j, R.nOut);
  }
}
// One block takes 64 output rows at a time: 64 threads look up what a row's cells share (its sample, the
// input coordinates of its field's corner, the sample's bitmap, first input row and background row), then
// all 256 threads fill the rows' cells in storage order.  Per cell that leaves one bitmap word and, for an
// active cell, one sortedRow entry to read.
template <int DIM>
__global__ void __launch_bounds__(256) k_fill_t(Regions R, int batch, const int *__restrict__ inOff, const int *__restrict__ inBg,
                                                const uint2 *__restrict__ dir, const int *__restrict__ sortedRow,
                                                const int *__restrict__ outOff, const int *__restrict__ outKeys, int *rules,
                                                int capacity, const int *__restrict__ result) {
  constexpr int RB = 64;
  __shared__ int sSample[RB], sBg[RB], sFirst[RB], sCorner[RB][DIM];
  __shared__ unsigned char sCell[MAX_CUBE][DIM];
  const int tid = threadIdx.x;
  const int nRows = min(result[0], capacity);
  for (int col = tid; col < R.sd; col += blockDim.x) {
    int cc[DIM];
    decode_f<DIM>(R.cellOfCol[col], R.size, R.rSize, cc);
#pragma unroll
    for (int a = 0; a < DIM; ++a) sCell[col][a] = (unsigned char)cc[a];
  }
  for (long long row0 = (long long)blockIdx.x * RB; row0 < nRows; row0 += (long long)gridDim.x * RB) {
    __syncthreads();
    if (tid < RB && row0 + tid < nRows) {
      const int r = (int)row0 + tid;
      const int b = find_sample(outOff, batch, r);
      const int key = outKeys[r];
      sSample[tid] = key >= 0 ? b : -1; // -1: the sample's background row, every cell holds the input's background row
      sBg[tid] = inBg[b];
      sFirst[tid] = inOff[b];
      if (key >= 0) {
        int j[DIM];
        decode_f<DIM>(key, R.nOut, R.rNOut, j);
#pragma unroll
        for (int a = 0; a < DIM; ++a) sCorner[tid][a] = j[a] * R.stride;
      }
    }
    __syncthreads();
    const int cells = (int)min((long long)RB, nRows - row0) * R.sd;
    int *dst = rules + row0 * R.sd;
    for (int c = tid; c < cells; c += blockDim.x) {
      int col;
      const int rl = fdiv(c, R.sd, R.rSd, &col);
      int v = sBg[rl];
      const int b = sSample[rl];
      if (b >= 0) {
        int ii[DIM];
#pragma unroll
        for (int a = 0; a < DIM; ++a) ii[a] = sCorner[rl][a] + sCell[col][a];
        const int ck = encode_f<DIM>(ii, R.nIn);
        const uint2 e = (dir + (size_t)b * R.W)[ck >> 5];
        if ((e.x >> (ck & 31)) & 1u) v = sortedRow[sFirst[rl] + e.y + __popc(e.x & ((1u << (ck & 31)) - 1u))];
      }
      dst[c] = v;
    }
  }
}

// TerminalPoolingLayer.cu:8-20: sample b's rows in ascending key order, padded with -1.
__global__ void k_terminal(int batch, int S, const int *__restrict__ inOff, const int *__restrict__ inBg,
                           const int *__restrict__ nSites, const int *__restrict__ sortedRow, int *rules,
                           int *outKeys, int *outOff, int *outBg, int *result) {
  const long long n = (long long)batch * S;
  for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < n; q += (long long)gridDim.x * blockDim.x) {
    int b = (int)(q / S), p = (int)(q % S);
    int ns = nSites[b];
    int v = -1;
    if (p < ns) v = sortedRow[inOff[b] + p];
    else if (p == 0) v = inBg[b]; // no site at all: the background row stands in
    rules[q] = v;
    if (p == 0) {
      outKeys[b] = 0; outOff[b] = b; outBg[b] = -1;
      if (ns > S) atomicOr(result + 2, SCN_DEV_ERR_CAPACITY);
      if (b == 0) { outOff[batch] = batch; result[0] = batch; result[1] = batch; result[3] = 1; }
    }
  }
}

struct Workspace {
  uint2 *dir; int *nSites; int *sortedRow; int *cnt; int *partial; unsigned char *flags;
  size_t bytes;
};

Workspace carve(void *base, int batch, int W, int rows, int T) {
  Workspace w;
  size_t o = 0;
  auto take = [&](size_t n) { size_t at = o; o = align_up(o + n, 256); return (char *)base + at; };
  w.dir = (uint2 *)take((size_t)batch * W * sizeof(uint2));
  w.nSites = (int *)take((size_t)batch * sizeof(int));
  w.sortedRow = (int *)take((size_t)rows * sizeof(int));
  w.cnt = (int *)take(((size_t)rows + 1) * sizeof(int));
  w.partial = (int *)take(((size_t)rows / SCAN_CHUNK + 2) * sizeof(int));
  w.flags = (unsigned char *)take((size_t)rows * (T > 0 ? T : 0));
  w.bytes = o;
  return w;
}

int make_regions(const scn_regions_t *r, Regions *out) {
  if (!r) return fail(SCN_ERR_INVALID, "regions is NULL");
  Regions R;
  R.lattice = r->lattice; R.dim = r->dim; R.nIn = r->nIn; R.nOut = r->nOut;
  R.size = r->size; R.stride = r->stride; R.minActive = r->minActive;
  R.fmp = 0; R.tickStride = 0; R.ticks = nullptr;
  if (R.lattice != SCN_LATTICE_SQUARE && R.lattice != SCN_LATTICE_TRIANGULAR) return fail(SCN_ERR_INVALID, "unknown lattice");
  if (R.dim < 1 || R.dim > 4) return fail(SCN_ERR_INVALID, "dimension must be 1..4");
  if (R.size < 1 || R.stride < 1 || R.nOut < 1) return fail(SCN_ERR_INVALID, "size, stride and nOut must be positive");
  // the assert of both region constructors (Regions.cu:17, 823)
  if (R.nIn != R.size + (R.nOut - 1) * R.stride) return fail(SCN_ERR_INVALID, "nIn != size + (nOut-1)*stride");
  if (R.minActive == 0 || R.minActive < -1) return fail(SCN_ERR_INVALID, "minActive must be -1 or >= 1");
  if (R.minActive == -1 && (R.size != 3 || R.stride != 1 || R.lattice != SCN_LATTICE_SQUARE))
    return fail(SCN_ERR_INVALID, "valid mode needs a 3^dim stride-1 square filter (Regions.cu:665)");
  long long cube = ipowll(R.size, R.dim), cells = ipowll(R.nIn, R.dim);
  if (cube > MAX_CUBE) return fail(SCN_ERR_UNSUPPORTED, "receptive field larger than 256 cells");
  if (cells >= (1ll << 31)) return fail(SCN_ERR_UNSUPPORTED, "nIn^dim must be below 2^31");
  R.cube = (int)cube; R.cells = (int)cells;
  int S = 0;
  for (int c = 0; c < R.cube; ++c) {
    int j = c, J = 0;
    while (j > 0) { J += j % R.size; j /= R.size; }
    if (R.lattice == SCN_LATTICE_SQUARE || J < R.size) { R.ord[c] = (signed char)S; R.cellOfCol[S] = (unsigned char)c; ++S; }
    else R.ord[c] = -1;
  }
  R.sd = S;
  R.Tax = (R.minActive == -1) ? 1 : (R.size + R.stride - 1) / R.stride;
  long long T = (R.minActive == -1) ? 1 : ipowll(R.Tax, R.dim);
  if (T > 4096) return fail(SCN_ERR_UNSUPPORTED, "too many touched outputs per input");
  R.T = (int)T;
  R.W = (int)((cells + 31) / 32);
  R.rNIn = 1.0f / R.nIn; R.rNOut = 1.0f / R.nOut; R.rSize = 1.0f / R.size; R.rSd = 1.0f / R.sd; R.rT = 1.0f / R.T; R.rTax = 1.0f / R.Tax; R.rStride = 1.0f / R.stride;
  if (R.lattice == SCN_LATTICE_SQUARE) R.fullSize = (int)ipowll(R.nOut, R.dim);
  else { long long fs = 1; for (int i = 1; i <= R.dim; ++i) fs = fs * (R.nOut + R.dim - i) / i; R.fullSize = (int)fs; }
  *out = R;
  return SCN_OK;
}

} // namespace

// ---------------------------------------------------------------------------------------------
// Fused rule chain for small samples: ONE kernel builds the rulebooks of every geometry layer
// of a network.  CTA = one sample, all of that sample's per-layer state (bitmap + rank
// directory, key lists, creation flags, prefix sums) lives in shared memory, and the layers
// are walked in order.  The only thing a sample needs from the others is, per layer, how many
// output rows the samples before it produced (row ids run on across the batch): each CTA
// publishes its count and sums its predecessors' counts (bounded spin on a device array).
// Samples are handed out by an atomic ticket, so every predecessor of a CTA has already
// started and never waits on a later one.  Same arithmetic as the kernels above, same outputs.
namespace {

struct ChainLayer {
  Regions R;
  int *outKeys, *outOff, *outBg, *rules, *result;
  int capacity;
};
struct ChainParams {
  const ChainLayer *layers; int nLayers, batch;
  const int *inKeys, *inOff, *inBg;
  int *counts;  // [nLayers x batch], -1 until published; value = rows | needBg << 30
  int *ticket;
  int rowsMax, wMax, tMax, flagBytes;
  // Resident use (scn_rules_chain_build_resident): this launch leaves the state the NEXT launch will use ready
  // (its counters at -1, its ticket at -1, its result records at 0), so no stream operation has to run in front
  // of that launch.  All three are null otherwise.
  int *nextCounts, *nextTicket, *nextResults;
  int nNextResults; // ints to clear at nextResults
  int *bgOut; // not null: inBg is null, every sample's background row is found here and written to bgOut
};

constexpr int CHAIN_THREADS = 512;
constexpr unsigned long long CHAIN_WAIT_NS = 2000000000ull;

__device__ __forceinline__ unsigned long long chain_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

template <int DIM>
__global__ void __launch_bounds__(1024) k_rule_chain(const ChainParams P) {
  extern __shared__ __align__(16) unsigned char chain_smem[];
  __shared__ Regions R;
  __shared__ int sTicket, sBase, sSitesBase, colOff[MAX_CUBE], sScan[2][32];
  uint2 *dir = reinterpret_cast<uint2 *>(chain_smem);
  int *keysA = reinterpret_cast<int *>(dir + P.wMax);
  int *keysB = keysA + P.rowsMax;
  int *sorted = keysB + P.rowsMax;
  int *cnt = sorted + P.rowsMax; // rowsMax + 1
  int *pairs = cnt + P.rowsMax + 1; // rowsMax + 1: which (site, output) pair made each output row
  unsigned char *flags = reinterpret_cast<unsigned char *>(pairs + P.rowsMax + 1);
  const int tid = threadIdx.x;
  const int NT = blockDim.x;

  // Exclusive scan over the block with one barrier: every warp publishes its total, then every warp scans the
  // totals for itself.  Two buffers alternate, so a call's reads are over (the next call's barrier) before
  // the buffer is written again.
  int scanFlip = 0;
  auto scan = [&](int v, int *total) -> int {
    const int lane = tid & 31, warp = tid >> 5, nWarps = NT >> 5;
    int incl = v;
    for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += u; }
    int *buf = sScan[scanFlip];
    scanFlip ^= 1;
    if (lane == 31) buf[warp] = incl;
    __syncthreads();
    const int t = lane < nWarps ? buf[lane] : 0;
    int tincl = t;
    for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, tincl, o); if (lane >= o) tincl += u; }
    *total = __shfl_sync(0xffffffffu, tincl, nWarps - 1);
    return __shfl_sync(0xffffffffu, tincl - t, warp) + incl - v;
  };
  if (tid == 0) { sTicket = atomicAdd(P.ticket, 1) + 1; sBase = -1; } // the ticket starts at -1
  __syncthreads();
  const int b = sTicket;
  if (b >= P.batch) return;
  if (P.nextCounts) { // nothing reads these before the next launch, which stream order puts behind this one
    for (int l = tid; l < P.nLayers; l += NT) P.nextCounts[l * P.batch + b] = -1;
    if (b == 0) {
      if (tid == 0) *P.nextTicket = -1;
      for (int i = tid; i < P.nNextResults; i += NT) P.nextResults[i] = 0;
    }
  }

  int *inKeys = keysA, *outKeysS = keysB;
  int inBase = P.inOff[b];
  int nRows = P.inOff[b + 1] - inBase;
  int inBgGlobal = P.inBg ? P.inBg[b] : -1;
  if (nRows > P.rowsMax) { // the caller's bound was wrong: report on every layer and stop
    if (tid == 0) for (int l = 0; l < P.nLayers; ++l) { atomicOr(P.layers[l].result + 2, SCN_DEV_ERR_CAPACITY); P.counts[l * P.batch + b] = 0; }
    return;
  }
  for (int j = tid; j < nRows; j += NT) {
    const int k = P.inKeys[inBase + j];
    inKeys[j] = k;
    if (P.bgOut && k < 0) sBase = inBase + j; // at most one background row per sample
  }
  if (P.bgOut) {
    __syncthreads();
    inBgGlobal = sBase;
    if (tid == 0) P.bgOut[b] = inBgGlobal;
  }

  for (int l = 0; l < P.nLayers; ++l) {
    const ChainLayer &L = P.layers[l];
    __syncthreads();
    for (int i = tid; i < (int)(sizeof(Regions) / 4); i += NT) reinterpret_cast<int *>(&R)[i] = reinterpret_cast<const int *>(&L.R)[i];
    for (int w = tid; w < P.wMax; w += NT) dir[w] = make_uint2(0u, 0u);
    __syncthreads();
    // 1. occupancy bits
    for (int j = tid; j < nRows; j += NT) {
      const int key = inKeys[j];
      if (key < 0) continue;
      if (key >= R.cells) { atomicOr(L.result + 2, SCN_DEV_ERR_KEY); continue; }
      const unsigned bit = 1u << (key & 31);
      if (atomicOr(&dir[key >> 5].x, bit) & bit) atomicOr(L.result + 2, SCN_DEV_ERR_DUPLICATE);
    }
    __syncthreads();
    // 2. rank directory
    int nSites = 0;
    {
      int carry = 0;
      for (int w0 = 0; w0 < R.W; w0 += NT) {
        const int w = w0 + tid;
        const int c = (w < R.W) ? __popc(dir[w].x) : 0;
        int total;
        const int ex = scan(c, &total);
        if (w < R.W) dir[w].y = carry + ex;
        carry += total;
      }
      nSites = carry;
    }
    __syncthreads();
    if ((long long)nSites * R.T > P.flagBytes) { // more sites than the caller's hint allowed for
      if (tid == 0) { atomicOr(L.result + 2, SCN_DEV_ERR_CAPACITY); for (int l2 = l; l2 < P.nLayers; ++l2) P.counts[l2 * P.batch + b] = 0; }
      return;
    }
    // 3. ascending-key order, 4. which outputs each site creates
    for (int j = tid; j < nRows; j += NT) {
      const int key = inKeys[j];
      if (key >= 0 && key < R.cells) sorted[cell_rank(dir, key)] = j;
    }
    __syncthreads();
    for (int slot = tid; slot < nSites; slot += NT) {
      int i[DIM], j[DIM];
      decode_f<DIM>(inKeys[sorted[slot]], R.nIn, R.rNIn, i);
      int c = 0;
      if (DIM == 2 && R.stride == 1 && R.minActive >= 0 && R.minActive <= 1 && R.size <= 8 && R.lattice != SCN_LATTICE_TRIANGULAR && !R.fmp) {
        // Square filters of stride 1 in two dimensions: the `size` grid lines that can hold a smaller key than
        // this site's within any field it lies in are read once, as windows of 2 * size - 1 cells around the
        // site's column (cells off the grid read 0); each output's test is then two masks.
        const int y = i[0], x = i[DIM - 1], sz = R.size, left = x - sz + 1;
        const int c0 = max(left, 0), c1 = min(x + sz - 1, R.nIn - 1);
        unsigned win[7]; // the lines above the site's, nearest last
#pragma unroll
        for (int k = 0; k < 7; ++k) {
          const int yy = y - sz + 1 + k;
          win[k] = (k < sz - 1 && yy >= 0) ? range_bits(dir, yy * R.nIn + c0, c1 - c0 + 1) << (c0 - left) : 0u;
        }
        const unsigned own = range_bits(dir, y * R.nIn + c0, c1 - c0 + 1) << (c0 - left); // the site's own line
        const int loY = max(y - sz + 1, 0), hiY = min(y + 1, R.nOut), loX = max(left, 0), hiX = min(x + 1, R.nOut);
        const unsigned full = (1u << sz) - 1u;
        int t = 0;
        for (int ty = 0; ty < R.Tax; ++ty) {
          const int jy = loY + ty;
          unsigned above = 0u; // the field's lines in front of the site's
#pragma unroll
          for (int k = 0; k < 7; ++k)
            if (k < sz - 1 && y - sz + 1 + k >= jy) above |= win[k];
          for (int tx = 0; tx < R.Tax; ++tx, ++t) {
            const int jx = loX + tx, sh = jx - left;
            const bool ok = jy < hiY && jx < hiX;
            // cells of the field in front of the site: its lines above, and the site's own line left of it
            const unsigned blocked = ok ? (((above >> sh) & full) | ((own >> sh) & ((1u << (x - jx)) - 1u))) : 1u;
            const bool f = blocked == 0u;
            flags[slot * R.T + t] = f;
            c += f;
          }
        }
      } else {
        for (int t = 0; t < R.T; ++t) {
          const bool f = touched_output_f<DIM>(R, i, t, j) && creates_f<DIM>(R, dir, i, j);
          flags[slot * R.T + t] = f;
          c += f;
        }
      }
      cnt[slot] = c;
    }
    __syncthreads();
    // 5. prefix sums of the counts
    int sitesOut = 0;
    {
      int carry = 0;
      for (int s0 = 0; s0 < nSites; s0 += NT) {
        const int s = s0 + tid;
        const int c = (s < nSites) ? cnt[s] : 0;
        int total;
        const int ex = scan(c, &total);
        if (s < nSites) cnt[s] = carry + ex; // (read back by this thread only until the next barrier)
        carry += total;
      }
      sitesOut = carry; // every thread holds the total
    }
    const int needBg = sitesOut < R.fullSize;
    const int rowsOut = sitesOut + needBg;
    // 6. publish this sample's count, sum the earlier samples' counts
    if (tid == 0) { // (no fence: the other samples read nothing of this one but the count itself)
      atomicExch(P.counts + l * P.batch + b, rowsOut | (needBg << 30));
      atomicMax(L.result + 3, sitesOut);
      sBase = 0; sSitesBase = 0;
    }
    // 7a. output keys into the shared copy (the next layer's input): needs no other sample, so it runs
    // while the published count travels and the earlier samples' counts arrive
    // First the (site, output) pair behind every output row (a cheap pass over the flags), then one thread
    // per output row: the coordinate arithmetic runs once per output instead of once per warp and flag.
    if (rowsOut <= P.rowsMax) {
      for (int slot = tid; slot < nSites; slot += NT) {
        int r = cnt[slot];
        for (int t = 0; t < R.T; ++t)
          if (flags[slot * R.T + t]) pairs[r++] = slot * R.T + t;
      }
    }
    __syncthreads();
    if (rowsOut <= P.rowsMax) {
      for (int r = tid; r < sitesOut; r += NT) {
        int t;
        const int slot = fdiv(pairs[r], R.T, R.rT, &t);
        int i[DIM], j[DIM];
        decode_f<DIM>(inKeys[sorted[slot]], R.nIn, R.rNIn, i);
        touched_output_f<DIM>(R, i, t, j);
        outKeysS[r] = encode_f<DIM>(j, R.nOut);
#pragma unroll
        for (int a = 0; a < DIM; ++a) j[a] *= R.stride;
        pairs[r] = encode_f<DIM>(j, R.nIn); // from here on: the key of the first cell of the row's field
      }
      if (needBg && tid == 0) { outKeysS[sitesOut] = -1; pairs[sitesOut] = -1; }
      // key offset of every rule column's cell within a field
      for (int col = tid; col < R.sd; col += NT) {
        int cc[DIM];
        decode_f<DIM>(R.cellOfCol[col], R.size, R.rSize, cc);
        colOff[col] = encode_f<DIM>(cc, R.nIn);
      }
    }
    __syncthreads();
    {
      int rowsBefore = 0, bgBefore = 0;
      for (int p = tid; p < b; p += NT) {
        volatile int *slotp = P.counts + l * P.batch + p;
        int v = *slotp;
        if (v < 0) {
          const unsigned long long t0 = chain_ns();
          while ((v = *slotp) < 0) {
            if (chain_ns() - t0 > CHAIN_WAIT_NS) { atomicOr(L.result + 2, SCN_DEV_ERR_CAPACITY); v = 0; break; }
          }
        }
        rowsBefore += v & 0x3fffffff;
        bgBefore += (v >> 30) & 1;
      }
      if (rowsBefore) atomicAdd(&sBase, rowsBefore);
      if (bgBefore) atomicAdd(&sSitesBase, bgBefore);
    }
    __syncthreads();
    const int base = sBase;
    const bool fits = base + rowsOut <= L.capacity && rowsOut <= P.rowsMax;
    if (tid == 0) {
      L.outOff[b] = base;
      L.outBg[b] = needBg ? base + sitesOut : -1;
      if (!fits) atomicOr(L.result + 2, SCN_DEV_ERR_CAPACITY);
      if (b == P.batch - 1) {
        L.outOff[P.batch] = base + rowsOut;
        L.result[0] = base + rowsOut;
        L.result[1] = base + rowsOut - (sSitesBase + needBg);
      }
    }
    if (!fits) { // keep publishing zero-sized results so nobody behind this sample waits
      if (tid == 0) for (int l2 = l + 1; l2 < P.nLayers; ++l2) P.counts[l2 * P.batch + b] = 0;
      return;
    }
    // 7b. the interface's copy of the output keys (coalesced)
    for (int r = tid; r < rowsOut; r += NT) L.outKeys[base + r] = outKeysS[r];
    // 8. rule cells, coalesced over this sample's block of rows
    for (int q = tid; q < rowsOut * R.sd; q += NT) {
      int col;
      const int r = fdiv(q, R.sd, R.rSd, &col);
      const int first = pairs[r]; // key of the field's first cell, -1 on the background row
      int v = inBgGlobal;
      if (first >= 0) {
        const int ck = first + colOff[col];
        const uint2 e = dir[ck >> 5];
        if ((e.x >> (ck & 31)) & 1u) v = inBase + sorted[e.y + __popc(e.x & ((1u << (ck & 31)) - 1u))];
      }
      L.rules[(long long)base * R.sd + q] = v;
    }
    // the output is the next layer's input
    int *tmp = inKeys; inKeys = outKeysS; outKeysS = tmp;
    nRows = rowsOut;
    inBase = base;
    inBgGlobal = needBg ? base + sitesOut : -1;
  }
}

struct ChainPlan { int rowsMax, wMax, tMax; size_t smemBytes; bool ok; size_t flagBytes; };

// Shared-memory plan.  Without a hint the row bound is the worst case over the layers for a
// sample with at most `rowsIn` input rows; with a hint (rows per sample the caller expects at
// most, in any layer) the arrays are sized for the hint and the kernel reports
// SCN_DEV_ERR_CAPACITY if a sample exceeds it.
ChainPlan plan_chain(const Regions *Rs, int n, int rowsIn, int rowsHint) {
  ChainPlan p = {rowsIn, 1, 1, 0, true, 0};
  long long rows = rowsIn;
  size_t flagBytes = 0;
  for (int l = 0; l < n; ++l) {
    const Regions &R = Rs[l];
    if (R.W > p.wMax) p.wMax = R.W;
    if (R.T > p.tMax) p.tMax = R.T;
    flagBytes = std::max(flagBytes, (size_t)rows * R.T);
    long long out = std::min(rows * (long long)R.T, (long long)R.fullSize) + 1;
    rows = out;
    if (rows > p.rowsMax) p.rowsMax = (int)std::min<long long>(rows, 1 << 28);
  }
  if (rowsHint > 0 && rowsHint < p.rowsMax) {
    p.rowsMax = std::max(rowsHint, rowsIn);
    flagBytes = (size_t)p.rowsMax * p.tMax;
  }
  p.flagBytes = flagBytes;
  p.smemBytes = (size_t)p.wMax * 8 + (size_t)p.rowsMax * 12 + ((size_t)p.rowsMax + 1) * 8 + flagBytes + 64;
  p.ok = p.smemBytes <= 200 * 1024;
  return p;
}

} // namespace

} // namespace scn

using namespace scn;

extern "C" int scn_regions_cells(const scn_regions_t *r) {
  Regions R;
  if (make_regions(r, &R) != SCN_OK) return -1;
  return R.sd;
}

extern "C" size_t scn_rules_workspace_bytes(const scn_regions_t *r, int batch, int rows_in_bound) {
  Regions R;
  if (make_regions(r, &R) != SCN_OK || batch < 0 || rows_in_bound < 0) return 0;
  return carve(nullptr, batch, R.W, rows_in_bound, R.T).bytes;
}

static int run_rules(const Regions &R, int batch, const int *d_in_keys, const int *d_in_off, const int *d_in_bg, int rows_in_bound,
                     int *d_out_keys, int *d_out_off, int *d_out_bg, int *d_rules, int rows_out_capacity, int *d_result,
                     void *d_workspace, size_t workspace_bytes, scn_stream_t stream_);

extern "C" int scn_rules_build(const scn_regions_t *r, int batch, const int *d_in_keys, const int *d_in_off,
                               const int *d_in_bg, int rows_in_bound, int *d_out_keys, int *d_out_off,
                               int *d_out_bg, int *d_rules, int rows_out_capacity, int *d_result,
                               void *d_workspace, size_t workspace_bytes, scn_stream_t stream_) {
  clear_error();
  Regions R;
  int st = make_regions(r, &R);
  if (st != SCN_OK) return st;
  return run_rules(R, batch, d_in_keys, d_in_off, d_in_bg, rows_in_bound, d_out_keys, d_out_off, d_out_bg, d_rules, rows_out_capacity,
                   d_result, d_workspace, workspace_bytes, stream_);
}

// Regions of one fractional max-pooling layer: a square lattice whose `size` is the pool size; every
// input coordinate lies in at most `size` regions per axis.
static int make_fmp_regions(int dim, int nIn, int nOut, int poolSize, int overlapping, const int *d_ticks, Regions *out) {
  if (dim < 1 || dim > 4 || poolSize < 1 || nOut < 1) return fail(SCN_ERR_INVALID, "bad fractional pooling geometry");
  // the asserts of the tick constructors (Regions.cu:35, 58, 78, 104)
  if (nIn < nOut - 1 + poolSize || nIn <= nOut) return fail(SCN_ERR_INVALID, "fractional pooling needs nIn > nOut and nIn >= nOut - 1 + poolSize");
  scn_regions_t r = {SCN_LATTICE_SQUARE, dim, poolSize, 1, poolSize, 1, 1}; // a one-site stand-in for the shared bookkeeping
  Regions R;
  int st = make_regions(&r, &R);
  if (st != SCN_OK) return st;
  const long long cells = ipowll(nIn, dim), full = ipowll(nOut, dim);
  if (cells >= (1ll << 31)) return fail(SCN_ERR_UNSUPPORTED, "nIn^dim must be below 2^31");
  R.nIn = nIn; R.nOut = nOut; R.cells = (int)cells; R.W = (int)((cells + 31) / 32); R.fullSize = (int)full;
  R.Tax = poolSize; R.T = R.cube;
  R.rNIn = 1.0f / nIn; R.rNOut = 1.0f / nOut; R.rT = 1.0f / R.T; R.rTax = 1.0f / R.Tax;
  R.fmp = overlapping ? 1 : 2; R.tickStride = 2 * nOut + 2 * nIn; R.ticks = d_ticks;
  *out = R;
  return SCN_OK;
}

extern "C" size_t scn_fmp_rules_workspace_bytes(int dim, int nIn, int nOut, int poolSize, int batch, int rows_in_bound) {
  Regions R;
  if (batch < 0 || rows_in_bound < 0 || make_fmp_regions(dim, nIn, nOut, poolSize, 1, nullptr, &R) != SCN_OK) return 0;
  return carve(nullptr, batch, R.W, rows_in_bound, R.T).bytes;
}

extern "C" int scn_fmp_rules_build(int dim, int nIn, int nOut, int poolSize, int overlapping, int batch, const int *d_ticks,
                                   const int *d_in_keys, const int *d_in_off, const int *d_in_bg, int rows_in_bound,
                                   int *d_out_keys, int *d_out_off, int *d_out_bg, int *d_rules, int rows_out_capacity,
                                   int *d_result, void *d_workspace, size_t workspace_bytes, scn_stream_t stream_) {
  clear_error();
  Regions R;
  int st = make_fmp_regions(dim, nIn, nOut, poolSize, overlapping, d_ticks, &R);
  if (st != SCN_OK) return st;
  if (!d_ticks) return fail(SCN_ERR_INVALID, "null pointer");
  return run_rules(R, batch, d_in_keys, d_in_off, d_in_bg, rows_in_bound, d_out_keys, d_out_off, d_out_bg, d_rules, rows_out_capacity,
                   d_result, d_workspace, workspace_bytes, stream_);
}

static int run_rules(const Regions &R, int batch, const int *d_in_keys, const int *d_in_off, const int *d_in_bg, int rows_in_bound,
                     int *d_out_keys, int *d_out_off, int *d_out_bg, int *d_rules, int rows_out_capacity, int *d_result,
                     void *d_workspace, size_t workspace_bytes, scn_stream_t stream_) {
  if (batch < 1 || rows_in_bound < 0 || rows_out_capacity < 0) return fail(SCN_ERR_INVALID, "bad batch/row counts");
  if ((!d_in_keys && rows_in_bound > 0) || !d_in_off || !d_in_bg || !d_out_keys || !d_out_off || !d_out_bg || !d_rules || !d_result || !d_workspace)
    return fail(SCN_ERR_INVALID, "null pointer");
  Workspace w = carve(d_workspace, batch, R.W, rows_in_bound, R.T);
  if (w.bytes > workspace_bytes) return fail(SCN_ERR_WORKSPACE, "workspace smaller than scn_rules_workspace_bytes()");
  cudaStream_t s = (cudaStream_t)stream_;
  const int rows = rows_in_bound > 0 ? rows_in_bound : 1;

  SCN_CUDA_TRY(cudaMemsetAsync(w.dir, 0, (size_t)batch * R.W * sizeof(uint2), s));
  SCN_CUDA_TRY(cudaMemsetAsync(w.cnt, 0, ((size_t)rows_in_bound + 1) * sizeof(int), s));
  SCN_CUDA_TRY(cudaMemsetAsync(d_result, 0, 4 * sizeof(int), s));
  // slots no site maps to (a sample's background row, skipped keys) must read as "creates nothing"
  if (rows_in_bound > 0) SCN_CUDA_TRY(cudaMemsetAsync(w.flags, 0, (size_t)rows_in_bound * R.T, s));
  k_mark<<<grid_for(rows, 256), 256, 0, s>>>(R, batch, d_in_keys, d_in_off, w.dir, d_result);
  SCN_LAUNCH_CHECK("k_mark");
  k_rank<<<batch < sm_count() * 4 ? batch : sm_count() * 4, 256, 0, s>>>(R, batch, w.dir, w.nSites);
  SCN_LAUNCH_CHECK("k_rank");
  const bool fast = R.cells < (1 << 24) && !R.fmp; // float-assisted coordinate arithmetic is exact below 2^24
#define SCN_DIM_DISPATCH(KERNEL, GRID, BLOCK, ...)                                                       \
  switch (R.dim) {                                                                                       \
  case 1: KERNEL<1><<<GRID, BLOCK, 0, s>>>(__VA_ARGS__); break;                                          \
  case 2: KERNEL<2><<<GRID, BLOCK, 0, s>>>(__VA_ARGS__); break;                                          \
  case 3: KERNEL<3><<<GRID, BLOCK, 0, s>>>(__VA_ARGS__); break;                                          \
  default: KERNEL<4><<<GRID, BLOCK, 0, s>>>(__VA_ARGS__); break;                                         \
  }
  if (fast) { SCN_DIM_DISPATCH(k_flags_t, grid_for(rows, 128), 128, R, batch, d_in_keys, d_in_off, w.dir, w.sortedRow, w.flags, w.cnt) }
  else k_flags<<<grid_for(rows, 128), 128, 0, s>>>(R, batch, d_in_keys, d_in_off, w.dir, w.sortedRow, w.flags, w.cnt, true);
  SCN_LAUNCH_CHECK("k_flags");
  const int chunks = rows / SCAN_CHUNK + 1;
  k_scan_reduce<<<grid_for(chunks, 1), SCAN_THREADS, 0, s>>>(w.cnt, d_in_off, batch, w.partial);
  SCN_LAUNCH_CHECK("k_scan_reduce");
  k_scan_partials<<<1, 1024, 0, s>>>(d_in_off, batch, w.partial);
  SCN_LAUNCH_CHECK("k_scan_partials");
  k_scan_apply<<<grid_for(chunks, 1), SCAN_THREADS, 0, s>>>(w.cnt, d_in_off, batch, w.partial);
  SCN_LAUNCH_CHECK("k_scan_apply");
  k_samples<<<1, 1024, 0, s>>>(R, batch, d_in_off, w.cnt, d_out_off, d_out_bg, d_out_keys, rows_out_capacity, d_result);
  SCN_LAUNCH_CHECK("k_samples");
  if (fast) { SCN_DIM_DISPATCH(k_assign_t, grid_for((long long)rows * R.T, 256), 256, R, batch, d_in_keys, d_in_off, w.sortedRow, w.flags, w.cnt, d_out_off, d_out_keys, rows_out_capacity) }
  else k_assign<<<grid_for((long long)rows * R.T, 256), 256, 0, s>>>(R, batch, d_in_keys, d_in_off, w.sortedRow, w.flags, w.cnt,
                                                                      d_out_off, d_out_keys, rows_out_capacity);
  SCN_LAUNCH_CHECK("k_assign");
  const int fillGrid = fast ? grid_for((long long)(rows_out_capacity > 0 ? rows_out_capacity : 1) * 4, 256)  // 64 rows per block and trip
                            : grid_for((long long)(rows_out_capacity > 0 ? rows_out_capacity : 1) * R.sd, 256);
  if (fast) { SCN_DIM_DISPATCH(k_fill_t, fillGrid, 256, R, batch, d_in_off, d_in_bg, w.dir, w.sortedRow, d_out_off, d_out_keys, d_rules, rows_out_capacity, d_result) }
  else k_fill<<<fillGrid, 256, 0, s>>>(R, batch, d_in_off, d_in_bg, w.dir, w.sortedRow, d_out_off, d_out_keys, d_rules, rows_out_capacity, d_result);
  SCN_LAUNCH_CHECK("k_fill");
#undef SCN_DIM_DISPATCH
  return SCN_OK;
}

extern "C" size_t scn_terminal_rules_workspace_bytes(int dim, int spatial_size, int batch, int rows_in_bound) {
  if (dim < 1 || dim > 4 || spatial_size < 1 || batch < 0 || rows_in_bound < 0) return 0;
  long long cells = ipowll(spatial_size, dim);
  if (cells >= (1ll << 31)) return 0;
  return carve(nullptr, batch, (int)((cells + 31) / 32), rows_in_bound, 0).bytes;
}

extern "C" int scn_terminal_rules_build(int dim, int spatial_size, int batch, const int *d_in_keys,
                                        const int *d_in_off, const int *d_in_bg, int rows_in_bound, int S,
                                        int *d_out_keys, int *d_out_off, int *d_out_bg, int *d_rules,
                                        int *d_result, void *d_workspace, size_t workspace_bytes,
                                        scn_stream_t stream_) {
  clear_error();
  if (dim < 1 || dim > 4 || spatial_size < 1 || batch < 1 || rows_in_bound < 0 || S < 1)
    return fail(SCN_ERR_INVALID, "bad terminal pooling geometry");
  if ((!d_in_keys && rows_in_bound > 0) || !d_in_off || !d_in_bg || !d_out_keys || !d_out_off || !d_out_bg || !d_rules || !d_result || !d_workspace)
    return fail(SCN_ERR_INVALID, "null pointer");
  long long cells = ipowll(spatial_size, dim);
  if (cells >= (1ll << 31)) return fail(SCN_ERR_UNSUPPORTED, "spatial_size^dim must be below 2^31");
  Regions R = {};
  R.dim = dim; R.nIn = spatial_size; R.cells = (int)cells; R.W = (int)((cells + 31) / 32); R.T = 0;
  Workspace w = carve(d_workspace, batch, R.W, rows_in_bound, 0);
  if (w.bytes > workspace_bytes) return fail(SCN_ERR_WORKSPACE, "workspace smaller than scn_terminal_rules_workspace_bytes()");
  cudaStream_t s = (cudaStream_t)stream_;
  const int rows = rows_in_bound > 0 ? rows_in_bound : 1;
  SCN_CUDA_TRY(cudaMemsetAsync(w.dir, 0, (size_t)batch * R.W * sizeof(uint2), s));
  SCN_CUDA_TRY(cudaMemsetAsync(d_result, 0, 4 * sizeof(int), s));
  k_mark<<<grid_for(rows, 256), 256, 0, s>>>(R, batch, d_in_keys, d_in_off, w.dir, d_result);
  SCN_LAUNCH_CHECK("k_mark");
  k_rank<<<batch < sm_count() * 4 ? batch : sm_count() * 4, 256, 0, s>>>(R, batch, w.dir, w.nSites);
  SCN_LAUNCH_CHECK("k_rank");
  k_flags<<<grid_for(rows, 128), 128, 0, s>>>(R, batch, d_in_keys, d_in_off, w.dir, w.sortedRow, nullptr, nullptr, false);
  SCN_LAUNCH_CHECK("k_flags");
  k_terminal<<<grid_for((long long)batch * S, 256), 256, 0, s>>>(batch, S, d_in_off, d_in_bg, w.nSites, w.sortedRow, d_rules,
                                                                d_out_keys, d_out_off, d_out_bg, d_result);
  SCN_LAUNCH_CHECK("k_terminal");
  return SCN_OK;
}

// ---------------------------------------------------------------------------------------------
// Rule construction for callers that may not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need rules: code
// running inside a framework that owns all device memory and forbids foreign allocations, a
// real-time loop that must not take the allocator's lock or risk a device synchronisation,
// a plugin loaded after the process has handed every free byte to a memory pool.  For them the
// scratch that scn_rules_build takes from its caller lives here, in a fixed array inside the
// library image: every device that loads the library holds these bytes from load until exit.
namespace {
constexpr size_t STATIC_SCRATCH_BYTES = (size_t)SCN_RULES_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];
// In host code `g_static_scratch` is only a stand-in for the symbol, not a device address; the
// address is asked from the runtime once per device, with that device current.
void *g_static_scratch_ptr[64] = {nullptr};
std::mutex g_static_scratch_mu;
} // namespace

extern "C" size_t scn_rules_static_scratch_bytes(void) { return STATIC_SCRATCH_BYTES; }

extern "C" int scn_rules_build_static(const scn_regions_t *r, int batch, const int *d_in_keys, const int *d_in_off,
                                      const int *d_in_bg, int rows_in_bound, int *d_out_keys, int *d_out_off,
                                      int *d_out_bg, int *d_rules, int rows_out_capacity, int *d_result,
                                      scn_stream_t stream) {
  clear_error();
  Regions R;
  int st = make_regions(r, &R);
  if (st != SCN_OK) return st;
  if (batch < 1 || rows_in_bound < 0) return fail(SCN_ERR_INVALID, "bad batch/row counts");
  const size_t need = carve(nullptr, batch, R.W, rows_in_bound, R.T).bytes;
  if (need > STATIC_SCRATCH_BYTES) {
    set_error("this build needs %zu bytes of scratch but the library's fixed scratch array holds %zu: "
              "use smaller batches or scn_rules_build with a caller-owned workspace", need, STATIC_SCRATCH_BYTES);
    return SCN_ERR_WORKSPACE;
  }
  int dev = 0;
  SCN_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(SCN_ERR_UNSUPPORTED, "device ordinal beyond 63");
  void *scratch = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_static_scratch_mu);
    if (!g_static_scratch_ptr[dev]) { // first call on this device: resolve the array's device address
      void *p = nullptr;
      SCN_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
      g_static_scratch_ptr[dev] = p;
    }
    scratch = g_static_scratch_ptr[dev];
  }
  // Same kernels as the allocating caller's path; they zero every part of the scratch that must
  // start at zero (bitmap, counts, flags), so what the previous call left behind does not matter.
  return scn_rules_build(r, batch, d_in_keys, d_in_off, d_in_bg, rows_in_bound, d_out_keys, d_out_off, d_out_bg, d_rules,
                         rows_out_capacity, d_result, scratch, STATIC_SCRATCH_BYTES, stream);
}

// ---------------------------------------------------------------------------------------------
extern "C" size_t scn_rules_chain_workspace_bytes(int n_layers, int batch) {
  if (n_layers < 1 || batch < 1) return 0;
  return align_up(sizeof(ChainLayer) * (size_t)n_layers, 256) + align_up(sizeof(int) * ((size_t)n_layers * batch + 1), 256);
}

extern "C" int scn_rules_chain_supported(const scn_chain_layer_t *layers, int n_layers, int batch, int max_rows_per_sample,
                                         int rows_hint) {
  if (!layers || n_layers < 1 || n_layers > 64 || batch < 1 || max_rows_per_sample < 0) return 0;
  std::vector<Regions> Rs(n_layers);
  for (int l = 0; l < n_layers; ++l)
    if (make_regions(&layers[l].regions, &Rs[l]) != SCN_OK) return 0;
  clear_error();
  return plan_chain(Rs.data(), n_layers, max_rows_per_sample, rows_hint).ok ? 1 : 0;
}

namespace {
// Checks the caller's layers and turns them into kernel descriptors and a shared-memory plan.
int chain_prepare(const scn_chain_layer_t *layers, int n_layers, int batch, int max_rows_per_sample, int rows_hint,
                  std::vector<ChainLayer> &h, ChainPlan &plan, int *dim) {
  if (!layers || n_layers < 1 || n_layers > 64 || batch < 1 || max_rows_per_sample < 0) return fail(SCN_ERR_INVALID, "bad chain arguments");
  h.resize(n_layers);
  std::vector<Regions> Rs(n_layers);
  for (int l = 0; l < n_layers; ++l) {
    int st = make_regions(&layers[l].regions, &Rs[l]);
    if (st != SCN_OK) return st;
    if (!layers[l].d_out_keys || !layers[l].d_out_off || !layers[l].d_out_bg || !layers[l].d_rules || !layers[l].d_result)
      return fail(SCN_ERR_INVALID, "null pointer in a chain layer");
    if (l > 0 && (Rs[l].nIn != Rs[l - 1].nOut || Rs[l].dim != Rs[l - 1].dim)) return fail(SCN_ERR_INVALID, "chain layers do not fit together");
    std::memset(&h[l], 0, sizeof(ChainLayer)); // descriptors are compared bytewise by the resident build: no stray padding
    h[l].R = Rs[l];
    h[l].outKeys = layers[l].d_out_keys; h[l].outOff = layers[l].d_out_off; h[l].outBg = layers[l].d_out_bg;
    h[l].rules = layers[l].d_rules; h[l].result = layers[l].d_result; h[l].capacity = layers[l].rows_out_capacity;
  }
  plan = plan_chain(Rs.data(), n_layers, max_rows_per_sample, rows_hint);
  if (!plan.ok) return fail(SCN_ERR_UNSUPPORTED, "samples too large for the fused rule chain: build layer by layer with scn_rules_build");
  *dim = Rs[0].dim;
  return SCN_OK;
}

int chain_launch(ChainParams &P, const ChainPlan &plan, int dim, int batch, cudaStream_t s) {
  static bool attrSet[64] = {false};
  int dev = 0;
  SCN_CUDA_TRY(cudaGetDevice(&dev));
  if (!attrSet[dev & 63]) {
    SCN_CUDA_TRY(cudaFuncSetAttribute(k_rule_chain<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    SCN_CUDA_TRY(cudaFuncSetAttribute(k_rule_chain<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    SCN_CUDA_TRY(cudaFuncSetAttribute(k_rule_chain<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    SCN_CUDA_TRY(cudaFuncSetAttribute(k_rule_chain<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attrSet[dev & 63] = true;
  }
  P.batch = batch;
  P.rowsMax = plan.rowsMax; P.wMax = plan.wMax; P.tMax = plan.tMax; P.flagBytes = (int)std::min<size_t>(plan.flagBytes, 0x7fffffff);
  const int chainThreads = CHAIN_THREADS;
  switch (dim) {
  case 1: k_rule_chain<1><<<batch, chainThreads, plan.smemBytes, s>>>(P); break;
  case 2: k_rule_chain<2><<<batch, chainThreads, plan.smemBytes, s>>>(P); break;
  case 3: k_rule_chain<3><<<batch, chainThreads, plan.smemBytes, s>>>(P); break;
  default: k_rule_chain<4><<<batch, chainThreads, plan.smemBytes, s>>>(P); break;
  }
  SCN_LAUNCH_CHECK("k_rule_chain");
  return SCN_OK;
}
} // namespace

extern "C" int scn_rules_chain_build(const scn_chain_layer_t *layers, int n_layers, int batch, const int *d_in_keys,
                                     const int *d_in_off, const int *d_in_bg, int max_rows_per_sample, int rows_hint,
                                     void *d_workspace, size_t workspace_bytes, scn_stream_t stream_) {
  clear_error();
  if (!d_in_off || !d_in_bg || !d_workspace) return fail(SCN_ERR_INVALID, "null pointer");
  std::vector<ChainLayer> h;
  ChainPlan plan;
  int dim = 0;
  int st = chain_prepare(layers, n_layers, batch, max_rows_per_sample, rows_hint, h, plan, &dim);
  if (st != SCN_OK) return st;
  if (scn_rules_chain_workspace_bytes(n_layers, batch) > workspace_bytes) return fail(SCN_ERR_WORKSPACE, "workspace smaller than scn_rules_chain_workspace_bytes()");
  cudaStream_t s = (cudaStream_t)stream_;
  ChainLayer *dLayers = (ChainLayer *)d_workspace;
  int *counts = (int *)((char *)d_workspace + align_up(sizeof(ChainLayer) * (size_t)n_layers, 256));
  int *ticket = counts + (size_t)n_layers * batch;
  // the descriptors travel through a pinned-free path: a small synchronous-to-stream copy from pageable memory
  SCN_CUDA_TRY(cudaMemcpyAsync(dLayers, h.data(), sizeof(ChainLayer) * n_layers, cudaMemcpyHostToDevice, s));
  // few stream operations in front of the kernel (each costs a couple of microseconds of an idle GPU): counts and
  // ticket are set by one fill (the ticket counts up from -1), the result records by one when they are contiguous
  SCN_CUDA_TRY(cudaMemsetAsync(counts, 0xff, sizeof(int) * ((size_t)n_layers * batch + 1), s));
  bool contiguous = true;
  for (int l = 1; l < n_layers; ++l) contiguous = contiguous && layers[l].d_result == layers[0].d_result + 4 * l;
  if (contiguous) SCN_CUDA_TRY(cudaMemsetAsync(layers[0].d_result, 0, 4 * sizeof(int) * (size_t)n_layers, s));
  else for (int l = 0; l < n_layers; ++l) SCN_CUDA_TRY(cudaMemsetAsync(layers[l].d_result, 0, 4 * sizeof(int), s));
  ChainParams P;
  P.layers = dLayers; P.nLayers = n_layers;
  P.inKeys = d_in_keys; P.inOff = d_in_off; P.inBg = d_in_bg;
  P.counts = counts; P.ticket = ticket;
  P.nextCounts = nullptr; P.nextTicket = nullptr; P.nextResults = nullptr; P.nNextResults = 0; P.bgOut = nullptr;
  return chain_launch(P, plan, dim, batch, s);
}

// ---- resident form: the caller keeps the workspace to itself, so the state of one launch is prepared by the launch before it
struct scn_chain_resident {
  void *workspace = nullptr;            // the device block the shadows below describe
  int nLayers = 0, batch = 0;
  std::vector<ChainLayer> shadow[2];    // descriptors resident on the device, per phase
  bool ready[2] = {false, false};       // phase state (counters, ticket, result records) prepared by the launch before
  int *preparedResults = nullptr;       // the result records that launch cleared
  int lastPhase = -1;
};

extern "C" scn_chain_resident_t *scn_rules_chain_resident_create(void) { return new (std::nothrow) scn_chain_resident(); }
extern "C" void scn_rules_chain_resident_destroy(scn_chain_resident_t *st) { delete st; }
extern "C" void scn_rules_chain_resident_invalidate(scn_chain_resident_t *st) {
  if (st) { st->workspace = nullptr; st->ready[0] = st->ready[1] = false; st->shadow[0].clear(); st->shadow[1].clear(); st->lastPhase = -1; }
}
extern "C" size_t scn_rules_chain_resident_workspace_bytes(int n_layers, int batch) {
  return 2 * scn_rules_chain_workspace_bytes(n_layers, batch);
}

extern "C" int scn_rules_chain_build_resident(scn_chain_resident_t *st, const scn_chain_layer_t *layers, int n_layers, int batch,
                                              const int *d_in_keys, const int *d_in_off, const int *d_in_bg, int *d_in_bg_out,
                                              int max_rows_per_sample, int rows_hint, void *d_workspace, size_t workspace_bytes,
                                              int phase, int *d_result_next, int n_result_next, scn_stream_t stream_) {
  clear_error();
  if (!st || !d_in_off || !d_workspace || (phase != 0 && phase != 1)) return fail(SCN_ERR_INVALID, "bad resident chain arguments");
  if (!d_in_bg && !d_in_bg_out) return fail(SCN_ERR_INVALID, "need the background rows or a place to write them");
  std::vector<ChainLayer> h;
  ChainPlan plan;
  int dim = 0;
  int rc = chain_prepare(layers, n_layers, batch, max_rows_per_sample, rows_hint, h, plan, &dim);
  if (rc != SCN_OK) return rc;
  if (d_result_next && n_result_next < 1) return fail(SCN_ERR_INVALID, "resident chain: n_result_next must be positive");
  const size_t half = scn_rules_chain_workspace_bytes(n_layers, batch);
  if (2 * half > workspace_bytes) return fail(SCN_ERR_WORKSPACE, "workspace smaller than scn_rules_chain_resident_workspace_bytes()");
  cudaStream_t s = (cudaStream_t)stream_;
  if (st->workspace != d_workspace || st->nLayers != n_layers || st->batch != batch) {
    scn_rules_chain_resident_invalidate(st);
    st->workspace = d_workspace; st->nLayers = n_layers; st->batch = batch;
  }
  char *base = (char *)d_workspace + (size_t)phase * half, *other = (char *)d_workspace + (size_t)(1 - phase) * half;
  const size_t descBytes = align_up(sizeof(ChainLayer) * (size_t)n_layers, 256);
  ChainLayer *dLayers = (ChainLayer *)base;
  int *counts = (int *)(base + descBytes), *ticket = counts + (size_t)n_layers * batch;
  int *nextCounts = (int *)(other + descBytes), *nextTicket = nextCounts + (size_t)n_layers * batch;
  if (st->shadow[phase].size() != (size_t)n_layers || std::memcmp(st->shadow[phase].data(), h.data(), sizeof(ChainLayer) * n_layers) != 0) {
    SCN_CUDA_TRY(cudaMemcpyAsync(dLayers, h.data(), sizeof(ChainLayer) * n_layers, cudaMemcpyHostToDevice, s));
    st->shadow[phase] = h;
  }
  if (!st->ready[phase] || st->lastPhase == phase || st->preparedResults != layers[0].d_result) { // first use of this phase, the same phase twice, other result records: prepare it here
    SCN_CUDA_TRY(cudaMemsetAsync(counts, 0xff, sizeof(int) * ((size_t)n_layers * batch + 1), s));
    for (int l = 0; l < n_layers; ++l) SCN_CUDA_TRY(cudaMemsetAsync(layers[l].d_result, 0, 4 * sizeof(int), s));
  }
  ChainParams P;
  P.layers = dLayers; P.nLayers = n_layers;
  P.inKeys = d_in_keys; P.inOff = d_in_off; P.inBg = d_in_bg;
  P.counts = counts; P.ticket = ticket;
  P.nNextResults = d_result_next ? n_result_next : 0;
  P.nextCounts = d_result_next ? nextCounts : nullptr; P.nextTicket = d_result_next ? nextTicket : nullptr; P.nextResults = d_result_next;
  P.bgOut = d_in_bg ? nullptr : d_in_bg_out;
  rc = chain_launch(P, plan, dim, batch, s);
  st->ready[phase] = false;
  st->ready[1 - phase] = (rc == SCN_OK && d_result_next != nullptr);
  st->preparedResults = d_result_next;
  st->lastPhase = phase;
  return rc;
}
