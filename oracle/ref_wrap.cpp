// TEST INFRASTRUCTURE ONLY.  C wrapper around the REFERENCE's own host rule construction,
// compiled from the reference sources where they lie (see oracle/Makefile, target _ref).
// Nothing here restates an algorithm: it builds `SparseGrid` objects from flat arrays,
// calls the reference's `gridRules` overloads (Regions.h:84-87 square/cubic lattices,
// Regions.h:120-127 triangular/tetrahedral lattices) once per sample exactly as the layer
// `preprocess` methods do (ConvolutionalLayer.cu:111-118, MaxPoolingLayer.cu:113-118,
// ConvolutionalTriangularLayer.cu:35-39, MaxPoolingTriangularLayer.cu:29-33), and flattens
// the results.  It pins oracle/scn_oracle.cpp and generates tests/golden/*.
#include "Regions.h"
#include "utilities.h"
#include <cstdint>
#include <cstring>
#include <vector>

namespace {
struct RefResult {
  std::vector<int> rules;
  std::vector<int64_t> outKeys; // per sample, in the map's iteration order
  std::vector<int> outRows;
  std::vector<int> outOff; // batch+1 offsets into outKeys/outRows
  std::vector<int> outBg;  // batch
  int nOutSites = 0;
};
} // namespace

template <class T>
static void fmpSample(RNG &rng, int dim, int nIn, int nOut, int poolSize, bool uniform, SparseGrid &in, SparseGrid &out,
                      RefResult *res, int *ticksOut) {
  FractionalPoolingRegions<T> regions(nIn, nOut, dim, poolSize, rng);
  for (int a = 0; a < dim; ++a) {
    int *t = ticksOut + a * (2 * nOut + 2 * nIn);
    for (int j = 0; j < nOut; ++j) { t[j] = regions.inputL(a, j); t[nOut + j] = regions.inputR(a, j); }
    for (int i = 0; i < nIn; ++i) { t[2 * nOut + i] = regions.outputL(a, i); t[2 * nOut + nIn + i] = regions.outputR(a, i); }
  }
  gridRules(in, out, regions, res->nOutSites, res->rules, uniform);
}
extern "C" {

// kind: 0 = RegularSquareRegions, 1 = RegularTriangularRegions.
// Input grids: sample b owns entries [inOff[b], inOff[b+1]) of (inKeys, inRows);
// inBg[b] is its SparseGrid::backgroundCol.  Entries are inserted in the order given.
void *ref_grid_rules(int kind, int dim, int nIn, int nOut, int size, int stride,
                     int minActive, int batch, const int64_t *inKeys,
                     const int *inRows, const int *inOff, const int *inBg) {
  RefResult *res = new RefResult();
  res->outOff.push_back(0);
  for (int b = 0; b < batch; ++b) {
    SparseGrid in, out;
    in.backgroundCol = inBg[b];
    for (int i = inOff[b]; i < inOff[b + 1]; ++i)
      in.mp[inKeys[i]] = inRows[i];
    if (kind == 0) {
      RegularSquareRegions regions(nIn, nOut, dim, size, stride);
      gridRules(in, out, regions, res->nOutSites, res->rules, true, minActive);
    } else {
      RegularTriangularRegions regions(nIn, nOut, dim, size, stride);
      gridRules(in, out, regions, res->nOutSites, res->rules, minActive);
    }
    for (auto it = out.mp.begin(); it != out.mp.end(); ++it) {
      res->outKeys.push_back((int64_t)it->first);
      res->outRows.push_back(it->second);
    }
    res->outOff.push_back((int)res->outKeys.size());
    res->outBg.push_back(out.backgroundCol);
  }
  return res;
}

// Fractional max-pooling rules as the four FMP layers' preprocess() builds them
// (MaxPoolingLayer.cu:171-186, 232-247, 293-308, 354-369): one RNG per layer, per sample a fresh
// FractionalPoolingRegions<ticks> (one ticks object per axis) and gridRules with uniformSizeRegions
// = true for the overlapping kinds, false for the non-overlapping ones.  The reference seeds the
// RNG from the clock; here rng.gen is re-seeded so that the draw sequence can be repeated.
// kind: 0 pseudorandom overlapping, 1 pseudorandom non-overlapping, 2 random overlapping,
// 3 random non-overlapping.  ticksOut[(b*dim + axis) * (2*nOut + 2*nIn)] receives
// inputL[nOut], inputR[nOut], outputL[nIn], outputR[nIn] of every sample and axis.
void *ref_fmp_rules(int kind, int dim, int nIn, int nOut, int poolSize, unsigned seed, int batch, const int64_t *inKeys,
                    const int *inRows, const int *inOff, const int *inBg, int *ticksOut) {
  RefResult *res = new RefResult();
  res->outOff.push_back(0);
  RNG rng;
  rng.gen.seed(seed);
  for (int b = 0; b < batch; ++b) {
    SparseGrid in, out;
    in.backgroundCol = inBg[b];
    for (int i = inOff[b]; i < inOff[b + 1]; ++i)
      in.mp[inKeys[i]] = inRows[i];
    int *t = ticksOut + (size_t)b * dim * (2 * nOut + 2 * nIn);
    if (kind == 0) fmpSample<PseudorandomOverlappingFmpTicks>(rng, dim, nIn, nOut, poolSize, true, in, out, res, t);
    else if (kind == 1) fmpSample<PseudorandomNonOverlappingFmpTicks>(rng, dim, nIn, nOut, poolSize, false, in, out, res, t);
    else if (kind == 2) fmpSample<RandomOverlappingFmpTicks>(rng, dim, nIn, nOut, poolSize, true, in, out, res, t);
    else fmpSample<RandomNonOverlappingFmpTicks>(rng, dim, nIn, nOut, poolSize, false, in, out, res, t);
    for (auto it = out.mp.begin(); it != out.mp.end(); ++it) {
      res->outKeys.push_back((int64_t)it->first);
      res->outRows.push_back(it->second);
    }
    res->outOff.push_back((int)res->outKeys.size());
    res->outBg.push_back(out.backgroundCol);
  }
  return res;
}

long long ref_result_n_rules(void *h) { return (long long)((RefResult *)h)->rules.size(); }
long long ref_result_n_out(void *h) { return (long long)((RefResult *)h)->outKeys.size(); }
int ref_result_n_sites(void *h) { return ((RefResult *)h)->nOutSites; }

void ref_result_fetch(void *h, int *rules, int64_t *outKeys, int *outRows, int *outOff,
                      int *outBg) {
  RefResult *r = (RefResult *)h;
  if (!r->rules.empty())
    std::memcpy(rules, r->rules.data(), r->rules.size() * sizeof(int));
  if (!r->outKeys.empty()) {
    std::memcpy(outKeys, r->outKeys.data(), r->outKeys.size() * sizeof(int64_t));
    std::memcpy(outRows, r->outRows.data(), r->outRows.size() * sizeof(int));
  }
  std::memcpy(outOff, r->outOff.data(), r->outOff.size() * sizeof(int));
  if (!r->outBg.empty())
    std::memcpy(outBg, r->outBg.data(), r->outBg.size() * sizeof(int));
}

void ref_result_free(void *h) { delete (RefResult *)h; }

// The reference's scalar helpers, exported so the oracle's copies can be pinned.
int ref_ipow(int base, int exp) { return ipow(base, exp); }
int ref_triangleSize(int linearSize, int dimension) {
  return triangleSize(linearSize, dimension);
}
int ref_intRound(int a, int d) { return intRound(a, d); }
// utilities.cu:35-56; requires n >= k >= 1.
void ref_vectorTopIndices(const float *v, int n, int k, int *out) {
  std::vector<float> test(v, v + n);
  std::vector<int> idx = vectorTopIndices(test, k);
  std::memcpy(out, idx.data(), k * sizeof(int));
}
}
