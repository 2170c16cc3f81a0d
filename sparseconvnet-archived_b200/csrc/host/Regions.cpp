#include "Regions.h"
#include <algorithm>
#include <cmath>

RectangularRegions::RectangularRegions(int nIn, int nOut, int dimension, int s)
    : nIn(nIn), nOut(nOut), dimension(dimension), s(s), sd(ipow(s, dimension)) {}
RectangularRegions::~RectangularRegions() {}

RegularSquareRegions::RegularSquareRegions(int nIn, int nOut, int dimension, int poolSize, int poolStride)
    : RectangularRegions(nIn, nOut, dimension, poolSize), poolSize(poolSize), poolStride(poolStride) {
  if (nIn != poolSize + (nOut - 1) * poolStride) throw ScnException("RegularSquareRegions: nIn != poolSize + (nOut-1)*poolStride");
}
RegularSquareRegions::~RegularSquareRegions() {}
int RegularSquareRegions::inputL(int, int j) { return j * poolStride; }
int RegularSquareRegions::inputR(int, int j) { return j * poolStride + poolSize; }
int RegularSquareRegions::outputL(int, int i) { return std::max(0, (i - poolSize + poolStride) / poolStride); }
int RegularSquareRegions::outputR(int, int i) { return std::min(i / poolStride + 1, nOut); }

// ---- fractional max-pooling ticks (Regions.cu:31-125)
void FractionalMaxPoolingTicks::fillOutputRanges(int nIn, int nOut) {
  outputL.assign(nIn, nOut);
  outputR.assign(nIn, 0);
  for (int i = 0; i < nOut; i++)
    for (int j = inputL[i]; j < inputR[i]; j++) {
      outputL[j] = std::min(outputL[j], i);
      outputR[j] = std::max(outputR[j], i + 1);
    }
}
PseudorandomOverlappingFmpTicks::PseudorandomOverlappingFmpTicks(int nIn, int nOut, int poolSize, RNG &rng) {
  if (nIn < nOut - 1 + poolSize || nOut < 2) throw ScnException("PseudorandomOverlappingFmpTicks: needs nIn >= nOut - 1 + poolSize and nOut >= 2");
  const double alpha = (nIn - poolSize) * 1.0 / (nOut - 1);
  const double u = rng.uniform(0, 1);
  for (int j = 0; j < nOut; ++j) {
    const int i = (int)((j + u) * alpha) - (int)(u * alpha);
    inputL.push_back(i);
    inputR.push_back(i + poolSize);
  }
  if (inputR.back() != nIn) throw ScnException("PseudorandomOverlappingFmpTicks: regions do not end at nIn");
  fillOutputRanges(nIn, nOut);
}
PseudorandomNonOverlappingFmpTicks::PseudorandomNonOverlappingFmpTicks(int nIn, int nOut, int poolSize, RNG &rng) {
  const double alpha = nIn * 1.0 / nOut;
  const double u = rng.uniform(0, 1);
  if (nIn < nOut - 1 + poolSize || (int)std::ceil(alpha) != poolSize) throw ScnException("PseudorandomNonOverlappingFmpTicks: needs ceil(nIn/nOut) == poolSize");
  for (int j = 0; j < nOut; ++j) inputL.push_back((int)((j + u) * alpha) - (int)(u * alpha));
  for (int j = 1; j <= nOut; ++j) inputR.push_back((int)((j + u) * alpha) - (int)(u * alpha));
  if (inputR.back() != nIn) throw ScnException("PseudorandomNonOverlappingFmpTicks: regions do not end at nIn");
  fillOutputRanges(nIn, nOut);
}
RandomOverlappingFmpTicks::RandomOverlappingFmpTicks(int nIn, int nOut, int poolSize, RNG &rng) {
  if (nIn <= nOut) throw ScnException("RandomOverlappingFmpTicks: needs nIn > nOut");
  const int alpha = (int)(nIn * 1.0 / nOut);
  std::vector<int> inc;
  inc.resize(nOut * (alpha + 1) - nIn, alpha);
  inc.resize(nOut - 1, alpha + 1);
  rng.vectorShuffle(inc);
  inputL.push_back(0);
  inputR.push_back(poolSize);
  for (int i = 0; i < nOut - 1; i++) {
    inputL.push_back(inputL.back() + inc[i]);
    inputR.push_back(inputL.back() + poolSize);
  }
  if (inputR.back() != nIn) throw ScnException("RandomOverlappingFmpTicks: regions do not end at nIn (poolSize must be floor(nIn/nOut) + 1)");
  fillOutputRanges(nIn, nOut);
}
RandomNonOverlappingFmpTicks::RandomNonOverlappingFmpTicks(int nIn, int nOut, int poolSize, RNG &rng) {
  if (nIn <= nOut) throw ScnException("RandomNonOverlappingFmpTicks: needs nIn > nOut");
  const int alpha = (int)(nIn * 1.0 / nOut);
  if (alpha + 1 > poolSize) throw ScnException("RandomNonOverlappingFmpTicks: poolSize must be at least floor(nIn/nOut) + 1");
  std::vector<int> inc;
  inc.resize(nOut * (alpha + 1) - nIn, alpha);
  inc.resize(nOut, alpha + 1);
  rng.vectorShuffle(inc);
  inputL.push_back(0);
  inputR.push_back(inc[0]);
  for (int i = 0; i < nOut - 1; i++) {
    inputL.push_back(inputL.back() + inc[i]);
    inputR.push_back(inputR.back() + inc[i + 1]);
  }
  if (inputR.back() != nIn) throw ScnException("RandomNonOverlappingFmpTicks: regions do not end at nIn");
  for (int i = 0; i < nOut; i++)
    for (int j = inputL[i]; j < inputR[i]; j++) {
      outputL.push_back(i);
      outputR.push_back(i + 1);
    }
}

RegularTriangularRegions::RegularTriangularRegions(int nIn, int nOut, int dimension, int poolSize, int poolStride)
    : poolSize(poolSize), poolStride(poolStride), nIn(nIn), nOut(nOut), dimension(dimension), s(poolSize), S(0) {
  if (nIn != poolSize + (nOut - 1) * poolStride) throw ScnException("RegularTriangularRegions: nIn != poolSize + (nOut-1)*poolStride");
  ord.assign(ipow(s, dimension), -1);
  for (int c = 0; c < (int)ord.size(); ++c) {
    int digits = 0;
    for (int j = c; j > 0; j /= s) digits += j % s;
    if (digits < s) ord[c] = S++;
  }
}
int RegularTriangularRegions::inputL(int j) { return j * poolStride; }
int RegularTriangularRegions::outputL(int i) { return std::max(0, (i - poolSize + poolStride) / poolStride); }
int RegularTriangularRegions::outputR(int i) { return std::min(i / poolStride + 1, nOut); }

namespace {
struct DevBuf {
  void *p = nullptr;
  explicit DevBuf(size_t bytes) { cudaSafeCall(cudaMalloc(&p, bytes ? bytes : 16)); }
  ~DevBuf() { cudaFree(p); }
  template <class T> T *as() { return (T *)p; }
};

// fmpTables: nullptr for regular regions, else the tick tables of this one sample and R = {square, dim, nIn, nOut, poolSize, .., ..}
void oneSample(const scn_regions_t &R, SparseGrid &in, SparseGrid &out, int &nOutSites, std::vector<int> &rules,
               const std::vector<int> *fmpTables = nullptr, bool fmpOverlapping = true) {
  // rows of the sample need not be contiguous here: renumber, build, map back
  std::vector<int> keys, rowOf;
  for (auto &kv : in.mp) { keys.push_back((int)kv.first); rowOf.push_back(kv.second); }
  int bgLocal = -1;
  if (in.backgroundCol >= 0) { bgLocal = (int)keys.size(); keys.push_back(-1); rowOf.push_back(in.backgroundCol); }
  const int rowsIn = (int)keys.size();
  int sd = fmpTables ? ipow(R.size, R.dim) : scn_regions_cells(&R);
  if (sd < 0) throw ScnException(std::string("gridRules: ") + scn_last_error());
  long long T = 1;
  if (fmpTables) T = sd;
  else if (R.minActive != -1) for (int a = 0; a < R.dim; ++a) T *= (R.size + R.stride - 1) / R.stride;
  const int cap = (int)std::min<long long>((long long)rowsIn * T + 1, 1ll << 30);
  int off[2] = {0, rowsIn};
  size_t wsBytes = fmpTables ? scn_fmp_rules_workspace_bytes(R.dim, R.nIn, R.nOut, R.size, 1, rowsIn) : scn_rules_workspace_bytes(&R, 1, rowsIn);
  DevBuf dTicks(fmpTables ? fmpTables->size() * 4 : 16);
  if (fmpTables) cudaSafeCall(cudaMemcpy(dTicks.p, fmpTables->data(), fmpTables->size() * 4, cudaMemcpyHostToDevice));
  DevBuf dKeys(rowsIn * 4), dOff(8), dBg(4), dOutKeys((size_t)cap * 4), dOutOff(8), dOutBg(4), dRules((size_t)cap * sd * 4), dRes(16), dWs(wsBytes);
  if (rowsIn) cudaSafeCall(cudaMemcpy(dKeys.p, keys.data(), rowsIn * 4, cudaMemcpyHostToDevice));
  cudaSafeCall(cudaMemcpy(dOff.p, off, 8, cudaMemcpyHostToDevice));
  cudaSafeCall(cudaMemcpy(dBg.p, &bgLocal, 4, cudaMemcpyHostToDevice));
  if (fmpTables)
    scnSafeCall(scn_fmp_rules_build(R.dim, R.nIn, R.nOut, R.size, fmpOverlapping ? 1 : 0, 1, dTicks.as<int>(), dKeys.as<int>(), dOff.as<int>(),
                                    dBg.as<int>(), rowsIn, dOutKeys.as<int>(), dOutOff.as<int>(), dOutBg.as<int>(), dRules.as<int>(), cap,
                                    dRes.as<int>(), dWs.p, wsBytes, nullptr));
  else
    scnSafeCall(scn_rules_build(&R, 1, dKeys.as<int>(), dOff.as<int>(), dBg.as<int>(), rowsIn, dOutKeys.as<int>(), dOutOff.as<int>(),
                                dOutBg.as<int>(), dRules.as<int>(), cap, dRes.as<int>(), dWs.p, wsBytes, nullptr));
  int res[4];
  cudaSafeCall(cudaMemcpy(res, dRes.p, 16, cudaMemcpyDeviceToHost)); // default-stream copy waits for the build
  if (res[2]) throw ScnException("gridRules: device error bits " + std::to_string(res[2]));
  const int rowsOut = res[0];
  std::vector<int> outKeys(rowsOut), r(rowsOut * (size_t)sd);
  int outBg = -1;
  if (rowsOut) {
    cudaSafeCall(cudaMemcpy(outKeys.data(), dOutKeys.p, rowsOut * 4, cudaMemcpyDeviceToHost));
    cudaSafeCall(cudaMemcpy(r.data(), dRules.p, r.size() * 4, cudaMemcpyDeviceToHost));
  }
  cudaSafeCall(cudaMemcpy(&outBg, dOutBg.p, 4, cudaMemcpyDeviceToHost));
  for (int v : r) rules.push_back(v >= 0 ? rowOf[v] : v);
  for (int i = 0; i < rowsOut; ++i)
    if (outKeys[i] >= 0) out.mp[outKeys[i]] = nOutSites + i;
  out.backgroundCol = outBg >= 0 ? nOutSites + outBg : -1;
  nOutSites += rowsOut;
}
} // namespace

void fmpGridRulesOneSample(int dimension, int nIn, int nOut, int poolSize, bool overlapping, const std::vector<int> &tables,
                           SparseGrid &inputGrid, SparseGrid &outputGrid, int &nOutputSpatialSites, std::vector<int> &rules) {
  scn_regions_t R = {SCN_LATTICE_SQUARE, dimension, nIn, nOut, poolSize, 1, 1};
  oneSample(R, inputGrid, outputGrid, nOutputSpatialSites, rules, &tables, overlapping);
}

void gridRules(SparseGrid &inputGrid, SparseGrid &outputGrid, RegularSquareRegions &regions, int &nOutputSpatialSites,
               std::vector<int> &rules, bool uniformSizeRegions, int minActiveInputs) {
  if (!uniformSizeRegions) throw ScnException("gridRules: RegularSquareRegions are uniform; pass uniformSizeRegions = true");
  scn_regions_t R = {SCN_LATTICE_SQUARE, regions.dimension, regions.nIn, regions.nOut, regions.poolSize, regions.poolStride, minActiveInputs};
  oneSample(R, inputGrid, outputGrid, nOutputSpatialSites, rules);
}
void gridRules(SparseGrid &inputGrid, SparseGrid &outputGrid, RegularTriangularRegions &regions,
               int &nOutputSpatialSites, std::vector<int> &rules, int minActiveInputs) {
  scn_regions_t R = {SCN_LATTICE_TRIANGULAR, regions.dimension, regions.nIn, regions.nOut, regions.poolSize, regions.poolStride, minActiveInputs};
  oneSample(R, inputGrid, outputGrid, nOutputSpatialSites, rules);
}
