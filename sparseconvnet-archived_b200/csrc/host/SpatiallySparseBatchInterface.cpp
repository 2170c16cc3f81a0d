#include "SpatiallySparseBatchInterface.h"
#include <iostream>

SpatiallySparseBatchSubInterface::SpatiallySparseBatchSubInterface() { reset(); }
void SpatiallySparseBatchSubInterface::reset() {
  features.resize(0);
  dfeatures.resize(0);
  poolingChoices.resize(0);
}

SpatiallySparseBatchInterface::SpatiallySparseBatchInterface(SpatiallySparseBatchSubInterface *s)
    : sub(s), featuresPresent(false, 0), rules(true, 0) {
  nFeatures = 0; spatialSize = 0;
  reset();
}
SpatiallySparseBatchInterface::SpatiallySparseBatchInterface(SpatiallySparseBatchInterface &&o) noexcept
    : sub(o.sub), nFeatures(o.nFeatures), featuresPresent(std::move(o.featuresPresent)), nSpatialSites(o.nSpatialSites),
      spatialSize(o.spatialSize), backpropErrors(o.backpropErrors), grids(std::move(o.grids)), rules(std::move(o.rules)),
      siteKeys(std::move(o.siteKeys)), sampleOffsets(std::move(o.sampleOffsets)), backgroundRows(std::move(o.backgroundRows)),
      maxSitesPerSample(o.maxSitesPerSample), gridOwner(this), deferredFrom(nullptr), deferredCells(0), deferredLearnt(nullptr), deferredLearntInput(nullptr),
      presentSubset(std::move(o.presentSubset)), presentMask(std::move(o.presentMask)), learntOutput(o.learntOutput) {}
void SpatiallySparseBatchInterface::summary() {
  std::cout << "nFeatures " << nFeatures << " featuresPresent " << featuresPresent.size() << " spatialSize " << spatialSize
            << " nSpatialSites " << nSpatialSites << " features " << sub->features.size() << " grids " << grids.size() << std::endl;
}
void SpatiallySparseBatchInterface::reset() {
  featuresPresent.resize(0);
  featuresPresent.copyToCPU();
  nSpatialSites = 0;
  siteKeys.dropBorrowed(); sampleOffsets.dropBorrowed(); backgroundRows.dropBorrowed(); // a device-input call's arrays
  grids.resize(0);
  rules.resize(0);
  backpropErrors = false;
  presentSubset.clear();
  presentMask.resize(0);
  learntOutput = false;
  maxSitesPerSample = 0;
  gridOwner = this;
  deferredFrom = nullptr;
  deferredCells = 0;
  deferredLearnt = nullptr;
  deferredLearntInput = nullptr;
}

// Flatten host grids into keys[row] / offsets / background rows.  Rows of a sample must be
// contiguous, as every Picture::codifyInputData produces them (e.g. OpenCVPicture.cpp:373-375).
void SpatiallySparseBatchInterface::uploadGrids(cudaMemStream &ms) {
  const int batch = (int)grids.size();
  std::vector<int> &keys = siteKeys.hVector();
  std::vector<int> &off = sampleOffsets.hVector();
  std::vector<int> &bg = backgroundRows.hVector();
  keys.assign(nSpatialSites, -2);
  off.assign(batch + 1, 0);
  bg.assign(batch, -1);
  int row = 0;
  maxSitesPerSample = 0;
  for (int b = 0; b < batch; ++b) {
    off[b] = row;
    const SparseGrid &g = grids[b];
    int rows = (int)g.mp.size() + (g.backgroundCol >= 0 ? 1 : 0);
    maxSitesPerSample = std::max(maxSitesPerSample, (int)g.mp.size());
    for (auto &kv : g.mp) {
      if (kv.second < row || kv.second >= row + rows || kv.second >= nSpatialSites) throw ScnException("uploadGrids: a sample's rows are not contiguous");
      keys[kv.second] = (int)kv.first;
    }
    if (g.backgroundCol >= 0) {
      if (g.backgroundCol < row || g.backgroundCol >= row + rows) throw ScnException("uploadGrids: background row outside its sample");
      keys[g.backgroundCol] = -1;
      bg[b] = g.backgroundCol;
    }
    row += rows;
  }
  off[batch] = row;
  if (row != nSpatialSites) throw ScnException("uploadGrids: nSpatialSites does not match the grids");
  siteKeys.copyToGPUAsync(ms);
  sampleOffsets.copyToGPUAsync(ms);
  backgroundRows.copyToGPUAsync(ms);
  gridOwner = this;
}

void SpatiallySparseBatchInterface::materializeGrids(cudaMemStream &ms) {
  SpatiallySparseBatchInterface *o = gridOwner;
  // copies, so the device arrays stay where they are
  std::vector<int> keys(o->siteKeys.size()), off(o->sampleOffsets.size()), bg(o->backgroundRows.size());
  cudaSafeCall(cudaStreamSynchronize(ms.stream));
  if (!keys.empty()) cudaSafeCall(cudaMemcpy(keys.data(), o->siteKeys.dPtr(), keys.size() * sizeof(int), cudaMemcpyDeviceToHost));
  if (!off.empty()) cudaSafeCall(cudaMemcpy(off.data(), o->sampleOffsets.dPtr(), off.size() * sizeof(int), cudaMemcpyDeviceToHost));
  if (!bg.empty()) cudaSafeCall(cudaMemcpy(bg.data(), o->backgroundRows.dPtr(), bg.size() * sizeof(int), cudaMemcpyDeviceToHost));
  const int batch = (int)bg.size();
  grids.assign(batch, SparseGrid());
  for (int b = 0; b < batch; ++b) {
    grids[b].backgroundCol = bg[b];
    for (int r = off[b]; r < off[b + 1]; ++r)
      if (keys[r] >= 0) grids[b].mp[keys[r]] = r;
  }
}
