#include "SpatiallySparseLayer.h"

SpatiallySparseLayer::SpatiallySparseLayer(cudaMemStream &memStream) : memStream(memStream), changesGeometry(false) {}
SpatiallySparseLayer::~SpatiallySparseLayer() {}
void SpatiallySparseLayer::scaleWeights(SpatiallySparseBatchInterface &, SpatiallySparseBatchInterface &, float &, bool) {} // SpatiallySparseLayer.cu:3-6
void SpatiallySparseLayer::backwards(SpatiallySparseBatch &, SpatiallySparseBatchInterface &, SpatiallySparseBatchInterface &, float, float) {
  throw ScnException("backwards: this layer type has no backward pass");
}
void SpatiallySparseLayer::loadWeightsFromStream(std::ifstream &, bool) {}
void SpatiallySparseLayer::putWeightsToStream(std::ofstream &, bool) {}
long long SpatiallySparseLayer::enqueueRules(SpatiallySparseBatch &, SpatiallySparseBatchInterface &, SpatiallySparseBatchInterface &,
                                             long long rowsInBound, int *) { return rowsInBound; }
void SpatiallySparseLayer::finishRules(SpatiallySparseBatch &, SpatiallySparseBatchInterface &, SpatiallySparseBatchInterface &, const int *) {}
