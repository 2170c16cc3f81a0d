#include "SpatiallySparseBatch.h"

SpatiallySparseBatch::SpatiallySparseBatch(SpatiallySparseBatchSubInterface *inputSub) : inputSub(inputSub) {
  interfaces.emplace_back(inputSub);
  type = TESTBATCH;
  reset();
}
void SpatiallySparseBatch::reset() {
  batchSize = 0;
  sampleNumbers.clear();
  for (auto &i : interfaces) i.reset();
  interfaces[0].sub->reset();
  labels.resize(0);
  predictions.clear();
  probabilities.clear();
  negativeLogLikelihood = 0;
  mistakes = 0;
}
