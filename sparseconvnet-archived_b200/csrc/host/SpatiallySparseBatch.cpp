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
  for (auto &v : predictions) sparePredictions.emplace_back(std::move(v));
  for (auto &v : probabilities) spareProbabilities.emplace_back(std::move(v));
  predictions.clear();
  probabilities.clear();
  negativeLogLikelihood = 0;
  mistakes = 0;
}
