// One batch travelling through the network (SpatiallySparseBatch.h:7-22).
#pragma once
#include <vector>
#include "SpatiallySparseBatchInterface.h"
#include "types.h"

class SpatiallySparseBatch {
  SpatiallySparseBatchSubInterface *inputSub;

public:
  explicit SpatiallySparseBatch(SpatiallySparseBatchSubInterface *inputSub);
  batchType type;
  int batchSize;
  std::vector<int> sampleNumbers;
  std::vector<SpatiallySparseBatchInterface> interfaces; // layers + 1
  vectorCUDA<int> labels;
  std::vector<std::vector<int>> predictions;
  std::vector<std::vector<float>> probabilities;
  // the per-sample vectors of the previous batch, kept by reset() so that the classifier refills them
  // instead of allocating two vectors per sample for every batch
  std::vector<std::vector<int>> sparePredictions;
  std::vector<std::vector<float>> spareProbabilities;
  float negativeLogLikelihood;
  int mistakes;
  void reset();
};
