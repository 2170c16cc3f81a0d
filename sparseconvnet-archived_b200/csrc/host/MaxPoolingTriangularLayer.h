// Max pooling on a triangular/tetrahedral lattice (MaxPoolingTriangularLayer.h).
#pragma once
#include "SpatiallySparseLayer.h"

class MaxPoolingTriangularLayer : public SpatiallySparseLayer {
public:
  int inSpatialSize, outSpatialSize, poolSize, poolStride, dimension, S;
  MaxPoolingTriangularLayer(cudaMemStream &memStream, int poolSize, int poolStride, int dimension);
  void preprocess(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output);
  void forwards(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output);
  void backwards(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output, float learningRate,
                 float momentum);
  int calculateInputSpatialSize(int outputSpatialSize);
  long long enqueueRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                         long long rowsInBound, int *d_result);
  void finishRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                   const int *h_result);
};
