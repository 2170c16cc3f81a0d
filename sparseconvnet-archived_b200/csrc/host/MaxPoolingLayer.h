// Max pooling over square/cubic regions (MaxPoolingLayer.h:6-38).
#pragma once
#include "SpatiallySparseLayer.h"

void maxPool(float *g1, float *g2, int *rules, int count, int sd, int nOut, int *d_choice, cudaMemStream &memStream);

class MaxPoolingLayer : public SpatiallySparseLayer {
public:
  int inSpatialSize, outSpatialSize, poolSize, poolStride, dimension, sd;
  MaxPoolingLayer(cudaMemStream &memStream, int poolSize, int poolStride, int dimension);
  void preprocess(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output);
  void forwards(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output);
  int calculateInputSpatialSize(int outputSpatialSize);
  long long enqueueRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                         long long rowsInBound, int *d_result);
  void finishRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                   const int *h_result);
};
