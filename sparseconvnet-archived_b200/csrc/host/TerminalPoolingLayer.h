// Average over everything that reaches the last grid (TerminalPoolingLayer.h).
#pragma once
#include "SpatiallySparseLayer.h"

class TerminalPoolingLayer : public SpatiallySparseLayer {
public:
  int inSpatialSize;  // == poolSize
  int outSpatialSize; // 1
  int poolSize;
  int S;         // constructor argument (the reference stores it and never reads it again)
  int dimension; // needed by the device grid index; set by SparseConvNetCUDA (default 2)
  TerminalPoolingLayer(cudaMemStream &memStream, int poolSize, int S);
  void preprocess(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output);
  void forwards(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output);
  void backwards(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output, float learningRate,
                 float momentum);
  int calculateInputSpatialSize(int outputSpatialSize);
  long long enqueueRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                         long long rowsInBound, int *d_result);
  void finishRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                   const int *h_result);

private:
  int widthBuilt; // rule columns of the build enqueued by enqueueRules
};
