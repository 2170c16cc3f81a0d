// Convolution on a triangular/tetrahedral lattice (ConvolutionalTriangularLayer.h).
#pragma once
#include "SpatiallySparseLayer.h"

class ConvolutionalTriangularLayer : public SpatiallySparseLayer {
private:
  int fs;

public:
  int inSpatialSize, outSpatialSize, filterSize, filterStride, dimension, nFeaturesIn, nFeaturesOut, minActiveInputs;
  bool fuseWithNext;
  ConvolutionalTriangularLayer(cudaMemStream &memStream, int filterSize, int filterStride, int dimension, int nFeaturesIn,
                               int minActiveInputs = 1);
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
