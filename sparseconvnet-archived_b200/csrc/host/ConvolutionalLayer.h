// ConvolutionalLayer (ConvolutionalLayer.h): on its own it only GATHERS the rows named by
// the rules into [rows x (fs*nIn)]; the arithmetic is the NetworkInNetworkLayer behind it.
// With fuseWithNext (set by SparseConvNetCUDA::addConvolutionalLayer) forwards() leaves the
// gather to that layer's fused kernel and the gathered matrix never exists.
#pragma once
#include "SpatiallySparseLayer.h"

class ConvolutionalLayer : public SpatiallySparseLayer {
private:
  int fs;

public:
  int inSpatialSize, outSpatialSize, filterSize, filterStride, dimension, nFeaturesIn, nFeaturesOut, minActiveInputs;
  bool fuseWithNext;
  ConvolutionalLayer(cudaMemStream &memStream, int filterSize, int filterStride, int dimension, int nFeaturesIn,
                     int minActiveInputs = 1); // -1: 'valid' mode
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

void propForwardToMatrixMultiply(float *inFeatures, float *outFeatures, int *rules, int count, int nIn, cudaMemStream &memStream);
// inDFeatures[rules[c]] += outDFeatures[c] for the count rule cells with a rule >= 0 (ConvolutionalLayer.cu:42-72): the
// caller zeroes inDFeatures first.
void propBackwardFromMatrixMultiply(float *inDFeatures, float *outDFeatures, int *rules, int count, int nIn, cudaMemStream &memStream);
