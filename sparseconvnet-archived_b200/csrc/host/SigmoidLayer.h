// applySigmoid / applySigmoidBackProp (SigmoidLayer.h:4-9): the stand-alone activation passes, and the layer that is
// nothing but one (SigmoidLayer.h:11-26).  The learnt layers fuse the activation into their kernels; these entry points
// exist for callers that apply one themselves.
#pragma once
#include "SpatiallySparseBatchInterface.h"
#include "SpatiallySparseLayer.h"
#include "types.h"
void applySigmoid(SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output, ActivationFunction fn,
                  cudaMemStream &memStream);
// input.dfeatures = output.dfeatures x the activation's derivative, read off the output's features (in place where the
// two interfaces share their sub-interface, as the learnt layers use it).
void applySigmoidBackProp(SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output, ActivationFunction fn,
                          cudaMemStream &memStream);

class SigmoidLayer : public SpatiallySparseLayer {
public:
  ActivationFunction fn;
  SigmoidLayer(cudaMemStream &memStream, ActivationFunction fn);
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
