// Layer interface (SpatiallySparseLayer.h:6-27).  preprocess() builds the output grids and
// rules (on the device here), forwards() enqueues the layer's kernels on memStream.stream
// and returns without synchronising; backwards() enqueues the layer's share of a training step;
// scaleWeights() is a learnt layer's share of a RESCALEBATCH pass.
#pragma once
#include <fstream>
#include <iostream>
#include "SpatiallySparseBatch.h"
#include "SpatiallySparseBatchInterface.h"

class SpatiallySparseLayer {
public:
  cudaMemStream &memStream;
  virtual void preprocess(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                          SpatiallySparseBatchInterface &output) = 0;
  virtual void forwards(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                        SpatiallySparseBatchInterface &output) = 0;
  virtual void scaleWeights(SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                            float &scalingUnderneath, bool topLayer);
  virtual void backwards(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                         SpatiallySparseBatchInterface &output, float learningRate, float momentum);
  explicit SpatiallySparseLayer(cudaMemStream &memStream);
  virtual ~SpatiallySparseLayer();
  virtual void loadWeightsFromStream(std::ifstream &f, bool momentum);
  virtual void putWeightsToStream(std::ofstream &f, bool momentum);
  virtual int calculateInputSpatialSize(int outputSpatialSize) = 0;

  // ---- additions used by the batched rule chain (no reference counterpart)
  // Enqueue the geometry part of preprocess() without reading any count back: the output
  // interface's device grid arrays are sized for `rowsInBound`-derived upper bounds and the
  // layer's 4-int result record is written to d_result.  Returns the upper bound on output
  // rows.  Layers that do not change geometry return rowsInBound and enqueue nothing.
  virtual long long enqueueRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                                 SpatiallySparseBatchInterface &output, long long rowsInBound, int *d_result);
  // Finish preprocess() once the counts are known on the host.
  virtual void finishRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                           SpatiallySparseBatchInterface &output, const int *h_result);
  bool changesGeometry;
};
