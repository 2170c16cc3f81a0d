// Max pooling over square/cubic regions (MaxPoolingLayer.h:6-38).
#pragma once
#include "Rng.h"
#include "SpatiallySparseLayer.h"

void maxPool(float *g1, float *g2, int *rules, int count, int sd, int nOut, int *d_choice, cudaMemStream &memStream);
// d1[d_choice[i]] += d2[i] for the count x nOut pooled values (MaxPoolingLayer.cu:74-93): the caller zeroes d1 first.
void maxPoolBackProp(float *d1, float *d2, int count, int nOut, int *d_choice, cudaMemStream &memStream);

class MaxPoolingLayer : public SpatiallySparseLayer {
public:
  int inSpatialSize, outSpatialSize, poolSize, poolStride, dimension, sd;
  bool fusedLast; // the last forward ran inside the kernel of the convolution + learnt layer in front of it
  // With layer timing on: recorded between the learnt layer's kernel and the pooling kernel when this layer
  // ran both (the learnt layer had left its output to it, and the one-kernel form did not take the case).
  cudaEvent_t splitEvent;
  bool splitRecorded;
  MaxPoolingLayer(cudaMemStream &memStream, int poolSize, int poolStride, int dimension);
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

// Fractional max-pooling (MaxPoolingLayer.h:34-143): per sample a fresh set of random region
// bounds (one tick object per axis, drawn on the host from the layer's rng), rules built on the
// device, then the same maxPool kernel.  One base class, four named layers as in the reference.
class FractionalMaxPoolingLayerBase : public SpatiallySparseLayer {
public:
  int inSpatialSize, outSpatialSize, poolSize, dimension, sd;
  float fmpShrink;
  RNG rng;
  vectorCUDA<int> ticks; // this batch's tables, [sample][axis][inputL | inputR | outputL | outputR]
  FractionalMaxPoolingLayerBase(cudaMemStream &memStream, int poolSize, float fmpShrink, int dimension, const char *label, const char *tag);
  void preprocess(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output);
  void forwards(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output);
  void backwards(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output, float learningRate,
                 float momentum);
  int calculateInputSpatialSize(int outputSpatialSize);
  long long enqueueRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                         long long rowsInBound, int *d_result);
  void finishRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                   const int *h_result);

protected:
  virtual bool overlapping() const = 0;
  virtual void appendSampleTables(std::vector<int> &dst) = 0; // one FractionalPoolingRegions<ticks>(..., rng)
  const char *tag;
};
class PseudorandomOverlappingFractionalMaxPoolingLayer : public FractionalMaxPoolingLayerBase {
public:
  PseudorandomOverlappingFractionalMaxPoolingLayer(cudaMemStream &memStream, int poolSize, float fmpShrink, int dimension);
protected:
  bool overlapping() const;
  void appendSampleTables(std::vector<int> &dst);
};
class PseudorandomNonOverlappingFractionalMaxPoolingLayer : public FractionalMaxPoolingLayerBase {
public:
  PseudorandomNonOverlappingFractionalMaxPoolingLayer(cudaMemStream &memStream, int poolSize, float fmpShrink, int dimension);
protected:
  bool overlapping() const;
  void appendSampleTables(std::vector<int> &dst);
};
class RandomOverlappingFractionalMaxPoolingLayer : public FractionalMaxPoolingLayerBase {
public:
  RandomOverlappingFractionalMaxPoolingLayer(cudaMemStream &memStream, int poolSize, float fmpShrink, int dimension);
protected:
  bool overlapping() const;
  void appendSampleTables(std::vector<int> &dst);
};
class RandomNonOverlappingFractionalMaxPoolingLayer : public FractionalMaxPoolingLayerBase {
public:
  RandomNonOverlappingFractionalMaxPoolingLayer(cudaMemStream &memStream, int poolSize, float fmpShrink, int dimension);
protected:
  bool overlapping() const;
  void appendSampleTables(std::vector<int> &dst);
};
