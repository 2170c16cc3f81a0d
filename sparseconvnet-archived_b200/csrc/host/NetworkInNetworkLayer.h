// 1x1 convolution: out = act(p * X W + p * B) at test time (NetworkInNetworkLayer.h:6-45); in a training batch
// with dropout, out = act(X W + B) on the features the batch keeps and zero on the others.
// Behind a fused ConvolutionalLayer it is the whole convolution: one kernel gathers the rows
// named by the rules, contracts them with W and applies bias, dropout scaling and activation.
#pragma once
#include <fstream>
#include <mutex>
#include "Rng.h"
#include "SpatiallySparseLayer.h"

class NetworkInNetworkLayer : public SpatiallySparseLayer {
public:
  vectorCUDA<float> W;  // [nFeaturesIn x nFeaturesOut], row-major
  vectorCUDA<float> MW; // momentum of the SGD update (zero until the first training step)
  vectorCUDA<float> B;  // [nFeaturesOut]
  vectorCUDA<float> MB;
  vectorCUDA<float> splitScratch; // partial sums when the kernel splits K (layers with few rows)
  vectorCUDA<float> dw, db;       // gradients of the last training step
  vectorCUDA<float> Wt, zeroBias, dGathered; // backward pass: transposed weights, a zero bias for them, the gathered matrix's gradient
  ActivationFunction fn;
  int nFeaturesIn, nFeaturesOut;
  float dropout;
  int precision; // scn_precision used by forwards(); SCN_PREC_AUTO by default
  bool fusePoolNext; // set by the builders when a non-overlapping max-pooling layer follows: forwards() then leaves the
                     // output unmaterialised and the pooling layer runs gather + this layer + pooling as one kernel
  RNG rng; // draws the features each training batch keeps (NetworkInNetworkLayer.h:8)
  std::mutex rngMutex; // BatchProducer threads preprocess different batches through the same layer object
  // The features the next training batches keep instead of a random draw (ascending indices below nFeaturesOut), so that a
  // run can be repeated with the subsets another run drew; an empty vector returns to random draws.
  std::vector<int> forcedPresent;
  bool precisionFallback; // true: a tensor-core precision falls back to the CUDA-core kernel where the shape has no tensor-core path (false: throw)
  NetworkInNetworkLayer(cudaMemStream &memStream, cublasHandle_t &cublasHandle, int nFeaturesIn, int nFeaturesOut,
                        float dropout = 0, ActivationFunction fn = NOSIGMOID, float alpha = 1);
  ~NetworkInNetworkLayer();
  void preprocess(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output);
  void forwards(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output);
  void scaleWeights(SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output, float &scalingUnderneath, bool topLayer) override;
  void backwards(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output, float learningRate,
                 float momentum);
  void loadWeightsFromStream(std::ifstream &f, bool momentum);
  void putWeightsToStream(std::ofstream &f, bool momentum);
  int calculateInputSpatialSize(int outputSpatialSize);
  long long enqueueRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                         long long rowsInBound, int *d_result);
  void finishRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                   const int *h_result);
  // Call after writing W directly (e.g. W.hVector()[i] = ...): drops the packed copy the
  // tensor-core kernel reads.
  void weightsChanged();
  // forwards() of a fused convolution + this layer before the host knows the row count: rowsBound is an
  // upper bound (rules and output are sized for it), the kernel reads the count from d_rows.  Returns
  // false (nothing launched) unless the 3xTF32 tensor-core kernel takes the shape without a K split.
  bool forwardsEarly(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &source, SpatiallySparseBatchInterface &input,
                     SpatiallySparseBatchInterface &output, int cells, long long rowsBound, const int *d_rows);
  // Convolution + this layer + the max pooling behind it in one kernel: the pooled features and choices go to
  // poolOutput, this layer's own output is never written.  d_rowsPool: device-side pooled row count (then
  // rowsPoolBound is an upper bound) or nullptr.  False (nothing launched) if the kernel does not take the case.
  // This layer and the small learnt layer behind it (the classifier) in one call, where this layer splits K (few
  // rows): the kernel that adds the partial sums applies `next` as well.  Both outputs are written.  false: not
  // taken, run the two layers.
  bool forwardsWithNext(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                        NetworkInNetworkLayer &next, SpatiallySparseBatchInterface &nextOutput);
  bool forwardsPooled(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &source, SpatiallySparseBatchInterface &input,
                      SpatiallySparseBatchInterface &poolOutput, int convCells, int poolCells, long long rowsPoolBound, const int *d_rowsPool,
                      int rowsUnpooled = 0);
  // forwards() without the deferral to a pooling layer.
  void forwardsNow(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output);
  void countMultiplyAdds(SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output);
  // The bookkeeping forwards() would have done, once the counts are known.
  void finishEarly(SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output);

protected:
  virtual float *slopes(); // per-channel PReLU slopes, or nullptr
  virtual float *slopeGradient();                               // where backwards() leaves the slopes' gradient, or nullptr
  virtual void updateSlopes(float learningRate, float momentum, const float *presentMask); // SGD step on the slopes (PReLU layers); presentMask: 0/1 per output feature or nullptr
  void *packedT;           // Wt repacked for the tensor-core kernel (input gradient)
  size_t packedTBytes;
  void *packed;            // W repacked for `packedPrecision`
  size_t packedBytes;
  int packedPrecision;
  int packedFs;
  const void *packedWeights(int fs, int nIn, int prec);
};
void replicateArray(float *src, float *dst, int nRows, int nColumns, cudaMemStream &memStream);
