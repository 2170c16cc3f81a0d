// The network runtime (SparseConvNetCUDA.h:25-114): the layer list, the builder methods with
// the reference's rounding rules, the per-batch forward, dataset loops and weight files.
#pragma once
#include <fstream>
#include <iostream>
#include <mutex>
#include <string>
#include <vector>
#include "SpatiallySparseBatch.h"
#include "SpatiallySparseDataset.h"
#include "SpatiallySparseLayer.h"
#define N_MAX_BATCH_PRODUCER_THREADS 20

class SparseConvNetCUDA {
public:
  // The first convolution + NiN pair is launched right behind the rule chain, before the row counts are
  // read back (its kernel takes its count from device memory), so the GPU works while the host waits.
  bool fuseClassifier;      // forwardLayers() runs a learnt layer that splits K and the small learnt layer behind it (N <= 16) as one call
  bool fusePooling;         // builders mark learnt layers that a non-overlapping max pooling follows (see NetworkInNetworkLayer::fusePoolNext)
  bool earlyFirstLayer;
  int earlyLayers;          // layers of the current batch already launched by preprocessBatchOnDevice (0 or 2)
  cudaStream_t countStream; // the row counts are read back on this stream, so that the early first layer does not delay them
  cudaEvent_t chainDone;
  cudaEvent_t inputReady;   // if set: the input features are complete once this event has happened (waited for once, then cleared)
  std::vector<SpatiallySparseLayer *> layers; // owned
  std::vector<float> inputNormalizingConstants;
  int dimension, nClasses, nTop, inputSpatialSize, nInputFeatures, nOutputFeatures, deviceID, nBatchProducerThreads;
  cudaMemStream memStream;
  std::vector<SpatiallySparseBatch> batchPool;
  std::vector<SpatiallySparseBatchSubInterface *> initialSubInterfaces;
  std::vector<SpatiallySparseBatchSubInterface *> sharedSubInterfaces;
  cublasHandle_t cublasHandle; // unused, kept for the layer constructors' signatures

  SparseConvNetCUDA(int dimension, int nInputFeatures, int nClasses, int pciBusID = -1, int nTop = 1, int nBatchProducerThreads = 10);
  // Same, enqueueing on a stream the caller owns (no reference counterpart).
  SparseConvNetCUDA(int dimension, int nInputFeatures, int nClasses, cudaStream_t stream, int nTop, int nBatchProducerThreads);
  ~SparseConvNetCUDA();
  void processBatch(SpatiallySparseBatch &batch, float learningRate, float momentum, std::ofstream &f, std::ofstream &g);
  void addLearntLayer(int nFeatures, ActivationFunction activationFn = RELU, float dropout = 0.0f, float alpha = 1.0f);
  void addNetworkInNetworkLayer(int nFeatures, ActivationFunction activationFn = RELU, float dropout = 0.0f);
  void addConvolutionalLayer(int nFeatures, int filterSize, int filterStride, ActivationFunction activationFn = RELU, float dropout = 0.0f,
                             int minActiveInputs = 1, float poolingToFollow = 1.0f);
  void addLeNetLayerMP(int nFeatures, int filterSize, int filterStride, int poolSize, int poolStride, ActivationFunction activationFn = RELU,
                       float dropout = 0.0f, int minActiveInputs = 1);
  // SparseConvNetCUDA.h:67-82: convolution block followed by one of the four fractional max-pooling layers
  void addLeNetLayerROFMP(int nFeatures, int filterSize, int filterStride, int poolSize, float fmpShrink, ActivationFunction activationFn = RELU,
                          float dropout = 0.0f, int minActiveInputs = 1);
  void addLeNetLayerPOFMP(int nFeatures, int filterSize, int filterStride, int poolSize, float fmpShrink, ActivationFunction activationFn = RELU,
                          float dropout = 0.0f, int minActiveInputs = 1);
  void addLeNetLayerRDFMP(int nFeatures, int filterSize, int filterStride, int poolSize, float fmpShrink, ActivationFunction activationFn = RELU,
                          float dropout = 0.0f, int minActiveInputs = 1);
  void addLeNetLayerPDFMP(int nFeatures, int filterSize, int filterStride, int poolSize, float fmpShrink, ActivationFunction activationFn = RELU,
                          float dropout = 0.0f, int minActiveInputs = 1);
  void addTriangularConvolutionalLayer(int nFeatures, int filterSize, int filterStride, ActivationFunction activationFn = RELU,
                                       float dropout = 0.0f, int minActiveInputs = 1, float poolingToFollow = 1.0f);
  void addTriangularLeNetLayerMP(int nFeatures, int filterSize, int filterStride, int poolSize, int poolStride,
                                 ActivationFunction activationFn = RELU, float dropout = 0.0f, int minActiveInputs = 1);
  void addSoftmaxLayer();
  void addIndexLearnerLayer();
  void processBatchDumpTopLevelFeaturess(SpatiallySparseBatch &batch, std::ofstream &f);
  void processDatasetDumpTopLevelFeatures(SpatiallySparseDataset &dataset, int batchSize, int reps = 1);
  void calculateInputRegularizingConstants(SpatiallySparseDataset dataset);
  void processIndexLearnerBatch(SpatiallySparseBatch &batch, float learningRate, float momentum, std::ofstream &f);
  float processIndexLearnerDataset(SpatiallySparseDataset &dataset, int batchSize = 100, float learningRate = 0.0, float momentum = 0.99);
  void addTerminalPoolingLayer(int poolSize, int S);
  float processDataset(SpatiallySparseDataset &dataset, int batchSize = 100, float learningRate = 0, float momentum = 0.99);
  void processDatasetRepeatTest(SpatiallySparseDataset &dataset, int batchSize = 100, int nReps = 12,
                                std::string predictionsFilename = "", std::string confusionMatrixFilename = "");
  void loadWeights(std::string baseName, int epoch, bool momentum, int firstNlayers = 1000000);
  void saveWeights(std::string baseName, int epoch, bool momentum);

  // ---- additions (no reference counterpart)
  // Run every layer's rule construction on the device for a batch whose interface 0 holds
  // the input grids in device form, with a single read-back of all per-layer counts.
  void preprocessBatchOnDevice(SpatiallySparseBatch &batch);
  // Grow batch.interfaces to layers.size()+1.
  void prepareBatch(SpatiallySparseBatch &batch);
  // Forward of all layers without the classifier read-back.
  void forwardLayers(SpatiallySparseBatch &batch, size_t count = (size_t)-1); // the first `count` layers
  // CUDA-event timing per layer (off by default).  layerTimes() waits for the stream and
  // returns layers.size()+1 values in ms: each layer's forwards(), then the rule chain.
  void enableTiming(bool on);
  std::vector<float> layerTimes();
  // Set before preprocessBatchOnDevice when interface 0's backgroundRows have not been filled in: the rule chain's
  // kernel finds them on its way (a kernel of their own where the fused chain does not apply).
  bool inputBackgroundPending;

private:
  void init(int nInputFeatures, int nClasses);
  vectorCUDA<int> chainResults; // two sets of 4 ints per layer, used by alternate batches
  bool timing;
  int chainRowsHint; // rows per sample seen so far (+25 %): sizes the fused rule chain's shared memory
  int chainPhase;    // which of the two sets of rule-chain result records the next batch uses
  std::vector<cudaEvent_t> events; // layers.size()+1 layer boundaries, then rule chain begin/end
};
