// The public facade (SparseConvNet.h:20-99): thin forwarding classes over SparseConvNetCUDA
// for square/cubic lattices (SparseConvNet) and triangular/tetrahedral ones
// (SparseConvTriangLeNet), fractional max-pooling builders and the index-learner head included.
#pragma once
#include <memory>
#include <string>
#include "SpatiallySparseDataset.h"
#include "types.h"

class SparseConvNetCUDA;

class SparseConvNet {
public:
  std::unique_ptr<SparseConvNetCUDA> cnn;
  SparseConvNet(int dimension, int nInputFeatures, int nClasses, int pciBusID = -1, int nTop = 1);
  ~SparseConvNet();
  void addLeNetLayerMP(int nFeatures, int filterSize, int filterStride, int poolSize, int poolStride,
                       ActivationFunction activationFn = RELU, float dropout = 0.0f, int minActiveInputs = 1);
  // SparseConvNet.h:32-47
  void addLeNetLayerPOFMP(int nFeatures, int filterSize, int filterStride, int poolSize, float fmpShrink, ActivationFunction activationFn = RELU,
                          float dropout = 0.0f, int minActiveInputs = 1);
  void addLeNetLayerROFMP(int nFeatures, int filterSize, int filterStride, int poolSize, float fmpShrink, ActivationFunction activationFn = RELU,
                          float dropout = 0.0f, int minActiveInputs = 1);
  void addLeNetLayerPDFMP(int nFeatures, int filterSize, int filterStride, int poolSize, float fmpShrink, ActivationFunction activationFn = RELU,
                          float dropout = 0.0f, int minActiveInputs = 1);
  void addLeNetLayerRDFMP(int nFeatures, int filterSize, int filterStride, int poolSize, float fmpShrink, ActivationFunction activationFn = RELU,
                          float dropout = 0.0f, int minActiveInputs = 1);
  void addTerminalPoolingLayer(int poolSize);
  void addSoftmaxLayer();
  void addIndexLearnerLayer();
  float processIndexLearnerDataset(SpatiallySparseDataset &dataset, int batchSize = 100, float learningRate = 0.0, float momentum = 0.99);
  void processDatasetDumpTopLevelFeatures(SpatiallySparseDataset &dataset, int batchSize, int reps = 1);
  void calculateInputRegularizingConstants(SpatiallySparseDataset dataset);
  float processDataset(SpatiallySparseDataset &dataset, int batchSize = 100, float learningRate = 0, float momentum = 0.99);
  void processDatasetRepeatTest(SpatiallySparseDataset &dataset, int batchSize = 100, int nReps = 12,
                                std::string predictionsFilename = "", std::string confusionMatrixFilename = "");
  void loadWeights(std::string baseName, int epoch, bool momentum = false, int firstNlayers = 1000000);
  void saveWeights(std::string baseName, int epoch, bool momentum = false);
};

class SparseConvTriangLeNet {
public:
  std::unique_ptr<SparseConvNetCUDA> cnn; // public here so the harness can reach the runtime
  SparseConvTriangLeNet(int dimension, int nInputFeatures, int nClasses, int pciBusID = -1, int nTop = 1);
  ~SparseConvTriangLeNet();
  void addLeNetLayerMP(int nFeatures, int filterSize, int filterStride, int poolSize, int poolStride,
                       ActivationFunction activationFn = RELU, float dropout = 0.0f, int minActiveInputs = 1);
  void addTerminalPoolingLayer(int poolSize);
  void addSoftmaxLayer();
  void addIndexLearnerLayer();
  float processIndexLearnerDataset(SpatiallySparseDataset &dataset, int batchSize = 100, float learningRate = 0.0, float momentum = 0.99);
  void processDatasetDumpTopLevelFeatures(SpatiallySparseDataset &dataset, int batchSize, int reps = 1);
  void calculateInputRegularizingConstants(SpatiallySparseDataset dataset);
  float processDataset(SpatiallySparseDataset &dataset, int batchSize = 100, float learningRate = 0, float momentum = 0.99);
  void processDatasetRepeatTest(SpatiallySparseDataset &dataset, int batchSize = 100, int nReps = 12,
                                std::string predictionsFilename = "", std::string confusionMatrixFilename = "");
  void loadWeights(std::string baseName, int epoch, bool momentum = false, int firstNlayers = 1000000);
  void saveWeights(std::string baseName, int epoch, bool momentum = false);
};
