// Index learning (IndexLearnerLayer.h): the top layer of an unsupervised run in which every picture of the training set is
// its own class.  W is [nFeaturesIn x nFeaturesOut] with nFeaturesOut = the size of the training set, starts at zero and
// has no bias; a training batch of n pictures uses only the n columns its own pictures index (indexLearnerIndices), so
// the layer's output is n x n: row i holds the softmax over the batch's pictures, and picture i's target is column i.
#pragma once
#include <fstream>
#include <vector>
#include "SpatiallySparseLayer.h"
#include "utilities.h"
#include "vectorCUDA.h"

class IndexLearnerLayer : public SpatiallySparseLayer {
public:
  vectorCUDA<float> W;                  // [nFeaturesIn x nFeaturesOut]
  std::vector<int> indexLearnerIndices; // the columns of the batch in flight (its pictures' numbers in the data set)
  int nFeaturesIn;
  int nFeaturesOut;
  IndexLearnerLayer(cudaMemStream &memStream, cublasHandle_t &cublasHandle, int nFeaturesIn, int nFeaturesOut);
  void preprocess(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output);
  void forwards(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output);
  void backwards(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output, float learningRate,
                 float momentum);
  void loadWeightsFromStream(std::ifstream &f, bool momentum);
  void putWeightsToStream(std::ofstream &f, bool momentum);
  int calculateInputSpatialSize(int outputSpatialSize);
  long long enqueueRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                         long long rowsInBound, int *d_result);
  void finishRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                   const int *h_result);

private:
  vectorCUDA<int> indices;              // indexLearnerIndices on the device
  vectorCUDA<float> w, wt, dw, db, zeroBias; // the batch's columns of W, their transpose, the gradient, scratch
};

// Scores the n x n output of an IndexLearnerLayer (IndexLearnerLayer.cu:103-142): probabilities, top-n predictions,
// negative log-likelihood and mistakes with picture i's own column as its class, then the gradient of the cost with
// respect to the softmax input, which starts the backward pass.
void IndexLearner(SpatiallySparseBatchInterface &input, SpatiallySparseBatch &batch, int nTop, cudaMemStream &memStream);
