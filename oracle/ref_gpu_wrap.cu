// TEST INFRASTRUCTURE ONLY (part of the parity oracle; never linked into the product, never timed).
//
// C wrapper around the REFERENCE's own network classes and CUDA kernels, compiled for the GPU from
// the reference sources where they lie (oracle/Makefile, target _ref_gpu).  Nothing here restates an
// algorithm: it feeds pictures through the reference's `BatchProducer` (BatchProducer.cu:40-87,
// 108-142: every layer's `preprocess`, i.e. the reference's host rule construction with its
// vectorHash grid backend, then the uploads) and `SparseConvNetCUDA::processBatch`
// (SparseConvNetCUDA.cu:227-271: every layer's `forwards`, `SoftmaxClassifier`, and for TRAINBATCH
// every layer's `backwards`), and copies out what the batch interfaces hold afterwards
// (SpatiallySparseBatchInterface.h:8-46): features, dfeatures, poolingChoices, rules, grids,
// probabilities, predictions, negative log-likelihood, mistakes.  The GPU tests use it to pin the
// floating-point half of oracle/scn_oracle.cpp (gather, cuBLAS SGEMM + bias + activation, PReLU, max
// pooling with choices, terminal pooling, softmax) and the builder arithmetic to the reference.
//
// The reference's gather kernel reads in front of the feature buffer for a rule of -1
// (ConvolutionalLayer.cu:20-26) and its pooling kernel stores unset registers for a row without any
// non-negative rule (MaxPoolingLayer.cu:18-32).  Regular (non-fractional) layers over pictures that
// carry a background row never produce such rules; callers check that on the oracle's rulebooks
// before they run a forward here.
#include <cstdint>
#include <cstring>
#include <iostream>
#include <memory>
#include <sstream>
#include <string>
#include <vector>
#include <fstream>
#include "SpatiallySparseLayer.h"
#include "Rng.h"
// The learnt layers keep the generator that draws their dropout subsets private and seed it from the clock
// (NetworkInNetworkLayer.h:7-8, Rng.cpp:7-15).  This translation unit alone reads their two headers with the member
// reachable, so that refgpu_seed_dropout can make a dropout test repeat; the reference's own files are compiled as they are.
#define private public
#include "NetworkInNetworkLayer.h"
#include "NetworkInNetworkPReLULayer.h"
#include "IndexLearnerLayer.h" // (its weights are private too: read back by refgpu_layer_weights)
#undef private
#include "BatchProducer.h"
#include "ConvolutionalLayer.h"
#include "ConvolutionalTriangularLayer.h"
#include "MaxPoolingLayer.h"
#include "MaxPoolingTriangularLayer.h"
#include "TerminalPoolingLayer.h"
#include "NetworkArchitectures.h"
#include "NetworkInNetworkLayer.h"
#include "NetworkInNetworkPReLULayer.h"
#include "SparseConvNetCUDA.h"
#include "SpatiallySparseDataset.h"

namespace {
struct Quiet { // the reference prints banners and copy notices to std::cout
  std::streambuf *old;
  std::ostringstream sink;
  Quiet() : old(std::cout.rdbuf(sink.rdbuf())) {}
  ~Quiet() { std::cout.rdbuf(old); }
};

// The input contract of Picture::codifyInputData as the reference's pictures implement it
// (OpenCVPicture.cpp:368-401): a zero background row first, whose id becomes grid.backgroundCol, then
// one feature row per active site, grid.mp[key] = row id.
class FlatPicture : public Picture {
public:
  std::vector<int64_t> keys;
  std::vector<float> feats;
  int nFeatures;
  bool bg;
  FlatPicture(int nFeatures, int label, bool bg) : Picture(label), nFeatures(nFeatures), bg(bg) {}
  void codifyInputData(SparseGrid &grid, std::vector<float> &features, int &nSpatialSites, int) override {
    if (bg) {
      for (int i = 0; i < nFeatures; ++i) features.push_back(0);
      grid.backgroundCol = nSpatialSites++;
    }
    for (size_t s = 0; s < keys.size(); ++s) {
      grid.mp[keys[s]] = nSpatialSites++;
      features.insert(features.end(), feats.begin() + s * nFeatures, feats.begin() + (s + 1) * nFeatures);
    }
  }
};

struct Handle {
  std::unique_ptr<SparseConvNetCUDA> cnn;
  int lattice;
  std::vector<std::unique_ptr<FlatPicture>> pics;
  SpatiallySparseDataset ds;
  std::unique_ptr<BatchProducer> bp;
  SpatiallySparseBatch *batch = nullptr;
};

template <class T> void fetch(vectorCUDA<T> &v, T *dst) {
  const size_t n = v.size();
  if (!n || !dst) return;
  if (v.onGPU) cudaMemcpy(dst, v.dPtr(), sizeof(T) * n, cudaMemcpyDeviceToHost);
  else std::memcpy(dst, v.hVector().data(), sizeof(T) * n);
}
} // namespace

namespace {
template <class F> bool describeFmp(SpatiallySparseLayer *L, int *v) {
  if (auto f = dynamic_cast<F *>(L)) {
    int sd = 1; // poolSize^dimension, the width of a rule row
    for (int i = 0; i < f->dimension; ++i) sd *= f->poolSize;
    int w[10] = {6, f->poolSize, 1, 1, 0, 0, sd, 0, f->inSpatialSize, f->outSpatialSize};
    std::memcpy(v, w, sizeof(w));
    return true;
  }
  return false;
}
} // namespace

extern "C" {

void *refgpu_create(int dimension, int nInputFeatures, int nClasses, int nTop, int lattice) {
  Quiet q;
  Handle *h = new Handle();
  h->lattice = lattice;
  h->cnn.reset(new SparseConvNetCUDA(dimension, nInputFeatures, nClasses, -1, nTop, 1)); // one producer thread
  return h;
}
void refgpu_destroy(void *p) {
  Quiet q;
  Handle *h = (Handle *)p;
  h->bp.reset();
  delete h;
}
// SparseConvNetCUDA::addLeNetLayerMP (SparseConvNetCUDA.cu:98-111) or, on the triangular lattice,
// addTriangularLeNetLayerMP (:179-192), called as SparseConvNet / SparseConvTriangLeNet forward them.
void refgpu_addLeNetLayerMP(void *p, int nFeatures, int fs, int fstride, int ps, int pstride, int act, float dropout, int minActive) {
  Quiet q;
  Handle *h = (Handle *)p;
  if (h->lattice == 0) h->cnn->addLeNetLayerMP(nFeatures, fs, fstride, ps, pstride, (ActivationFunction)act, dropout, minActive);
  else h->cnn->addTriangularLeNetLayerMP(nFeatures, fs, fstride, ps, pstride, (ActivationFunction)act, dropout, minActive);
}
void refgpu_addTerminalPoolingLayer(void *p, int poolSize, int S) {
  Quiet q;
  ((Handle *)p)->cnn->addTerminalPoolingLayer(poolSize, S);
}
void refgpu_addSoftmaxLayer(void *p) {
  Quiet q;
  ((Handle *)p)->cnn->addSoftmaxLayer();
}
// One of the reference's named architectures (NetworkArchitectures.cpp): the class is constructed as a
// caller of the reference would, then its runtime (`cnn`, a public member, SparseConvNet.h:20-23) is
// taken over by the handle.  Names: DeepCNet DeepC2 DeepCNiN DeepC2C2 DeepC3C3Valid DeepC3C3
// POFMPSparseConvNet ROFMPSparseConvNet PDFMPSparseConvNet RDFMPSparseConvNet; fmpShrink is read by
// the last four only.  Returns NULL for an unknown name.
void *refgpu_named(const char *name, int dimension, int l, int k, float fmpShrink, int fn, int nInputFeatures, int nClasses, float p, int nTop) {
  Quiet q;
  const std::string n(name);
  const ActivationFunction a = (ActivationFunction)fn;
  std::unique_ptr<SparseConvNet> net;
  if (n == "DeepCNet") net.reset(new DeepCNet(dimension, l, k, a, nInputFeatures, nClasses, p, -1, nTop));
  else if (n == "DeepC2") net.reset(new DeepC2(dimension, l, k, a, nInputFeatures, nClasses, p, -1, nTop));
  else if (n == "DeepCNiN") net.reset(new DeepCNiN(dimension, l, k, a, nInputFeatures, nClasses, p, -1, nTop));
  else if (n == "DeepC2C2") net.reset(new DeepC2C2(dimension, l, k, a, nInputFeatures, nClasses, p, -1, nTop));
  else if (n == "DeepC3C3Valid") net.reset(new DeepC3C3Valid(dimension, l, k, a, nInputFeatures, nClasses, p, -1, nTop));
  else if (n == "DeepC3C3") net.reset(new DeepC3C3(dimension, l, k, a, nInputFeatures, nClasses, p, -1, nTop));
  else if (n == "POFMPSparseConvNet") net.reset(new POFMPSparseConvNet(dimension, l, k, fmpShrink, a, nInputFeatures, nClasses, p, -1, nTop));
  else if (n == "ROFMPSparseConvNet") net.reset(new ROFMPSparseConvNet(dimension, l, k, fmpShrink, a, nInputFeatures, nClasses, p, -1, nTop));
  else if (n == "PDFMPSparseConvNet") net.reset(new PDFMPSparseConvNet(dimension, l, k, fmpShrink, a, nInputFeatures, nClasses, p, -1, nTop));
  else if (n == "RDFMPSparseConvNet") net.reset(new RDFMPSparseConvNet(dimension, l, k, fmpShrink, a, nInputFeatures, nClasses, p, -1, nTop));
  else return nullptr;
  Handle *h = new Handle();
  h->lattice = 0;
  h->cnn = std::move(net->cnn);
  h->cnn->nBatchProducerThreads = 1; // samples reach the fractional pooling layers' generators in batch order
  return h;
}
// Seed the generator of fractional max-pooling layer l (MaxPoolingLayer.h:44,72,99,126: a public RNG
// member per layer) with seed + l, so that a test can give two implementations the same stream.
void refgpu_seed_fmp(void *p, unsigned seed) {
  Handle *h = (Handle *)p;
  for (size_t l = 0; l < h->cnn->layers.size(); ++l) {
    SpatiallySparseLayer *L = h->cnn->layers[l];
    if (auto f = dynamic_cast<PseudorandomOverlappingFractionalMaxPoolingLayer *>(L)) f->rng.gen.seed(seed + (unsigned)l);
    else if (auto f = dynamic_cast<PseudorandomNonOverlappingFractionalMaxPoolingLayer *>(L)) f->rng.gen.seed(seed + (unsigned)l);
    else if (auto f = dynamic_cast<RandomOverlappingFractionalMaxPoolingLayer *>(L)) f->rng.gen.seed(seed + (unsigned)l);
    else if (auto f = dynamic_cast<RandomNonOverlappingFractionalMaxPoolingLayer *>(L)) f->rng.gen.seed(seed + (unsigned)l);
  }
}
// The same for the generators the learnt layers draw their dropout subsets from.
void refgpu_seed_dropout(void *p, unsigned seed) {
  Handle *h = (Handle *)p;
  for (size_t l = 0; l < h->cnn->layers.size(); ++l) {
    SpatiallySparseLayer *L = h->cnn->layers[l];
    if (auto f = dynamic_cast<NetworkInNetworkLayer *>(L)) f->rng.gen.seed(seed + (unsigned)l);
    else if (auto f = dynamic_cast<NetworkInNetworkPReLULayer *>(L)) f->rng.gen.seed(seed + (unsigned)l);
  }
}
int refgpu_n_layers(void *p) { return (int)((Handle *)p)->cnn->layers.size(); }
int refgpu_input_spatial_size(void *p) { return ((Handle *)p)->cnn->inputSpatialSize; }
// info: {isLearnt, nFeaturesIn, nFeaturesOut, fn, isPReLU}; dropout as the builder re-quantised it
void refgpu_layer_info(void *p, int layer, int *info, float *dropout) {
  Handle *h = (Handle *)p;
  info[0] = info[1] = info[2] = info[3] = info[4] = 0;
  *dropout = 0;
  SpatiallySparseLayer *L = h->cnn->layers.at(layer);
  if (auto n = dynamic_cast<NetworkInNetworkLayer *>(L)) {
    info[0] = 1; info[1] = n->nFeaturesIn; info[2] = n->nFeaturesOut; info[3] = (int)n->fn;
    *dropout = n->dropout;
  } else if (auto n = dynamic_cast<NetworkInNetworkPReLULayer *>(L)) {
    info[0] = 1; info[1] = n->nFeaturesIn; info[2] = n->nFeaturesOut; info[3] = (int)PRELU; info[4] = 1;
    *dropout = n->dropout;
  } else if (auto n = dynamic_cast<IndexLearnerLayer *>(L)) {
    info[0] = 2; info[1] = n->nFeaturesIn; info[2] = n->nFeaturesOut; info[3] = (int)SOFTMAX;
  }
}
// The layer as the builder made it, ten ints: {type, size, stride, minActiveInputs, nFeaturesIn,
// nFeaturesOut, multiplier, fn, inSpatialSize, outSpatialSize} with type 0 convolution, 1 triangular
// convolution, 2 learnt layer, 3 max pooling, 4 triangular max pooling, 5 terminal pooling,
// 6 fractional max pooling (size = poolSize, multiplier = sd), -1 anything else.
void refgpu_layer_describe(void *p, int layer, int *info) {
  Handle *h = (Handle *)p;
  SpatiallySparseLayer *L = h->cnn->layers.at(layer);
  int v[10] = {-1, 1, 1, 1, 0, 0, 1, 0, 0, 0};
  if (auto c = dynamic_cast<ConvolutionalLayer *>(L)) {
    int w[10] = {0, c->filterSize, c->filterStride, c->minActiveInputs, c->nFeaturesIn, c->nFeaturesOut, c->nFeaturesOut / c->nFeaturesIn, 0, c->inSpatialSize, c->outSpatialSize};
    std::memcpy(v, w, sizeof(v));
  } else if (auto c = dynamic_cast<ConvolutionalTriangularLayer *>(L)) {
    int w[10] = {1, c->filterSize, c->filterStride, c->minActiveInputs, c->nFeaturesIn, c->nFeaturesOut, c->nFeaturesOut / c->nFeaturesIn, 0, c->inSpatialSize, c->outSpatialSize};
    std::memcpy(v, w, sizeof(v));
  } else if (auto n = dynamic_cast<NetworkInNetworkLayer *>(L)) {
    int w[10] = {2, 1, 1, 1, n->nFeaturesIn, n->nFeaturesOut, 1, (int)n->fn, 0, 0};
    std::memcpy(v, w, sizeof(v));
  } else if (auto n = dynamic_cast<NetworkInNetworkPReLULayer *>(L)) {
    int w[10] = {2, 1, 1, 1, n->nFeaturesIn, n->nFeaturesOut, 1, (int)PRELU, 0, 0};
    std::memcpy(v, w, sizeof(v));
  } else if (auto m = dynamic_cast<MaxPoolingLayer *>(L)) {
    int w[10] = {3, m->poolSize, m->poolStride, 1, 0, 0, m->sd, 0, m->inSpatialSize, m->outSpatialSize};
    std::memcpy(v, w, sizeof(v));
  } else if (auto m = dynamic_cast<MaxPoolingTriangularLayer *>(L)) {
    int w[10] = {4, m->poolSize, m->poolStride, 1, 0, 0, m->S, 0, m->inSpatialSize, m->outSpatialSize};
    std::memcpy(v, w, sizeof(v));
  } else if (auto t = dynamic_cast<TerminalPoolingLayer *>(L)) {
    int w[10] = {5, t->poolSize, 1, 1, 0, 0, 1, 0, t->inSpatialSize, t->outSpatialSize};
    std::memcpy(v, w, sizeof(v));
  } else if (describeFmp<PseudorandomOverlappingFractionalMaxPoolingLayer>(L, v) ||
             describeFmp<PseudorandomNonOverlappingFractionalMaxPoolingLayer>(L, v) ||
             describeFmp<RandomOverlappingFractionalMaxPoolingLayer>(L, v) ||
             describeFmp<RandomNonOverlappingFractionalMaxPoolingLayer>(L, v)) {
  }
  std::memcpy(info, v, sizeof(v));
}
// SparseConvNetCUDA::loadWeights (SparseConvNetCUDA.cu:406-424) on <base>_epoch-<epoch>.cnn
void refgpu_load_weights(void *p, const char *base, int epoch) {
  Quiet q;
  ((Handle *)p)->cnn->loadWeights(base, epoch, false);
}
void refgpu_save_weights(void *p, const char *base, int epoch) {
  Quiet q;
  ((Handle *)p)->cnn->saveWeights(base, epoch, false);
}

// One batch: sample s owns rows [off[s], off[s+1]) of (keys, features); a key of -1 marks the sample's
// background row (which must be its first row).  type: 0 TRAINBATCH, 1 TESTBATCH, 2 UNLABELEDBATCH.
// Returns the number of samples processed.
int refgpu_forward(void *p, int nSamples, const int64_t *keys, const int *off, const float *features, const int *labels, int type,
                   float learningRate, float momentum) {
  Quiet q;
  Handle *h = (Handle *)p;
  SparseConvNetCUDA &cnn = *h->cnn;
  h->bp.reset(); // drains and joins the previous producer
  h->batch = nullptr;
  h->pics.clear();
  h->ds = SpatiallySparseDataset();
  h->ds.name = "flat";
  h->ds.nFeatures = cnn.nInputFeatures;
  h->ds.nClasses = cnn.nClasses;
  h->ds.type = (batchType)type;
  const int nF = cnn.nInputFeatures;
  for (int s = 0; s < nSamples; ++s) {
    bool bg = off[s + 1] > off[s] && keys[off[s]] < 0;
    h->pics.emplace_back(new FlatPicture(nF, labels ? labels[s] : -1, bg));
    for (int r = off[s] + (bg ? 1 : 0); r < off[s + 1]; ++r) {
      h->pics.back()->keys.push_back(keys[r]);
      h->pics.back()->feats.insert(h->pics.back()->feats.end(), features + (size_t)r * nF, features + (size_t)(r + 1) * nF);
    }
    h->ds.pictures.push_back(h->pics.back().get());
  }
  multiplyAddCount = 0;
  h->bp.reset(new BatchProducer(cnn, h->ds, cnn.inputSpatialSize, nSamples));
  h->batch = h->bp->nextBatch();
  if (!h->batch) return 0;
  std::ofstream f, g;
  cnn.processBatch(*h->batch, learningRate, momentum, f, g);
  cudaStreamSynchronize(cnn.memStream.stream);
  cudaDeviceSynchronize();
  return h->batch->batchSize;
}
void refgpu_addIndexLearnerLayer(void *p) {
  Quiet q;
  ((Handle *)p)->cnn->addIndexLearnerLayer();
}
// One index-learning step (SparseConvNetCUDA.cu:443-474) on the FIRST batch of `batchSize` pictures that the reference's
// BatchProducer draws from the nSamples pictures given (a TRAINBATCH data set is shuffled: refgpu_sample_numbers tells
// which pictures the batch holds, in order).  Returns the number of pictures processed.
int refgpu_index_learner_batch(void *p, int nSamples, const int64_t *keys, const int *off, const float *features, int batchSize,
                               float learningRate, float momentum) {
  Quiet q;
  Handle *h = (Handle *)p;
  SparseConvNetCUDA &cnn = *h->cnn;
  h->bp.reset();
  h->batch = nullptr;
  h->pics.clear();
  h->ds = SpatiallySparseDataset();
  h->ds.name = "flat";
  h->ds.nFeatures = cnn.nInputFeatures;
  h->ds.nClasses = cnn.nClasses;
  h->ds.type = TRAINBATCH;
  const int nF = cnn.nInputFeatures;
  for (int s = 0; s < nSamples; ++s) {
    bool bg = off[s + 1] > off[s] && keys[off[s]] < 0;
    h->pics.emplace_back(new FlatPicture(nF, s, bg));
    for (int r = off[s] + (bg ? 1 : 0); r < off[s + 1]; ++r) {
      h->pics.back()->keys.push_back(keys[r]);
      h->pics.back()->feats.insert(h->pics.back()->feats.end(), features + (size_t)r * nF, features + (size_t)(r + 1) * nF);
    }
    h->ds.pictures.push_back(h->pics.back().get());
  }
  multiplyAddCount = 0;
  h->bp.reset(new BatchProducer(cnn, h->ds, cnn.inputSpatialSize, batchSize));
  h->batch = h->bp->nextBatch();
  if (!h->batch) return 0;
  std::ofstream f;
  cnn.processIndexLearnerBatch(*h->batch, learningRate, momentum, f);
  cudaStreamSynchronize(cnn.memStream.stream);
  cudaDeviceSynchronize();
  return h->batch->batchSize;
}
// probabilities [batch x width] of the last batch (an index-learning batch has width = batch), stats as refgpu_results
void refgpu_results_wide(void *p, int width, float *probs, double *stats) {
  Handle *h = (Handle *)p;
  SpatiallySparseBatch &b = *h->batch;
  for (int s = 0; s < b.batchSize && probs; ++s) std::memcpy(probs + (size_t)s * width, b.probabilities[s].data(), sizeof(float) * width);
  if (stats) { stats[0] = b.negativeLogLikelihood; stats[1] = b.mistakes; }
}
double refgpu_multiply_adds(void) { return (double)multiplyAddCount; }
int refgpu_last_cuda_error(void) { return (int)cudaGetLastError(); }

// sizes: nSpatialSites, nFeatures, spatialSize, rules, featuresPresent, features, dfeatures, poolingChoices
void refgpu_iface_sizes(void *p, int i, long long *sizes) {
  Handle *h = (Handle *)p;
  SpatiallySparseBatchInterface &I = h->batch->interfaces.at(i);
  sizes[0] = I.nSpatialSites; sizes[1] = I.nFeatures; sizes[2] = I.spatialSize; sizes[3] = I.rules.size();
  sizes[4] = I.featuresPresent.size(); sizes[5] = I.sub->features.size(); sizes[6] = I.sub->dfeatures.size();
  sizes[7] = I.sub->poolingChoices.size();
}
// rowKeys[row] = key of the site stored in that row, -1 for background rows, -2 for rows no grid names
void refgpu_iface_fetch(void *p, int i, float *features, float *dfeatures, int *choices, int *rules, long long *rowKeys, int *backgroundCols) {
  Quiet q;
  Handle *h = (Handle *)p;
  SpatiallySparseBatchInterface &I = h->batch->interfaces.at(i);
  fetch(I.sub->features, features);
  fetch(I.sub->dfeatures, dfeatures);
  fetch(I.sub->poolingChoices, choices);
  fetch(I.rules, rules);
  if (rowKeys) {
    for (int r = 0; r < I.nSpatialSites; ++r) rowKeys[r] = -2;
    for (auto &g : I.grids) {
      for (auto it = g.mp.begin(); it != g.mp.end(); ++it) rowKeys[it->second] = (long long)it->first;
      if (g.backgroundCol >= 0) rowKeys[g.backgroundCol] = -1;
    }
  }
  if (backgroundCols)
    for (size_t s = 0; s < I.grids.size(); ++s) backgroundCols[s] = I.grids[s].backgroundCol;
}
// The features interface i holds (featuresPresent: all of them except behind a learnt layer with dropout in a TRAINBATCH).
void refgpu_iface_features_present(void *p, int i, int *out) {
  Quiet q;
  fetch(((Handle *)p)->batch->interfaces.at(i).featuresPresent, out);
}
// probabilities [batch x nClasses], predictions [batch x nTop], stats = {negativeLogLikelihood, mistakes}
void refgpu_results(void *p, float *probs, int *pred, double *stats) {
  Handle *h = (Handle *)p;
  SpatiallySparseBatch &b = *h->batch;
  for (int s = 0; s < b.batchSize; ++s) {
    if (probs) std::memcpy(probs + (size_t)s * h->cnn->nClasses, b.probabilities[s].data(), sizeof(float) * h->cnn->nClasses);
    if (pred) std::memcpy(pred + (size_t)s * h->cnn->nTop, b.predictions[s].data(), sizeof(int) * h->cnn->nTop);
  }
  if (stats) { stats[0] = b.negativeLogLikelihood; stats[1] = b.mistakes; }
}
// The order in which the batch holds the caller's samples: BatchProducer shuffles a TRAINBATCH dataset
// (BatchProducer.cu:24-27), so row blocks of a training batch follow this permutation.
void refgpu_sample_numbers(void *p, int *out) {
  Handle *h = (Handle *)p;
  for (size_t i = 0; i < h->batch->sampleNumbers.size(); ++i) out[i] = h->batch->sampleNumbers[i];
}
// A learnt layer's weights as they are now (after a TRAINBATCH step: updated by the reference's SGD).
void refgpu_layer_weights(void *p, int layer, float *W, float *B, float *prelu) {
  Quiet q;
  Handle *h = (Handle *)p;
  SpatiallySparseLayer *L = h->cnn->layers.at(layer);
  cudaStreamSynchronize(h->cnn->memStream.stream);
  if (auto n = dynamic_cast<NetworkInNetworkLayer *>(L)) { fetch(n->W, W); fetch(n->B, B); }
  else if (auto n = dynamic_cast<NetworkInNetworkPReLULayer *>(L)) { fetch(n->W, W); fetch(n->B, B); fetch(n->PReLU, prelu); }
  else if (auto n = dynamic_cast<IndexLearnerLayer *>(L)) fetch(n->W, W);
}
}
