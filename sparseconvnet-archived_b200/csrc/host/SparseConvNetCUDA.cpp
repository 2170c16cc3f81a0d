#include "SparseConvNetCUDA.h"
#include "IndexLearnerLayer.h"
#include <chrono>
#include <cmath>
#include "BatchProducer.h"
#include "ConvolutionalLayer.h"
#include "ConvolutionalTriangularLayer.h"
#include "MaxPoolingLayer.h"
#include "MaxPoolingTriangularLayer.h"
#include "NetworkInNetworkLayer.h"
#include "NetworkInNetworkPReLULayer.h"
#include "RuleChain.h"
#include "SoftmaxClassifier.h"
#include "TerminalPoolingLayer.h"

void SparseConvNetCUDA::init(int nInputFeatures_, int nClasses_) {
  if (nBatchProducerThreads < 1 || nBatchProducerThreads > N_MAX_BATCH_PRODUCER_THREADS) throw ScnException("nBatchProducerThreads must be 1..20");
  std::cout << "Sparse CNN - dimension=" << dimension << " nInputFeatures=" << nInputFeatures_ << " nClasses=" << nClasses_ << std::endl;
  nOutputFeatures = nInputFeatures_;
  timing = false;
  // off by default: with BatchProducer threads the next batch is preprocessed while the current one is
  // still in its layers, and the features buffers behind the first layers are shared by the batch pool
  fusePooling = true;
  fuseClassifier = true;
  earlyFirstLayer = false; earlyLayers = 0; inputReady = nullptr; countStream = nullptr; chainDone = nullptr;
  chainRowsHint = 0;
  chainPhase = 0;
  inputBackgroundPending = false;
  inputSpatialSize = 0;
  cublasHandle = nullptr;
  batchPool.reserve(nBatchProducerThreads); // interfaces hold pointers into each other: no reallocation later
  for (int c = 0; c < nBatchProducerThreads; ++c) {
    initialSubInterfaces.push_back(new SpatiallySparseBatchSubInterface());
    batchPool.emplace_back(initialSubInterfaces.back());
  }
}
SparseConvNetCUDA::SparseConvNetCUDA(int dimension, int nInputFeatures, int nClasses, int pciBusID, int nTop, int nBatchProducerThreads)
    : dimension(dimension), nClasses(nClasses), nTop(nTop), nInputFeatures(nInputFeatures), deviceID(initializeGPU(pciBusID)),
      nBatchProducerThreads(nBatchProducerThreads), memStream() {
  init(nInputFeatures, nClasses);
}
SparseConvNetCUDA::SparseConvNetCUDA(int dimension, int nInputFeatures, int nClasses, cudaStream_t stream, int nTop, int nBatchProducerThreads)
    : dimension(dimension), nClasses(nClasses), nTop(nTop), nInputFeatures(nInputFeatures), deviceID(0),
      nBatchProducerThreads(nBatchProducerThreads), memStream(stream) {
  cudaSafeCall(cudaGetDevice(&deviceID));
  if (!scn_device_supported()) throw ScnException("this library runs on compute capability 10.x (B200) devices only");
  init(nInputFeatures, nClasses);
}
SparseConvNetCUDA::~SparseConvNetCUDA() {
  cudaStreamSynchronize(memStream.stream);
  for (auto e : events) cudaEventDestroy(e);
  if (chainDone) cudaEventDestroy(chainDone);
  if (countStream) cudaStreamDestroy(countStream);
  for (auto L : layers)
    if (auto m = dynamic_cast<MaxPoolingLayer *>(L))
      if (m->splitEvent) cudaEventDestroy(m->splitEvent);
  for (auto p : layers) delete p;
  batchPool.clear();
  for (auto p : initialSubInterfaces) delete p;
  for (auto p : sharedSubInterfaces) delete p;
}

// Widths are rounded to multiples of 32 and dropout is re-quantised the same way
// (SparseConvNetCUDA.cu:50-70): existing weight files assume these sizes.
void SparseConvNetCUDA::addLearntLayer(int nFeatures, ActivationFunction activationFn, float dropout, float alpha) {
  if (activationFn != SOFTMAX) nFeatures = std::max(KERNELBLOCKSIZE, intRound(nFeatures, KERNELBLOCKSIZE));
  if (dropout > 0) dropout = 1 - (intRound(nFeatures * (1 - dropout), KERNELBLOCKSIZE) + 0.01f) * 1.0f / nFeatures;
  if (dropout < 0) dropout = 0;
  std::cout << layers.size() << ":";
  if (activationFn == PRELU)
    layers.push_back(new NetworkInNetworkPReLULayer(memStream, cublasHandle, nOutputFeatures, nFeatures, dropout, alpha));
  else
    layers.push_back(new NetworkInNetworkLayer(memStream, cublasHandle, nOutputFeatures, nFeatures, dropout, activationFn, alpha));
  nOutputFeatures = nFeatures;
}
void SparseConvNetCUDA::addNetworkInNetworkLayer(int nFeatures, ActivationFunction activationFn, float dropout) {
  addLearntLayer(nFeatures, activationFn, dropout, 1.0f);
}
void SparseConvNetCUDA::addConvolutionalLayer(int nFeatures, int filterSize, int filterStride, ActivationFunction activationFn, float dropout,
                                              int minActiveInputs, float poolingToFollow) {
  if (filterSize > 1) {
    std::cout << layers.size() << ":";
    ConvolutionalLayer *c = new ConvolutionalLayer(memStream, filterSize, filterStride, dimension, nOutputFeatures, minActiveInputs);
    c->fuseWithNext = true; // the learnt layer added next runs gather + GEMM + epilogue as one kernel
    layers.push_back(c);
    nOutputFeatures *= ipow(filterSize, dimension);
  }
  addLearntLayer(nFeatures, activationFn, dropout, std::pow(filterSize * 1.0f / filterStride / poolingToFollow, 2.0f));
}
void SparseConvNetCUDA::addLeNetLayerMP(int nFeatures, int filterSize, int filterStride, int poolSize, int poolStride,
                                        ActivationFunction activationFn, float dropout, int minActiveInputs) {
  addConvolutionalLayer(nFeatures, filterSize, filterStride, activationFn, dropout, minActiveInputs, poolSize);
  if (poolSize > 1) {
    std::cout << layers.size() << ":";
    // windows that do not overlap and hold 2..32 cells (a power of two): the learnt layer leaves its output to the pooling layer's fused kernel
    const int cells = ipow(poolSize, dimension);
    if (poolSize == poolStride && cells >= 2 && cells <= 32 && (cells & (cells - 1)) == 0 && filterSize > 1)
      if (auto nin = dynamic_cast<NetworkInNetworkLayer *>(layers.back())) nin->fusePoolNext = fusePooling;
    layers.push_back(new MaxPoolingLayer(memStream, poolSize, poolStride, dimension));
  }
}
void SparseConvNetCUDA::addTriangularConvolutionalLayer(int nFeatures, int filterSize, int filterStride, ActivationFunction activationFn,
                                                        float dropout, int minActiveInputs, float poolingToFollow) {
  if (filterSize > 1) {
    std::cout << layers.size() << ":";
    ConvolutionalTriangularLayer *c =
        new ConvolutionalTriangularLayer(memStream, filterSize, filterStride, dimension, nOutputFeatures, minActiveInputs);
    c->fuseWithNext = true;
    layers.push_back(c);
    nOutputFeatures *= triangleSize(filterSize, dimension);
  }
  addLearntLayer(nFeatures, activationFn, dropout, std::pow(filterSize * 1.0f / filterStride / poolingToFollow, 2.0f));
}
// The reference passes poolSize where the callee expects minActiveInputs and
// minActiveInputs where it expects poolingToFollow (SparseConvNetCUDA.cu:183-185 against
// 165-168).  Networks trained with it depend on that, so the call is reproduced as is: with
// poolSize 2 the convolution keeps only sites with at least two active inputs.
void SparseConvNetCUDA::addTriangularLeNetLayerMP(int nFeatures, int filterSize, int filterStride, int poolSize, int poolStride,
                                                  ActivationFunction activationFn, float dropout, int minActiveInputs) {
  addTriangularConvolutionalLayer(nFeatures, filterSize, filterStride, activationFn, dropout, poolSize, (float)minActiveInputs);
  if (poolSize > 1) {
    std::cout << layers.size() << ":";
    layers.push_back(new MaxPoolingTriangularLayer(memStream, poolSize, poolStride, dimension));
  }
}
// SparseConvNetCUDA.cu:112-163: the shrink factor takes the poolingToFollow slot; no FMP layer if it does not shrink.
#define SCN_ADD_FMP(NAME, LAYER)                                                                                                      \
  void SparseConvNetCUDA::NAME(int nFeatures, int filterSize, int filterStride, int poolSize, float fmpShrink,                      \
                               ActivationFunction activationFn, float dropout, int minActiveInputs) {                               \
    addConvolutionalLayer(nFeatures, filterSize, filterStride, activationFn, dropout, minActiveInputs, fmpShrink);                  \
    if (fmpShrink > 1) {                                                                                                            \
      std::cout << layers.size() << ":";                                                                                            \
      layers.push_back(new LAYER(memStream, poolSize, fmpShrink, dimension));                                                       \
    }                                                                                                                               \
  }
SCN_ADD_FMP(addLeNetLayerROFMP, RandomOverlappingFractionalMaxPoolingLayer)
SCN_ADD_FMP(addLeNetLayerPOFMP, PseudorandomOverlappingFractionalMaxPoolingLayer)
SCN_ADD_FMP(addLeNetLayerRDFMP, RandomNonOverlappingFractionalMaxPoolingLayer)
SCN_ADD_FMP(addLeNetLayerPDFMP, PseudorandomNonOverlappingFractionalMaxPoolingLayer)
#undef SCN_ADD_FMP
void SparseConvNetCUDA::addTerminalPoolingLayer(int poolSize, int S) {
  std::cout << layers.size() << ":";
  TerminalPoolingLayer *t = new TerminalPoolingLayer(memStream, poolSize, S);
  t->dimension = dimension;
  layers.push_back(t);
}
void SparseConvNetCUDA::addSoftmaxLayer() {
  addLearntLayer(nClasses, SOFTMAX, 0.0f, 1);
  inputSpatialSize = 1;
  std::cout << "Spatially sparse CNN with layer sizes: " << inputSpatialSize;
  for (int i = (int)layers.size() - 1; i >= 0; --i) inputSpatialSize = layers[i]->calculateInputSpatialSize(inputSpatialSize);
  std::cout << std::endl << "Input-field dimensions = " << inputSpatialSize;
  for (int i = 1; i < dimension; ++i) std::cout << "x" << inputSpatialSize;
  std::cout << std::endl;
}

// SparseConvNetCUDA.cu:211-225: "nClasses" is the number of pictures of the training set.
void SparseConvNetCUDA::addIndexLearnerLayer() {
  std::cout << layers.size() << ":";
  layers.push_back(new IndexLearnerLayer(memStream, cublasHandle, nOutputFeatures, nClasses));
  std::cout << "Index Learner " << nOutputFeatures << "-> " << nClasses << std::endl;
  nOutputFeatures = nClasses;
  inputSpatialSize = 1;
  for (int i = (int)layers.size() - 1; i >= 0; --i) inputSpatialSize = layers[i]->calculateInputSpatialSize(inputSpatialSize);
  std::cout << "Spatially sparse CNN: input size " << inputSpatialSize;
  for (int i = 1; i < dimension; ++i) std::cout << "x" << inputSpatialSize;
  std::cout << std::endl;
}

void SparseConvNetCUDA::prepareBatch(SpatiallySparseBatch &batch) {
  if (batch.interfaces.size() == layers.size() + 1) return;
  batch.interfaces.reserve(layers.size() + 1); // before any pointer into the vector exists
  while (sharedSubInterfaces.size() < layers.size()) sharedSubInterfaces.push_back(new SpatiallySparseBatchSubInterface());
  // interfaces behind layer i share one sub-interface across the pool: one batch in flight
  // on the device at a time (BatchProducer.cu:28-33)
  while (batch.interfaces.size() < layers.size() + 1) batch.interfaces.emplace_back(sharedSubInterfaces[batch.interfaces.size() - 1]);
}

void SparseConvNetCUDA::preprocessBatchOnDevice(SpatiallySparseBatch &batch) {
  prepareBatch(batch);
  const int nL = (int)layers.size();
  // two sets of result records, used in turn: the fused rule chain of one batch clears the records of the next
  chainResults.resize(8 * nL + 4);
  const int phase = chainPhase;
  chainPhase ^= 1;
  int *d_res = chainResults.dPtr() + phase * 4 * nL;
  rulechain::ResidentChain resident = {phase, chainResults.dPtr() + (1 - phase) * 4 * nL, 4 * nL, inputBackgroundPending};
  inputBackgroundPending = false;
  long long bound = batch.interfaces[0].nSpatialSites, bound0 = 0, bound2 = 0;
  earlyLayers = 0;
  if (timing) cudaSafeCall(cudaEventRecord(events[nL + 1], memStream.stream));
  // Without terminal pooling (whose build reads its input grid at once) the region builds are
  // only recorded here and then run together: one fused kernel when the samples are small.
  bool defer = true;
  for (auto L : layers) defer = defer && dynamic_cast<TerminalPoolingLayer *>(L) == nullptr && dynamic_cast<FractionalMaxPoolingLayerBase *>(L) == nullptr;
  if (resident.findBackground && (!defer || nL == 0 || !layers[0]->changesGeometry)) { // no fused chain will look for them
    SpatiallySparseBatchInterface &in = batch.interfaces[0];
    scnSafeCall(scn_background_rows(in.siteKeys.dPtr(), in.sampleOffsets.dPtr(), batch.batchSize, in.backgroundRows.dPtr(), memStream.stream));
    resident.findBackground = false;
  }
  std::vector<rulechain::DeferredBuild> builds;
  if (defer) rulechain::beginDeferred(&builds);
  try {
    for (int i = 0; i < nL; ++i) {
      bound = layers[i]->enqueueRules(batch, batch.interfaces[i], batch.interfaces[i + 1], bound, d_res + 4 * i);
      if (i == 0) bound0 = bound;
      if (i == 2) bound2 = bound;
    }
  } catch (...) {
    rulechain::endDeferred();
    throw;
  }
  bool hinted = false;
  if (defer) {
    rulechain::endDeferred();
    hinted = rulechain::runDeferred(builds, batch.batchSize, batch.interfaces[0].maxSitesPerSample + 1, chainRowsHint, memStream, &resident);
  }
  if (timing) cudaSafeCall(cudaEventRecord(events[nL + 2], memStream.stream));
  if (inputReady) { // the features were uploaded on another stream while the rules were built
    cudaSafeCall(cudaStreamWaitEvent(memStream.stream, inputReady, 0));
    inputReady = nullptr;
  }
  int *h = (int *)memStream.staging(sizeof(int) * (4 * nL + 1));
  // The error word of the tensor-core kernels rides along with the counts: set by an earlier batch's kernels whose
  // results were never read through SoftmaxClassifier (the device-resident entry point), it is reported here.
  const int *tcWord = scn_conv_tc_error_word();
  h[4 * nL] = 0;
  bool countsRead = false;
  if (earlyFirstLayer && !timing && defer && nL >= 2) {
    ConvolutionalLayer *conv = dynamic_cast<ConvolutionalLayer *>(layers[0]);
    NetworkInNetworkLayer *nin = dynamic_cast<NetworkInNetworkLayer *>(layers[1]);
    if (conv && conv->fuseWithNext && nin) {
      if (!countStream) {
        cudaSafeCall(cudaStreamCreateWithFlags(&countStream, cudaStreamNonBlocking));
        cudaSafeCall(cudaEventCreateWithFlags(&chainDone, cudaEventDisableTiming));
      }
      cudaSafeCall(cudaEventRecord(chainDone, memStream.stream));
      const int convCells = ipow(conv->filterSize, conv->dimension);
      MaxPoolingLayer *pool = nL >= 3 ? dynamic_cast<MaxPoolingLayer *>(layers[2]) : nullptr;
      if (nin->fusePoolNext && pool && pool->poolSize == pool->poolStride &&
          nin->forwardsPooled(batch, batch.interfaces[0], batch.interfaces[1], batch.interfaces[3], convCells, pool->sd, bound2, d_res + 8))
      { earlyLayers = 3; pool->fusedLast = true; } // convolution + learnt layer + pooling, the pooled row count read from the pooling layer's record
      else if (nin->forwardsEarly(batch, batch.interfaces[0], batch.interfaces[1], batch.interfaces[2], convCells, bound0, d_res))
        earlyLayers = 2;
      if (earlyLayers) {
        // the counts come back on their own stream, behind the rule chain only, while the first layer runs
        cudaSafeCall(cudaStreamWaitEvent(countStream, chainDone, 0));
        cudaSafeCall(cudaMemcpyAsync(h, d_res, sizeof(int) * 4 * nL, cudaMemcpyDeviceToHost, countStream));
        if (tcWord) cudaSafeCall(cudaMemcpyAsync(h + 4 * nL, tcWord, sizeof(int), cudaMemcpyDeviceToHost, countStream));
        cudaSafeCall(cudaStreamSynchronize(countStream));
        countsRead = true;
      }
    }
  }
  if (!countsRead) {
    cudaSafeCall(cudaMemcpyAsync(h, d_res, sizeof(int) * 4 * nL, cudaMemcpyDeviceToHost, memStream.stream));
    if (tcWord) cudaSafeCall(cudaMemcpyAsync(h + 4 * nL, tcWord, sizeof(int), cudaMemcpyDeviceToHost, memStream.stream));
    cudaSafeCall(cudaStreamSynchronize(memStream.stream)); // the one host wait of the rule chain
  }
  if (h[4 * nL]) {
    const int code = h[4 * nL];
    scn_conv_tc_take_error(); // clear it: the kernels launched from here on wait with their full time limit again
    throw ScnException("a tensor-core kernel of an earlier batch gave up a time-limited wait (code " + std::to_string(code) +
                       "): that batch's results are not valid");
  }
  std::vector<int> counts(h, h + 4 * nL); // staging is reused below
  if (hinted) { // a sample outgrew the shared-memory hint learnt from earlier batches: rebuild for the worst case
    bool overflow = false;
    for (int i = 0; i < nL; ++i) overflow = overflow || (layers[i]->changesGeometry && (counts[4 * i + 2] & SCN_DEV_ERR_CAPACITY));
    if (overflow) {
      earlyLayers = 0; // the early kernel ran on truncated rules: the layers run again from the first
      chainRowsHint = 0;
      const rulechain::ResidentChain again = {phase, resident.resultNext, resident.nResultNext, false}; // (the background rows are known by now)
      rulechain::runDeferred(builds, batch.batchSize, batch.interfaces[0].maxSitesPerSample + 1, 0, memStream, &again);
      cudaSafeCall(cudaMemcpyAsync(h, d_res, sizeof(int) * 4 * nL, cudaMemcpyDeviceToHost, memStream.stream));
      cudaSafeCall(cudaStreamSynchronize(memStream.stream));
      counts.assign(h, h + 4 * nL);
    }
  }
  if (defer) { // remember how large samples get, with head-room, for the next batch's shared-memory plan
    int most = batch.interfaces[0].maxSitesPerSample + 1;
    for (int i = 0; i < nL; ++i) if (layers[i]->changesGeometry) most = std::max(most, counts[4 * i + 3] + 1);
    chainRowsHint = std::max(chainRowsHint, most + most / 4 + 32);
  }
  for (int i = 0; i < nL; ++i) layers[i]->finishRules(batch, batch.interfaces[i], batch.interfaces[i + 1], counts.data() + 4 * i);
}

void SparseConvNetCUDA::forwardLayers(SpatiallySparseBatch &batch, size_t count) {
  count = std::min(count, layers.size());
  for (size_t i = 0; i < count; ++i) {
    if (timing) cudaSafeCall(cudaEventRecord(events[i], memStream.stream));
    if ((int)i == 1 && earlyLayers == 2) { // already running: launched behind the rule chain
      static_cast<NetworkInNetworkLayer *>(layers[1])->finishEarly(batch.interfaces[1], batch.interfaces[2]);
      continue;
    }
    if (earlyLayers == 3 && (i == 1 || i == 2)) { // convolution + learnt layer + pooling already running as one kernel
      SpatiallySparseBatchInterface &out = batch.interfaces[i + 1];
      if (i == 1) {
        out.sub->reset();
        out.deferredLearnt = static_cast<NetworkInNetworkLayer *>(layers[1]);
        out.deferredLearntInput = &batch.interfaces[1];
        out.deferredLearnt->countMultiplyAdds(batch.interfaces[1], out);
      } else {
        const int n = out.nSpatialSites * out.featuresPresent.size();
        out.sub->features.resize(n);
        out.sub->poolingChoices.resize(n);
      }
      continue;
    }
    batch.interfaces[i + 1].sub->reset();
    batch.interfaces[i + 1].deferredFrom = nullptr;
    batch.interfaces[i + 1].deferredLearnt = nullptr;
    if (fuseClassifier && i + 1 < count) { // a learnt layer of few rows and the small learnt layer behind it (the classifier) as one call
      auto a = dynamic_cast<NetworkInNetworkLayer *>(layers[i]);
      auto b = dynamic_cast<NetworkInNetworkLayer *>(layers[i + 1]);
      if (a && b) {
        batch.interfaces[i + 2].sub->reset();
        batch.interfaces[i + 2].deferredFrom = nullptr;
        batch.interfaces[i + 2].deferredLearnt = nullptr;
        if (a->forwardsWithNext(batch, batch.interfaces[i], batch.interfaces[i + 1], *b, batch.interfaces[i + 2])) {
          if (timing) cudaSafeCall(cudaEventRecord(events[i + 1], memStream.stream));
          ++i;
          continue;
        }
      }
    }
    layers[i]->forwards(batch, batch.interfaces[i], batch.interfaces[i + 1]);
  }
  if (timing) cudaSafeCall(cudaEventRecord(events[count], memStream.stream));
}
void SparseConvNetCUDA::enableTiming(bool on) {
  timing = on;
  while (on && events.size() < layers.size() + 3) {
    cudaEvent_t e;
    cudaSafeCall(cudaEventCreate(&e));
    events.push_back(e);
  }
  for (auto L : layers)
    if (auto m = dynamic_cast<MaxPoolingLayer *>(L)) {
      if (on && !m->splitEvent) cudaSafeCall(cudaEventCreate(&m->splitEvent));
      if (!on && m->splitEvent) { cudaSafeCall(cudaEventDestroy(m->splitEvent)); m->splitEvent = nullptr; }
    }
}
std::vector<float> SparseConvNetCUDA::layerTimes() {
  std::vector<float> ms(layers.size() + 1, 0.f);
  if (!timing) return ms;
  cudaSafeCall(cudaStreamSynchronize(memStream.stream));
  const size_t nL = layers.size();
  for (size_t i = 0; i < nL; ++i) cudaSafeCall(cudaEventElapsedTime(&ms[i], events[i], events[i + 1]));
  cudaSafeCall(cudaEventElapsedTime(&ms[nL], events[nL + 1], events[nL + 2]));
  for (size_t i = 1; i < nL; ++i) // a pooling layer that ran the learnt layer in front of it as a kernel of its own
    if (auto m = dynamic_cast<MaxPoolingLayer *>(layers[i]))
      if (m->splitEvent && m->splitRecorded) {
        float t = 0;
        cudaSafeCall(cudaEventElapsedTime(&t, events[i], m->splitEvent));
        ms[i - 1] += t;
        ms[i] -= t;
      }
  return ms;
}

// SparseConvNetCUDA.cu:227-271: every layer's forwards (on a RESCALEBATCH each followed by its scaleWeights),
// SoftmaxClassifier and, for a TRAINBATCH, every layer's backwards in reverse order (each learnt layer updates its
// weights on the way).
void SparseConvNetCUDA::processBatch(SpatiallySparseBatch &batch, float learningRate, float momentum, std::ofstream &f, std::ofstream &g) {
  if (batch.type == RESCALEBATCH) {
    float scalingUnderneath = 1;
    for (size_t i = 0; i < layers.size(); ++i) {
      batch.interfaces[i + 1].sub->reset();
      batch.interfaces[i + 1].deferredFrom = nullptr;
      batch.interfaces[i + 1].deferredLearnt = nullptr;
      layers[i]->forwards(batch, batch.interfaces[i], batch.interfaces[i + 1]);
      layers[i]->scaleWeights(batch.interfaces[i], batch.interfaces[i + 1], scalingUnderneath, i + 1 == layers.size());
    }
  } else
    forwardLayers(batch);
  SoftmaxClassifier(batch.interfaces.back(), batch, nTop, memStream);
  if (batch.type == TRAINBATCH)
    for (int i = (int)layers.size() - 1; i >= 0; --i) layers[i]->backwards(batch, batch.interfaces[i], batch.interfaces[i + 1], learningRate, momentum);
  if (f)
    for (auto &p : batch.predictions) {
      for (size_t k = 0; k < p.size(); ++k) f << (k ? " " : "") << p[k];
      f << std::endl;
    }
  if (g)
    for (auto &p : batch.probabilities) {
      for (size_t k = 0; k < p.size(); ++k) g << (k ? " " : "") << p[k];
      g << std::endl;
    }
}

// SparseConvNetCUDA.cu:443-474: every layer but the index learner runs forwards; `f`, if open, receives the features under
// the index learner ("sample number, label, features" per picture); a TRAINBATCH then runs the index learner on the
// columns of its own pictures, IndexLearner, and every layer's backwards.
void SparseConvNetCUDA::processIndexLearnerBatch(SpatiallySparseBatch &batch, float learningRate, float momentum, std::ofstream &f) {
  const int n = (int)layers.size();
  auto top = n ? dynamic_cast<IndexLearnerLayer *>(layers[n - 1]) : nullptr;
  if (!top) throw ScnException("processIndexLearnerBatch: the network's last layer must be an IndexLearnerLayer (addIndexLearnerLayer)");
  forwardLayers(batch, n - 1);
  SpatiallySparseBatchInterface &under = batch.interfaces[n - 1];
  if (f.is_open()) {
    cudaSafeCall(cudaStreamSynchronize(memStream.stream));
    if (under.nSpatialSites != batch.batchSize) throw ScnException("processIndexLearnerBatch: the layer under the index learner must hold one row per picture");
    std::vector<float> feat((size_t)batch.batchSize * under.nFeatures);
    if (!feat.empty()) cudaSafeCall(cudaMemcpy(feat.data(), under.sub->features.dPtr(), sizeof(float) * feat.size(), cudaMemcpyDeviceToHost));
    std::vector<int> &labels = batch.labels.hVector();
    for (int i = 0; i < batch.batchSize; ++i) {
      f << batch.sampleNumbers[i] << " " << (i < (int)labels.size() ? labels[i] : -1);
      for (int j = 0; j < under.nFeatures; ++j) f << " " << feat[(size_t)i * under.nFeatures + j];
      f << std::endl;
    }
  }
  if (batch.type == TRAINBATCH) {
    top->indexLearnerIndices = batch.sampleNumbers;
    batch.interfaces[n].sub->reset();
    top->forwards(batch, under, batch.interfaces[n]);
    IndexLearner(batch.interfaces[n], batch, nTop, memStream);
    for (int i = n - 1; i >= 0; --i) layers[i]->backwards(batch, batch.interfaces[i], batch.interfaces[i + 1], learningRate, momentum);
  }
}

// SparseConvNetCUDA.cu:475-510: one pass; a data set that is not a training set writes "<name>.features" instead of learning.
float SparseConvNetCUDA::processIndexLearnerDataset(SpatiallySparseDataset &dataset, int batchSize, float learningRate, float momentum) {
  if (dataset.pictures.empty()) throw ScnException("processIndexLearnerDataset: empty dataset");
  float errorRate = 0, nll = 0;
  multiplyAddCount = 0;
  auto start = std::chrono::system_clock::now();
  std::ofstream f;
  BatchProducer bp(*this, dataset, inputSpatialSize, batchSize);
  if (dataset.type != TRAINBATCH) f.open((dataset.name + ".features").c_str());
  while (SpatiallySparseBatch *batch = bp.nextBatch()) {
    processIndexLearnerBatch(*batch, learningRate, momentum, f);
    errorRate += batch->mistakes * 1.0 / dataset.pictures.size();
    nll += batch->negativeLogLikelihood * 1.0 / dataset.pictures.size();
  }
  auto end = std::chrono::system_clock::now();
  double diff = std::chrono::duration_cast<std::chrono::nanoseconds>(end - start).count();
  if (dataset.type == TRAINBATCH)
    std::cout << dataset.name << " Mistakes:" << 100.0 * errorRate << "% NLL:" << nll
              << " MegaMultiplyAdds/sample:" << std::round((double)multiplyAddCount / dataset.pictures.size() / 1000000) << " time:" << diff / 1000000000L
              << "s GigaMultiplyAdds/s:" << std::round((double)multiplyAddCount / diff) << " rate:" << std::round(dataset.pictures.size() * 1000000000.0f / diff)
              << "/s" << std::endl;
  return nll; // (SparseConvNetCUDA.cu:505)
}

// SparseConvNetCUDA.cu:507-535: every layer but the last runs forwards and the features under it go to "<name>.features"
// ("sample number, label, features" per picture), `reps` passes over a data set that is not a training set.
void SparseConvNetCUDA::processBatchDumpTopLevelFeaturess(SpatiallySparseBatch &batch, std::ofstream &f) {
  const int n = (int)layers.size();
  if (n < 1) throw ScnException("processBatchDumpTopLevelFeaturess: the network has no layers");
  forwardLayers(batch, n - 1);
  cudaSafeCall(cudaStreamSynchronize(memStream.stream));
  SpatiallySparseBatchInterface &under = batch.interfaces[n - 1];
  if (under.nSpatialSites != batch.batchSize) throw ScnException("processBatchDumpTopLevelFeaturess: the layer under the top one must hold one row per picture");
  std::vector<float> feat((size_t)batch.batchSize * under.nFeatures);
  if (!feat.empty()) cudaSafeCall(cudaMemcpy(feat.data(), under.sub->features.dPtr(), sizeof(float) * feat.size(), cudaMemcpyDeviceToHost));
  std::vector<int> &labels = batch.labels.hVector();
  for (int i = 0; i < batch.batchSize; ++i) {
    f << batch.sampleNumbers[i] << " " << (i < (int)labels.size() ? labels[i] : -1);
    for (int j = 0; j < under.nFeatures; ++j) f << " " << feat[(size_t)i * under.nFeatures + j];
    f << std::endl;
  }
}
void SparseConvNetCUDA::processDatasetDumpTopLevelFeatures(SpatiallySparseDataset &dataset, int batchSize, int reps) {
  if (dataset.pictures.empty()) throw ScnException("processDatasetDumpTopLevelFeatures: empty dataset");
  if (dataset.type == TRAINBATCH) throw ScnException("processDatasetDumpTopLevelFeatures: not for a training set");
  std::ofstream f((dataset.name + ".features").c_str());
  for (int i = 0; i < reps; ++i) {
    BatchProducer bp(*this, dataset, inputSpatialSize, batchSize);
    while (SpatiallySparseBatch *batch = bp.nextBatch()) processBatchDumpTopLevelFeaturess(*batch, f);
  }
}

// SparseConvNetCUDA.cu:537-566: one over the largest absolute value of each input feature over (at most 10000 pictures of)
// the data set, read as a test set (no augmentation); BatchProducer multiplies every batch's input by them from then on
// and the weight files carry them.
void SparseConvNetCUDA::calculateInputRegularizingConstants(SpatiallySparseDataset dataset) { // (a copy, as in the reference)
  inputNormalizingConstants.resize(0); // no rescaling while the maxima are taken
  std::cout << "Using " << std::min(10000, (int)dataset.pictures.size()) << " out of " << dataset.pictures.size()
            << " training samples to calculate regularizing constants." << std::endl;
  if (dataset.pictures.size() > 10000) dataset.pictures.resize(10000);
  dataset.type = TESTBATCH;
  std::vector<float> c(nInputFeatures, 0.f);
  {
    BatchProducer bp(*this, dataset, inputSpatialSize, 100);
    while (SpatiallySparseBatch *batch = bp.nextBatch()) {
      cudaSafeCall(cudaStreamSynchronize(memStream.stream));
      std::vector<float> &features = batch->interfaces[0].sub->features.hVector();
      for (size_t i = 0; i < features.size(); ++i) c[i % nInputFeatures] = std::max(c[i % nInputFeatures], std::fabs(features[i]));
    }
  }
  for (int i = 0; i < nInputFeatures; ++i) {
    inputNormalizingConstants.push_back(c[i] > 0 ? 1.0f / c[i] : 0);
    std::cout << inputNormalizingConstants.back() << " ";
  }
  std::cout << std::endl;
}

// One pass over a dataset (SparseConvNetCUDA.cu:272-326): prints the reference's summary line and returns the mean
// negative log-likelihood.  A TRAINBATCH dataset is shuffled by the batch producer and every batch updates the weights.
float SparseConvNetCUDA::processDataset(SpatiallySparseDataset &dataset, int batchSize, float learningRate, float momentum) {
  if (dataset.pictures.empty()) throw ScnException("processDataset: empty dataset");
  float errorRate = 0, nll = 0;
  multiplyAddCount = 0;
  auto start = std::chrono::system_clock::now();
  std::ofstream f, g;
  BatchProducer bp(*this, dataset, inputSpatialSize, batchSize);
  if (dataset.type == UNLABELEDBATCH) {
    f.open("unlabelledData.predictions");
    g.open("unlabelledData.probabilities");
  }
  while (SpatiallySparseBatch *batch = bp.nextBatch()) {
    processBatch(*batch, learningRate, momentum, f, g);
    errorRate += batch->mistakes * 1.0 / dataset.pictures.size();
    nll += batch->negativeLogLikelihood * 1.0 / dataset.pictures.size();
  }
  auto end = std::chrono::system_clock::now();
  double diff = std::chrono::duration_cast<std::chrono::nanoseconds>(end - start).count();
  if (dataset.type != RESCALEBATCH) { // the summary line of SparseConvNetCUDA.cu:310-324
    std::cout << dataset.name;
    if (dataset.type != UNLABELEDBATCH) std::cout << " Mistakes:" << 100.0 * errorRate << "% NLL:" << nll;
    std::cout << " MegaMultiplyAdds/sample:" << std::round((double)multiplyAddCount / dataset.pictures.size() / 1000000)
              << " time:" << diff / 1000000000L << "s GigaMultiplyAdds/s:" << std::round((double)multiplyAddCount / diff)
              << " rate:" << std::round(dataset.pictures.size() * 1000000000.0f / diff) << "/s" << std::endl;
  }
  return nll; // (the mean negative log-likelihood, as SparseConvNetCUDA.cu:325 returns it; the error rate is in the printed line)
}

// Repeated test passes with averaged probabilities (SparseConvNetCUDA.cu:327-405): prints the
// cumulative error after each repetition and optionally writes predictions / a confusion matrix.
void SparseConvNetCUDA::processDatasetRepeatTest(SpatiallySparseDataset &dataset, int batchSize, int nReps, std::string predictionsFilename,
                                                 std::string confusionMatrixFilename) {
  const size_t n = dataset.pictures.size();
  std::vector<std::vector<float>> probs(n, std::vector<float>(dataset.nClasses, 0.f));
  std::ofstream nof, nog;
  for (int rep = 1; rep <= nReps; ++rep) {
    BatchProducer bp(*this, dataset, inputSpatialSize, batchSize);
    size_t at = 0;
    while (SpatiallySparseBatch *batch = bp.nextBatch()) {
      processBatch(*batch, 0, 0, nof, nog);
      for (int i = 0; i < batch->batchSize; ++i, ++at)
        for (int k = 0; k < dataset.nClasses; ++k) probs[at][k] += batch->probabilities[i][k];
    }
    int mistakes = 0;
    double nll = 0;
    std::vector<std::vector<int>> confusion(dataset.nClasses, std::vector<int>(dataset.nClasses, 0));
    std::ofstream pf;
    if (!predictionsFilename.empty()) pf.open(predictionsFilename.c_str());
    for (size_t i = 0; i < n; ++i) {
      std::vector<int> pred = vectorTopIndices(probs[i], nTop);
      const int label = dataset.pictures[i]->label;
      bool hit = false;
      for (int j = 0; j < nTop; ++j) hit = hit || pred[j] == label;
      if (label >= 0) {
        mistakes += !hit;
        nll -= std::log(std::max(probs[i][label] / rep, 1.0e-15f));
        confusion[label][pred[0]]++;
      }
      if (pf) { for (int j = 0; j < nTop; ++j) pf << (j ? " " : "") << pred[j]; pf << std::endl; }
    }
    std::cout << dataset.name << " rep " << rep << "/" << nReps << " Mistakes: " << 100.0 * mistakes / n << "% NLL " << nll / n << std::endl;
    if (!confusionMatrixFilename.empty()) {
      std::ofstream cm(confusionMatrixFilename.c_str());
      for (auto &row : confusion) { for (size_t k = 0; k < row.size(); ++k) cm << (k ? " " : "") << row[k]; cm << std::endl; }
    }
  }
}

// <base>_epoch-<n>.cnn: every layer's weights in order, then the input normalising constants
// (SparseConvNetCUDA.cu:406-442).
void SparseConvNetCUDA::loadWeights(std::string baseName, int epoch, bool momentum, int firstNlayers) {
  std::string filename = baseName + "_epoch-" + std::to_string(epoch) + ".cnn";
  std::ifstream f(filename.c_str(), std::ios::in | std::ios::binary);
  if (!f) throw ScnException("Cannot find " + filename);
  std::cout << "Loading network parameters from " << filename << std::endl;
  for (int i = 0; i < std::min((int)layers.size(), firstNlayers); ++i) layers[i]->loadWeightsFromStream(f, momentum);
  if (!inputNormalizingConstants.empty()) f.read((char *)inputNormalizingConstants.data(), sizeof(float) * inputNormalizingConstants.size());
}
void SparseConvNetCUDA::saveWeights(std::string baseName, int epoch, bool momentum) {
  std::string filename = baseName + "_epoch-" + std::to_string(epoch) + ".cnn";
  std::ofstream f(filename.c_str(), std::ios::binary);
  if (!f) throw ScnException("Cannot write " + filename);
  for (auto l : layers) l->putWeightsToStream(f, momentum);
  if (!inputNormalizingConstants.empty()) f.write((char *)inputNormalizingConstants.data(), sizeof(float) * inputNormalizingConstants.size());
}
