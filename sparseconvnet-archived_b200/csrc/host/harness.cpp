// extern "C" entry points over the C++ classes (include/scn_b200_net.h).
#include <cstring>
#include <memory>
#include <sstream>
#include "BatchProducer.h"
#include "ConvolutionalLayer.h"
#include "ConvolutionalTriangularLayer.h"
#include "MaxPoolingLayer.h"
#include "MaxPoolingTriangularLayer.h"
#include "NetworkArchitectures.h"
#include "IndexLearnerLayer.h"
#include "NetworkInNetworkLayer.h"
#include "NetworkInNetworkPReLULayer.h"
#include "ResultExchange.h"
#include "SoftmaxClassifier.h"
#include "SparseConvNetCUDA.h"
#include "TerminalPoolingLayer.h"
#include "scn_b200_net.h"

struct scn_net {
  std::unique_ptr<SparseConvNetCUDA> cnn;
  int lattice;
  SpatiallySparseBatch *last; // batch of the last forward
  vectorCUDA<int> top;
  // scn_net_forward_host uploads the features on a stream of their own, so that the copy (three
  // quarters of the input bytes) runs while the rule chain, which needs only keys and offsets, is built
  cudaStream_t copyStream = nullptr;
  cudaEvent_t copyDone = nullptr;
  // host buffers already seen to be page-locked (a driver query per buffer and call costs microseconds; should one
  // of them have become pageable since, its copy is still correct, only less asynchronous)
  std::vector<const void *> knownPinned;
  std::unique_ptr<ResultExchange> exchange; // results to and from the other ranks of a sharded batch
  // scn_net_forward_host_begin / _end: the inputs of the batch after the one being computed travel to one of two
  // device-side slots on the copy stream meanwhile (what the reference's producer threads do for its consumer)
  struct HostUpload {
    vectorCUDA<int> keys, off;
    vectorCUDA<float> feats;
    int batch = 0, rows = 0, maxSites = 0;
    cudaEvent_t keysDone = nullptr, featsDone = nullptr;
  } up[2];
  int upHead = 0, upTail = 0, upCount = 0;
  ~scn_net() {
    exchange.reset();
    for (HostUpload &u : up) {
      if (u.keysDone) cudaEventDestroy(u.keysDone);
      if (u.featsDone) cudaEventDestroy(u.featsDone);
    }
    if (copyDone) cudaEventDestroy(copyDone);
    if (copyStream) cudaStreamDestroy(copyStream);
  }
};

namespace {
thread_local std::string g_err;
struct Quiet { // the builders print the reference's architecture banner; keep harness runs silent
  std::streambuf *old;
  std::ostringstream sink;
  Quiet() : old(std::cout.rdbuf(sink.rdbuf())) {}
  ~Quiet() { std::cout.rdbuf(old); }
};
template <class F> int guarded(F f) {
  try { g_err.clear(); f(); return 0; }
  catch (const std::exception &e) { g_err = e.what(); return 1; }
  catch (...) { g_err = "unknown exception"; return 1; }
}
void describe(SpatiallySparseLayer *L, int *info, float *dropout) {
  int v[10] = {-1, 1, 1, 1, 0, 0, 1, 0, 0, 0};
  *dropout = 0;
  if (auto c = dynamic_cast<ConvolutionalLayer *>(L)) {
    int w[10] = {0, c->filterSize, c->filterStride, c->minActiveInputs, c->nFeaturesIn, c->nFeaturesOut, c->nFeaturesOut / c->nFeaturesIn, 0, c->inSpatialSize, c->outSpatialSize};
    std::memcpy(v, w, sizeof(v));
  } else if (auto c = dynamic_cast<ConvolutionalTriangularLayer *>(L)) {
    int w[10] = {1, c->filterSize, c->filterStride, c->minActiveInputs, c->nFeaturesIn, c->nFeaturesOut, c->nFeaturesOut / c->nFeaturesIn, 0, c->inSpatialSize, c->outSpatialSize};
    std::memcpy(v, w, sizeof(v));
  } else if (auto n = dynamic_cast<NetworkInNetworkLayer *>(L)) {
    int w[10] = {2, 1, 1, 1, n->nFeaturesIn, n->nFeaturesOut, 1, (int)n->fn, 0, 0};
    std::memcpy(v, w, sizeof(v));
    *dropout = n->dropout;
  } else if (auto m = dynamic_cast<MaxPoolingLayer *>(L)) {
    int w[10] = {3, m->poolSize, m->poolStride, 1, 0, 0, m->sd, m->fusedLast ? 1 : 0, m->inSpatialSize, m->outSpatialSize};
    std::memcpy(v, w, sizeof(v));
  } else if (auto m = dynamic_cast<MaxPoolingTriangularLayer *>(L)) {
    int w[10] = {4, m->poolSize, m->poolStride, 1, 0, 0, m->S, 0, m->inSpatialSize, m->outSpatialSize};
    std::memcpy(v, w, sizeof(v));
  } else if (auto f = dynamic_cast<FractionalMaxPoolingLayerBase *>(L)) {
    int w[10] = {6, f->poolSize, 1, 1, 0, 0, f->sd, 0, f->inSpatialSize, f->outSpatialSize};
    std::memcpy(v, w, sizeof(v));
  } else if (auto t = dynamic_cast<TerminalPoolingLayer *>(L)) {
    int w[10] = {5, t->poolSize, 1, 1, 0, 0, 1, 0, t->inSpatialSize, t->outSpatialSize};
    std::memcpy(v, w, sizeof(v));
  } else if (auto x = dynamic_cast<IndexLearnerLayer *>(L)) {
    int w[10] = {7, 1, 1, 1, x->nFeaturesIn, x->nFeaturesOut, 1, (int)SOFTMAX, 0, 0};
    std::memcpy(v, w, sizeof(v));
  }
  std::memcpy(info, v, sizeof(v));
}
// Fill interface 0 of a batch from device arrays.
void adoptDeviceInput(SparseConvNetCUDA &cnn, SpatiallySparseBatch &b, int batch, int rows, int maxSites, const int *d_keys,
                      const int *d_off, const int *d_bg, const float *d_features) {
  cnn.prepareBatch(b);
  b.reset();
  b.type = UNLABELEDBATCH;
  b.batchSize = batch;
  SpatiallySparseBatchInterface &in = b.interfaces[0];
  in.nFeatures = cnn.nInputFeatures;
  in.spatialSize = cnn.inputSpatialSize;
  in.featuresPresent.hVector() = range(cnn.nInputFeatures);
  in.nSpatialSites = rows;
  in.maxSitesPerSample = maxSites;
  in.gridOwner = &in;
  cudaStream_t s = cnn.memStream.stream;
  // no copies: the interface reads the caller's arrays (which must stay as they are until the forward has run)
  (void)s;
  in.siteKeys.borrowDevice(const_cast<int *>(d_keys), rows);
  in.sampleOffsets.borrowDevice(const_cast<int *>(d_off), batch + 1);
  in.backgroundRows.borrowDevice(const_cast<int *>(d_bg), batch);
  in.sub->features.borrowDevice(const_cast<float *>(d_features), rows * cnn.nInputFeatures);
}
// Interface 0 of the network's first pool slot filled from host arrays (pinned ones are copied from where they lie,
// pageable ones through the stream's staging block); the features travel on a stream of their own.
SpatiallySparseBatch &uploadHostInput(scn_net *net, int batch, const int *keys, const int *off, const float *features, batchType type) {
  SparseConvNetCUDA &cnn = *net->cnn;
  if (batch < 1) throw ScnException("batch must be positive");
  SpatiallySparseBatch &b = cnn.batchPool[0];
  cnn.prepareBatch(b);
  b.reset();
  b.type = type;
  b.batchSize = batch;
  SpatiallySparseBatchInterface &in = b.interfaces[0];
  const int rows = off[batch];
  const int nF = cnn.nInputFeatures;
  in.nFeatures = nF;
  in.spatialSize = cnn.inputSpatialSize;
  in.featuresPresent.hVector() = range(nF);
  in.nSpatialSites = rows;
  in.gridOwner = &in;
  in.backpropErrors = false;
  const size_t kb = sizeof(int) * rows, ob = sizeof(int) * (batch + 1), fb = sizeof(float) * (size_t)rows * nF;
  auto pinned = [&](const void *p) {
    for (const void *k : net->knownPinned) if (k == p) return true;
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
    if (a.type != cudaMemoryTypeHost) return false;
    if (net->knownPinned.size() >= 64) net->knownPinned.clear();
    net->knownPinned.push_back(p);
    return true;
  };
  const void *sk = keys, *so = off, *sf = features;
  if (!(pinned(keys) && pinned(off) && pinned(features))) {
    char *stage = (char *)cnn.memStream.staging(kb + ob + fb);
    std::memcpy(stage, keys, kb);
    std::memcpy(stage + kb, off, ob);
    std::memcpy(stage + kb + ob, features, fb);
    sk = stage; so = stage + kb; sf = stage + kb + ob;
  }
  int maxRows = 0;
  for (int s = 0; s < batch; ++s) maxRows = std::max(maxRows, off[s + 1] - off[s]);
  in.maxSitesPerSample = maxRows; // an upper bound (exact when a sample has no background row)
  if (!cnn.layers.empty() && dynamic_cast<TerminalPoolingLayer *>(cnn.layers[0])) { // its rule width needs the exact count
    int most = 0;
    for (int s = 0; s < batch; ++s) { int n = 0; for (int r = off[s]; r < off[s + 1]; ++r) n += keys[r] >= 0; most = std::max(most, n); }
    in.maxSitesPerSample = most;
  }
  in.siteKeys.copyToGPU(); in.sampleOffsets.copyToGPU(); in.backgroundRows.copyToGPU(); in.sub->features.copyToGPU();
  in.siteKeys.resize(rows); in.sampleOffsets.resize(batch + 1); in.backgroundRows.resize(batch); in.sub->features.resize(rows * nF);
  cudaStream_t s = cnn.memStream.stream;
  if (rows) cudaSafeCall(cudaMemcpyAsync(in.siteKeys.dPtr(), sk, kb, cudaMemcpyHostToDevice, s));
  cudaSafeCall(cudaMemcpyAsync(in.sampleOffsets.dPtr(), so, ob, cudaMemcpyHostToDevice, s));
  if (!net->copyStream) {
    cudaSafeCall(cudaStreamCreateWithFlags(&net->copyStream, cudaStreamNonBlocking));
    cudaSafeCall(cudaEventCreateWithFlags(&net->copyDone, cudaEventDisableTiming));
  }
  if (rows) { // nothing is in flight on the features buffer: the previous batch ended with a host wait
    float *dst = in.sub->features.dPtr();
    cudaSafeCall(cudaEventRecord(net->copyDone, s)); // ... but the resize above may have enqueued work on s
    cudaSafeCall(cudaStreamWaitEvent(net->copyStream, net->copyDone, 0));
    cudaSafeCall(cudaMemcpyAsync(dst, sf, fb, cudaMemcpyHostToDevice, net->copyStream));
    cudaSafeCall(cudaEventRecord(net->copyDone, net->copyStream));
  }
  cnn.inputBackgroundPending = true; // found by the rule chain's kernel (or by a kernel of its own where that one does not apply)
  if (rows) cnn.inputReady = net->copyDone; // the layers (not the rule chain) wait for the features
  return b;
}
} // namespace

extern "C" {

const char *scn_net_last_error(void) { return g_err.c_str(); }

scn_net_t *scn_net_create(int dimension, int nInputFeatures, int nClasses, int nTop, int lattice, void *stream) {
  scn_net *n = nullptr;
  int rc = guarded([&] {
    Quiet q;
    n = new scn_net();
    n->lattice = lattice;
    n->last = nullptr;
    if (stream) n->cnn.reset(new SparseConvNetCUDA(dimension, nInputFeatures, nClasses, (cudaStream_t)stream, nTop, 2));
    else n->cnn.reset(new SparseConvNetCUDA(dimension, nInputFeatures, nClasses, -1, nTop, 2));
  });
  if (rc) { delete n; return nullptr; }
  return n;
}
void scn_net_destroy(scn_net_t *net) { delete net; }

int scn_net_addLeNetLayerMP(scn_net_t *net, int nFeatures, int fs, int fstride, int ps, int pstride, int act, float dropout, int minActive) {
  return guarded([&] {
    Quiet q;
    if (net->lattice == 0) net->cnn->addLeNetLayerMP(nFeatures, fs, fstride, ps, pstride, (ActivationFunction)act, dropout, minActive);
    else net->cnn->addTriangularLeNetLayerMP(nFeatures, fs, fstride, ps, pstride, (ActivationFunction)act, dropout, minActive);
  });
}
int scn_net_addLeNetLayerFMP(scn_net_t *net, int kind, int nFeatures, int fs, int fstride, int ps, float fmpShrink, int act, float dropout,
                             int minActive) {
  return guarded([&] {
    Quiet q;
    if (net->lattice != 0) throw ScnException("fractional max-pooling exists on the square lattice only");
    SparseConvNetCUDA &c = *net->cnn;
    ActivationFunction a = (ActivationFunction)act;
    switch (kind) {
    case 0: c.addLeNetLayerPOFMP(nFeatures, fs, fstride, ps, fmpShrink, a, dropout, minActive); break;
    case 1: c.addLeNetLayerPDFMP(nFeatures, fs, fstride, ps, fmpShrink, a, dropout, minActive); break;
    case 2: c.addLeNetLayerROFMP(nFeatures, fs, fstride, ps, fmpShrink, a, dropout, minActive); break;
    case 3: c.addLeNetLayerRDFMP(nFeatures, fs, fstride, ps, fmpShrink, a, dropout, minActive); break;
    default: throw ScnException("unknown fractional max-pooling kind");
    }
  });
}
int scn_net_set_pool_fusion(scn_net_t *net, int on) {
  return guarded([&] {
    auto &L = net->cnn->layers;
    for (size_t i = 2; i < L.size(); ++i) {
      auto conv = dynamic_cast<ConvolutionalLayer *>(L[i - 2]);
      auto nin = dynamic_cast<NetworkInNetworkLayer *>(L[i - 1]);
      auto pool = dynamic_cast<MaxPoolingLayer *>(L[i]);
      if (!conv || !nin || !pool) continue;
      const int cells = pool->sd;
      nin->fusePoolNext = on && pool->poolSize == pool->poolStride && cells >= 2 && cells <= 32 && (cells & (cells - 1)) == 0;
    }
  });
}
int scn_net_seed_fmp(scn_net_t *net, unsigned seed) {
  return guarded([&] {
    for (size_t l = 0; l < net->cnn->layers.size(); ++l)
      if (auto f = dynamic_cast<FractionalMaxPoolingLayerBase *>(net->cnn->layers[l])) f->rng.gen.seed(seed + (unsigned)l);
  });
}
int scn_net_addTerminalPoolingLayer(scn_net_t *net, int poolSize) {
  return guarded([&] {
    Quiet q;
    int S = net->lattice == 0 ? ipow(poolSize, net->cnn->dimension) : triangleSize(poolSize, net->cnn->dimension);
    net->cnn->addTerminalPoolingLayer(poolSize, S);
  });
}
int scn_net_addSoftmaxLayer(scn_net_t *net) { return guarded([&] { Quiet q; net->cnn->addSoftmaxLayer(); }); }
int scn_net_addIndexLearnerLayer(scn_net_t *net) { return guarded([&] { Quiet q; net->cnn->addIndexLearnerLayer(); }); }

scn_net_t *scn_net_DeepCNet(int dimension, int l, int k, int fn, int nInputFeatures, int nClasses, float p, int nTop, void *stream) {
  scn_net_t *n = scn_net_create(dimension, nInputFeatures, nClasses, nTop, 0, stream);
  if (!n) return nullptr;
  int rc = guarded([&] {
    Quiet q; // the call sequence of DeepCNet::DeepCNet
    for (int i = 0; i <= l; ++i)
      n->cnn->addLeNetLayerMP((i + 1) * k, i == 0 ? 3 : 2, 1, i < l ? 3 : 1, i < l ? 2 : 1, (ActivationFunction)fn, p * i * 1.0f / l);
    n->cnn->addSoftmaxLayer();
  });
  if (rc) { scn_net_destroy(n); return nullptr; }
  return n;
}

scn_net_t *scn_net_named(const char *name, int dimension, int l, int k, float fmpShrink, int fn, int nInputFeatures, int nClasses, float p,
                         int nTop) {
  scn_net *n = nullptr;
  int rc = guarded([&] {
    Quiet q;
    const std::string s(name ? name : "");
    const ActivationFunction a = (ActivationFunction)fn;
    std::unique_ptr<SparseConvNet> net; // constructed as a caller of the class would; its runtime then moves into the handle
    if (s == "DeepCNet") net.reset(new DeepCNet(dimension, l, k, a, nInputFeatures, nClasses, p, -1, nTop));
    else if (s == "DeepC2") net.reset(new DeepC2(dimension, l, k, a, nInputFeatures, nClasses, p, -1, nTop));
    else if (s == "DeepCNiN") net.reset(new DeepCNiN(dimension, l, k, a, nInputFeatures, nClasses, p, -1, nTop));
    else if (s == "DeepC2C2") net.reset(new DeepC2C2(dimension, l, k, a, nInputFeatures, nClasses, p, -1, nTop));
    else if (s == "DeepC3C3Valid") net.reset(new DeepC3C3Valid(dimension, l, k, a, nInputFeatures, nClasses, p, -1, nTop));
    else if (s == "DeepC3C3") net.reset(new DeepC3C3(dimension, l, k, a, nInputFeatures, nClasses, p, -1, nTop));
    else if (s == "POFMPSparseConvNet") net.reset(new POFMPSparseConvNet(dimension, l, k, fmpShrink, a, nInputFeatures, nClasses, p, -1, nTop));
    else if (s == "ROFMPSparseConvNet") net.reset(new ROFMPSparseConvNet(dimension, l, k, fmpShrink, a, nInputFeatures, nClasses, p, -1, nTop));
    else if (s == "PDFMPSparseConvNet") net.reset(new PDFMPSparseConvNet(dimension, l, k, fmpShrink, a, nInputFeatures, nClasses, p, -1, nTop));
    else if (s == "RDFMPSparseConvNet") net.reset(new RDFMPSparseConvNet(dimension, l, k, fmpShrink, a, nInputFeatures, nClasses, p, -1, nTop));
    else throw ScnException("unknown architecture name '" + s + "'");
    n = new scn_net();
    n->lattice = 0;
    n->last = nullptr;
    n->cnn = std::move(net->cnn);
  });
  if (rc) { delete n; return nullptr; }
  return n;
}

int scn_net_n_layers(scn_net_t *net) { return (int)net->cnn->layers.size(); }
int scn_net_input_spatial_size(scn_net_t *net) { return net->cnn->inputSpatialSize; }
int scn_net_layer_info(scn_net_t *net, int layer, int *info, float *dropout) {
  return guarded([&] {
    if (layer < 0 || layer >= (int)net->cnn->layers.size()) throw ScnException("layer index out of range");
    describe(net->cnn->layers[layer], info, dropout);
  });
}
int scn_net_set_weights(scn_net_t *net, int layer, const float *W, const float *B, const float *prelu) {
  return guarded([&] {
    auto n = dynamic_cast<NetworkInNetworkLayer *>(net->cnn->layers.at(layer));
    if (!n) throw ScnException("layer has no weights");
    std::vector<float> &w = n->W.hVector(), &b = n->B.hVector();
    std::memcpy(w.data(), W, sizeof(float) * w.size());
    std::memcpy(b.data(), B, sizeof(float) * b.size());
    if (auto pr = dynamic_cast<NetworkInNetworkPReLULayer *>(n)) {
      if (prelu) { std::vector<float> &s = pr->PReLU.hVector(); std::memcpy(s.data(), prelu, sizeof(float) * s.size()); }
    }
    n->weightsChanged();
  });
}
int scn_net_load_weights(scn_net_t *net, const char *base, int epoch) { return guarded([&] { Quiet q; net->cnn->loadWeights(base, epoch, false); }); }
int scn_net_save_weights(scn_net_t *net, const char *base, int epoch) { return guarded([&] { net->cnn->saveWeights(base, epoch, false); }); }
int scn_net_set_precision(scn_net_t *net, int precision) {
  return guarded([&] {
    if (precision < SCN_PREC_AUTO || precision > SCN_PREC_SPLIT) throw ScnException("unknown precision");
    for (auto L : net->cnn->layers)
      if (auto n = dynamic_cast<NetworkInNetworkLayer *>(L)) { n->precision = precision; n->precisionFallback = true; }
  });
}

namespace {
void deliverExchange(ResultExchange &ex, bool any, float *gathered, int *rows) {
  if (any) { ex.deliver(gathered, rows); return; }
  for (int r = 0; r < ex.world && rows; ++r) rows[r] = -1; // nothing had been published before this step
}
// Rule chain, layers and the one copy-and-wait that ends a step, for a batch whose input interface is filled (its
// copies may still be on their way: the stream and the layers wait for them where they need them).  processBatch
// without the per-sample vectors of SpatiallySparseBatch: the results go straight to the caller's arrays.  With
// `exchange` the step's probabilities also go to the other ranks and theirs of the step before come back.
void runHostBatch(scn_net *net, SpatiallySparseBatch &b, int batch, float *probs, int *predictions, bool exchange, float *gathered_prev,
                  int *rows_prev) {
  SparseConvNetCUDA &cnn = *net->cnn;
  if (exchange && (!net->exchange || !net->exchange->connected())) throw ScnException("no connected exchange (scn_net_exchange_create / _connect)");
  cnn.earlyFirstLayer = true; // one batch in flight here: the first layer may start behind the rule chain
  cnn.preprocessBatchOnDevice(b); // waits once, after the key upload and the rule chain
  cnn.earlyFirstLayer = false;
  cnn.forwardLayers(b);
  net->last = &b;
  SpatiallySparseBatchInterface &topI = b.interfaces.back();
  if (batch != topI.nSpatialSites) throw ScnException("the top layer must hold one row per sample");
  bool any = false;
  if (exchange) {
    // the step before: every rank published it at the end of its previous call, so this wait is over at once unless a
    // rank has fallen a whole step behind; then this step's block goes out.  Both ride in front of the one copy + wait
    // that ends the step.
    ResultExchange &ex = *net->exchange;
    any = ex.published > 0;
    cudaStream_t s = cnn.memStream.stream;
    ex.step(topI.sub->features.dPtr(), batch, s);
    if (any) ex.copyBlockToHost(s);
  }
  const char *block = fetchClassifierResult(topI, batch, cnn.nTop, cnn.memStream);
  const size_t pb = sizeof(float) * (size_t)batch * cnn.nClasses;
  if (probs) std::memcpy(probs, block, pb);
  if (predictions) std::memcpy(predictions, block + pb, sizeof(int) * (size_t)batch * cnn.nTop);
  if (exchange) deliverExchange(*net->exchange, any, gathered_prev, rows_prev);
}
} // namespace

int scn_net_forward_host(scn_net_t *net, int batch, const int *keys, const int *off, const float *features, float *probs, int *predictions) {
  return guarded([&] {
    SpatiallySparseBatch &b = uploadHostInput(net, batch, keys, off, features, UNLABELEDBATCH);
    runHostBatch(net, b, batch, probs, predictions, false, nullptr, nullptr);
  });
}

int scn_net_forward_host_begin(scn_net_t *net, int batch, const int *keys, const int *off, const float *features) {
  return guarded([&] {
    SparseConvNetCUDA &cnn = *net->cnn;
    if (batch < 1) throw ScnException("batch must be positive");
    if (net->upCount == 2) throw ScnException("two batches are on their way already: take one with scn_net_forward_host_end first");
    scn_net::HostUpload &u = net->up[net->upHead];
    const int rows = off[batch], nF = cnn.nInputFeatures;
    int maxRows = 0;
    for (int s = 0; s < batch; ++s) maxRows = std::max(maxRows, off[s + 1] - off[s]);
    if (!cnn.layers.empty() && dynamic_cast<TerminalPoolingLayer *>(cnn.layers[0])) { // its rule width needs the exact count
      int most = 0;
      for (int s = 0; s < batch; ++s) { int n = 0; for (int r = off[s]; r < off[s + 1]; ++r) n += keys[r] >= 0; most = std::max(most, n); }
      maxRows = most;
    }
    u.batch = batch; u.rows = rows; u.maxSites = maxRows;
    u.keys.resize(rows); u.off.resize(batch + 1); u.feats.resize(rows * nF);
    if (!net->copyStream) {
      cudaSafeCall(cudaStreamCreateWithFlags(&net->copyStream, cudaStreamNonBlocking));
      cudaSafeCall(cudaEventCreateWithFlags(&net->copyDone, cudaEventDisableTiming));
    }
    if (!u.keysDone) {
      cudaSafeCall(cudaEventCreateWithFlags(&u.keysDone, cudaEventDisableTiming));
      cudaSafeCall(cudaEventCreateWithFlags(&u.featsDone, cudaEventDisableTiming));
    }
    // (the slot's buffers are idle: the batch that used them last ended with a host wait two calls ago; a resize may have
    // enqueued work on the network's stream, so the copies are ordered behind it)
    cudaStream_t cs = net->copyStream;
    cudaSafeCall(cudaEventRecord(net->copyDone, cnn.memStream.stream));
    cudaSafeCall(cudaStreamWaitEvent(cs, net->copyDone, 0));
    if (rows) cudaSafeCall(cudaMemcpyAsync(u.keys.dPtr(), keys, sizeof(int) * (size_t)rows, cudaMemcpyHostToDevice, cs));
    cudaSafeCall(cudaMemcpyAsync(u.off.dPtr(), off, sizeof(int) * (size_t)(batch + 1), cudaMemcpyHostToDevice, cs));
    cudaSafeCall(cudaEventRecord(u.keysDone, cs));
    if (rows) cudaSafeCall(cudaMemcpyAsync(u.feats.dPtr(), features, sizeof(float) * (size_t)rows * nF, cudaMemcpyHostToDevice, cs));
    cudaSafeCall(cudaEventRecord(u.featsDone, cs));
    net->upHead ^= 1;
    ++net->upCount;
  });
}

int scn_net_forward_host_end(scn_net_t *net, float *probs, int *predictions, float *gathered_prev, int *rows_prev) {
  return guarded([&] {
    SparseConvNetCUDA &cnn = *net->cnn;
    if (net->upCount == 0) throw ScnException("no batch is on its way (scn_net_forward_host_begin)");
    scn_net::HostUpload &u = net->up[net->upTail];
    net->upTail ^= 1;
    --net->upCount;
    SpatiallySparseBatch &b = cnn.batchPool[0];
    cnn.prepareBatch(b);
    b.reset();
    b.type = UNLABELEDBATCH;
    b.batchSize = u.batch;
    SpatiallySparseBatchInterface &in = b.interfaces[0];
    in.nFeatures = cnn.nInputFeatures;
    in.spatialSize = cnn.inputSpatialSize;
    in.featuresPresent.hVector() = range(cnn.nInputFeatures);
    in.nSpatialSites = u.rows;
    in.maxSitesPerSample = u.maxSites;
    in.gridOwner = &in;
    in.backpropErrors = false;
    in.backgroundRows.copyToGPU();
    in.backgroundRows.resize(u.batch);
    in.siteKeys.borrowDevice(u.keys.dPtr(), u.rows);
    in.sampleOffsets.borrowDevice(u.off.dPtr(), u.batch + 1);
    in.sub->features.borrowDevice(u.feats.dPtr(), u.rows * cnn.nInputFeatures);
    cudaSafeCall(cudaStreamWaitEvent(cnn.memStream.stream, u.keysDone, 0)); // the rule chain reads keys and offsets
    cnn.inputBackgroundPending = true;
    if (u.rows) cnn.inputReady = u.featsDone; // the layers wait for the features
    runHostBatch(net, b, u.batch, probs, predictions, gathered_prev != nullptr || rows_prev != nullptr, gathered_prev, rows_prev);
  });
}

int scn_net_exchange_create(scn_net_t *net, int world, int rank, int cap_rows, unsigned char *handle_out) {
  return guarded([&] {
    net->exchange.reset(new ResultExchange(world, rank, cap_rows, net->cnn->nClasses));
    if (handle_out) std::memcpy(handle_out, net->exchange->handle(), 64);
  });
}
void *scn_net_exchange_buffer(scn_net_t *net) { return net->exchange ? net->exchange->localBuffer() : nullptr; }
int scn_net_exchange_connect(scn_net_t *net, const unsigned char *handles) {
  return guarded([&] {
    if (!net->exchange) throw ScnException("no exchange (scn_net_exchange_create)");
    net->exchange->connect(handles);
  });
}
int scn_net_exchange_connect_local(scn_net_t *net, void *const *buffers) {
  return guarded([&] {
    if (!net->exchange) throw ScnException("no exchange (scn_net_exchange_create)");
    net->exchange->connectLocal(buffers);
  });
}
int scn_net_exchange_destroy(scn_net_t *net) { return guarded([&] { net->exchange.reset(); }); }

int scn_net_forward_host_exchange(scn_net_t *net, int batch, const int *keys, const int *off, const float *features, float *probs, int *predictions,
                                  float *gathered_prev, int *rows_prev) {
  return guarded([&] {
    if (!net->exchange || !net->exchange->connected()) throw ScnException("no connected exchange (scn_net_exchange_create / _connect)");
    SpatiallySparseBatch &b = uploadHostInput(net, batch, keys, off, features, UNLABELEDBATCH);
    runHostBatch(net, b, batch, probs, predictions, true, gathered_prev, rows_prev);
  });
}

int scn_net_exchange_flush(scn_net_t *net, float *gathered, int *rows) {
  return guarded([&] {
    if (!net->exchange || !net->exchange->connected()) throw ScnException("no connected exchange");
    ResultExchange &ex = *net->exchange;
    cudaStream_t s = net->cnn->memStream.stream;
    const bool any = ex.published > 0;
    ex.step(nullptr, 0, s);
    if (any) ex.copyBlockToHost(s);
    cudaSafeCall(cudaStreamSynchronize(s));
    deliverExchange(ex, any, gathered, rows);
  });
}

int scn_net_exchange_step_device(scn_net_t *net, const float *d_probs, int rows, float *d_gathered_prev, int *d_rows_status_prev) {
  return guarded([&] {
    if (!net->exchange || !net->exchange->connected()) throw ScnException("no connected exchange");
    ResultExchange &ex = *net->exchange;
    cudaStream_t s = net->cnn->memStream.stream;
    if ((d_gathered_prev == nullptr) != (d_rows_status_prev == nullptr)) throw ScnException("pass both result arrays or neither");
    ex.stepBeside(d_probs, rows, s, d_gathered_prev, d_rows_status_prev);
  });
}

int scn_net_train_batch(scn_net_t *net, int batch, const int *keys, const int *off, const float *features, const int *labels, float learningRate,
                        float momentum, float *probs, double *stats) {
  return guarded([&] {
    SparseConvNetCUDA &cnn = *net->cnn;
    if (!labels) throw ScnException("a training step needs labels");
    SpatiallySparseBatch &b = uploadHostInput(net, batch, keys, off, features, TRAINBATCH);
    b.labels.copyToCPU();
    b.labels.hVector().assign(labels, labels + batch);
    cnn.preprocessBatchOnDevice(b);
    std::ofstream nof, nog;
    cnn.processBatch(b, learningRate, momentum, nof, nog);
    net->last = &b;
    cudaSafeCall(cudaStreamSynchronize(cnn.memStream.stream));
    for (int i = 0; i < batch && probs; ++i) std::memcpy(probs + (size_t)i * cnn.nClasses, b.probabilities[i].data(), sizeof(float) * cnn.nClasses);
    if (stats) { stats[0] = b.negativeLogLikelihood; stats[1] = b.mistakes; }
  });
}

int scn_net_set_dropout_features(scn_net_t *net, int layer, const int *present, int n) {
  return guarded([&] {
    auto l = dynamic_cast<NetworkInNetworkLayer *>(net->cnn->layers.at(layer));
    if (!l) throw ScnException("layer has no weights");
    if (n < 0 || n > l->nFeaturesOut || (n && !present)) throw ScnException("bad feature subset");
    l->forcedPresent.assign(present, present + n);
  });
}

int scn_net_iface_present(scn_net_t *net, int i, int *present) {
  int n = -1;
  guarded([&] {
    if (!net->last) throw ScnException("no batch has run");
    SpatiallySparseBatchInterface &I = net->last->interfaces.at(i);
    if (I.presentMask.size() == 0) {
      n = I.nFeatures;
      for (int f = 0; f < n && present; ++f) present[f] = f;
    } else {
      n = (int)I.presentSubset.size();
      if (present) std::copy(I.presentSubset.begin(), I.presentSubset.end(), present);
    }
  });
  return n;
}

int scn_net_index_learner_batch(scn_net_t *net, int batch, const int *keys, const int *off, const float *features, const int *sample_numbers,
                                float learningRate, float momentum, float *probs, double *stats) {
  return guarded([&] {
    SparseConvNetCUDA &cnn = *net->cnn;
    if (!sample_numbers) throw ScnException("an index-learning step needs the pictures' numbers in the data set");
    SpatiallySparseBatch &b = uploadHostInput(net, batch, keys, off, features, TRAINBATCH);
    b.sampleNumbers.assign(sample_numbers, sample_numbers + batch);
    cnn.preprocessBatchOnDevice(b);
    std::ofstream nof;
    cnn.processIndexLearnerBatch(b, learningRate, momentum, nof);
    net->last = &b;
    cudaSafeCall(cudaStreamSynchronize(cnn.memStream.stream));
    for (int i = 0; i < batch && probs; ++i) std::memcpy(probs + (size_t)i * batch, b.probabilities[i].data(), sizeof(float) * batch);
    if (stats) { stats[0] = b.negativeLogLikelihood; stats[1] = b.mistakes; }
  });
}

int scn_net_rescale_batch(scn_net_t *net, int batch, const int *keys, const int *off, const float *features) {
  return guarded([&] {
    Quiet q; // (every learnt layer prints its featureScale line, as the reference does)
    SparseConvNetCUDA &cnn = *net->cnn;
    SpatiallySparseBatch &b = uploadHostInput(net, batch, keys, off, features, RESCALEBATCH);
    cnn.preprocessBatchOnDevice(b);
    std::ofstream nof, nog;
    cnn.processBatch(b, 0.f, 0.f, nof, nog);
    net->last = &b;
    cudaSafeCall(cudaStreamSynchronize(cnn.memStream.stream));
  });
}

int scn_net_get_weights(scn_net_t *net, int layer, float *W, float *B, float *prelu) {
  return guarded([&] {
    auto fetch = [&](vectorCUDA<float> &v, float *dst) {
      if (!dst || !v.size()) return;
      if (v.onGPU) cudaSafeCall(cudaMemcpy(dst, v.dPtr(), sizeof(float) * v.size(), cudaMemcpyDeviceToHost));
      else std::memcpy(dst, v.hVector().data(), sizeof(float) * v.size());
    };
    cudaSafeCall(cudaStreamSynchronize(net->cnn->memStream.stream));
    if (auto x = dynamic_cast<IndexLearnerLayer *>(net->cnn->layers.at(layer))) { fetch(x->W, W); return; } // (no bias)
    auto n = dynamic_cast<NetworkInNetworkLayer *>(net->cnn->layers.at(layer));
    if (!n) throw ScnException("layer has no weights");
    fetch(n->W, W);
    fetch(n->B, B);
    if (auto pr = dynamic_cast<NetworkInNetworkPReLULayer *>(n)) fetch(pr->PReLU, prelu);
  });
}

long long scn_net_iface_dfeatures(scn_net_t *net, int i, float *dfeatures) {
  long long n = -1;
  guarded([&] {
    if (!net->last) throw ScnException("no batch has run");
    SpatiallySparseBatchInterface &I = net->last->interfaces.at(i);
    cudaSafeCall(cudaStreamSynchronize(net->cnn->memStream.stream));
    n = I.sub->dfeatures.size();
    if (dfeatures && n) cudaSafeCall(cudaMemcpy(dfeatures, I.sub->dfeatures.dPtr(), sizeof(float) * n, cudaMemcpyDeviceToHost));
  });
  return n;
}

int scn_net_forward_device(scn_net_t *net, int batch, int rows, int maxSites, const int *d_keys, const int *d_off, const int *d_bg,
                           const float *d_features, float *d_probs, int *d_top) {
  return guarded([&] {
    SparseConvNetCUDA &cnn = *net->cnn;
    SpatiallySparseBatch &b = cnn.batchPool[0];
    adoptDeviceInput(cnn, b, batch, rows, maxSites, d_keys, d_off, d_bg, d_features);
    cnn.earlyFirstLayer = true; // one batch in flight here: the first layer may start behind the rule chain
    cnn.preprocessBatchOnDevice(b);
    cnn.earlyFirstLayer = false;
    cnn.forwardLayers(b);
    net->last = &b;
    SpatiallySparseBatchInterface &topI = b.interfaces.back();
    cudaStream_t s = cnn.memStream.stream;
    if (d_probs) cudaSafeCall(cudaMemcpyAsync(d_probs, topI.sub->features.dPtr(), sizeof(float) * (size_t)batch * cnn.nClasses, cudaMemcpyDeviceToDevice, s));
    if (d_top) scnSafeCall(scn_top_indices(topI.sub->features.dPtr(), batch, cnn.nClasses, cnn.nTop, d_top, s));
  });
}

int scn_net_copy_probs_device(scn_net_t *net, float *d_probs) {
  return guarded([&] {
    if (!net->last) throw ScnException("no forward has run");
    SpatiallySparseBatchInterface &topI = net->last->interfaces.back();
    const size_t n = (size_t)topI.nSpatialSites * topI.nFeatures;
    if (topI.sub->features.size() != n) throw ScnException("probabilities are no longer resident");
    cudaSafeCall(cudaMemcpyAsync(d_probs, topI.sub->features.dPtr(), sizeof(float) * n, cudaMemcpyDeviceToDevice, net->cnn->memStream.stream));
  });
}

int scn_net_iface_sizes(scn_net_t *net, int i, long long *sizes) {
  return guarded([&] {
    if (!net->last) throw ScnException("no forward has run");
    SpatiallySparseBatchInterface &I = net->last->interfaces.at(i);
    sizes[0] = I.nSpatialSites; sizes[1] = I.nFeatures; sizes[2] = I.spatialSize; sizes[3] = I.rules.size();
    bool pools = i > 0 && (dynamic_cast<MaxPoolingLayer *>(net->cnn->layers[i - 1]) || dynamic_cast<MaxPoolingTriangularLayer *>(net->cnn->layers[i - 1]) ||
                           dynamic_cast<FractionalMaxPoolingLayerBase *>(net->cnn->layers[i - 1]));
    sizes[4] = pools ? (long long)I.nSpatialSites * I.nFeatures : 0;
  });
}
// Interfaces behind layer i share sub-interface i across batches, so this is only valid
// until the next forward.
int scn_net_iface_fetch(scn_net_t *net, int i, float *features, int *rules, int *choices, int *rowKeys) {
  return guarded([&] {
    if (!net->last) throw ScnException("no forward has run");
    SpatiallySparseBatchInterface &I = net->last->interfaces.at(i);
    cudaSafeCall(cudaStreamSynchronize(net->cnn->memStream.stream));
    if (features) {
      if (I.deferredFrom) throw ScnException("this interface's gather is fused into the next layer and was never materialised");
      if (I.deferredLearnt) throw ScnException("this interface's learnt layer is fused into the pooling layer behind it and was never materialised");
      size_t n = (size_t)I.nSpatialSites * I.nFeatures;
      if (I.sub->features.size() != n) throw ScnException("interface features are no longer resident");
      if (n) cudaSafeCall(cudaMemcpy(features, I.sub->features.dPtr(), sizeof(float) * n, cudaMemcpyDeviceToHost));
    }
    if (rules && I.rules.size()) cudaSafeCall(cudaMemcpy(rules, I.rules.dPtr(), sizeof(int) * I.rules.size(), cudaMemcpyDeviceToHost));
    if (choices) {
      size_t n = (size_t)I.nSpatialSites * I.nFeatures;
      if (I.sub->poolingChoices.size() != n) throw ScnException("interface has no pooling choices");
      if (n) cudaSafeCall(cudaMemcpy(choices, I.sub->poolingChoices.dPtr(), sizeof(int) * n, cudaMemcpyDeviceToHost));
    }
    if (rowKeys && I.nSpatialSites) {
      SpatiallySparseBatchInterface *g = I.gridOwner;
      cudaSafeCall(cudaMemcpy(rowKeys, g->siteKeys.dPtr(), sizeof(int) * I.nSpatialSites, cudaMemcpyDeviceToHost));
    }
  });
}

double scn_net_take_multiply_adds(void) {
  double v = (double)multiplyAddCount;
  multiplyAddCount = 0;
  return v;
}
int scn_net_enable_timing(scn_net_t *net, int on) { return guarded([&] { net->cnn->enableTiming(on != 0); }); }
int scn_net_layer_times(scn_net_t *net, float *ms) {
  return guarded([&] {
    std::vector<float> t = net->cnn->layerTimes();
    std::memcpy(ms, t.data(), sizeof(float) * t.size());
  });
}

int scn_net_process_dataset(scn_net_t *net, int nSamples, const int *keys, const int *off, const float *features, const int *labels,
                            int batchSize, float *errorRate, float *probs) {
  return guarded([&] {
    Quiet q;
    SparseConvNetCUDA &cnn = *net->cnn;
    const int nF = cnn.nInputFeatures;
    std::vector<std::unique_ptr<SitesPicture>> pics;
    SpatiallySparseDataset ds;
    ds.name = "synthetic"; ds.nFeatures = nF; ds.nClasses = cnn.nClasses; ds.type = labels ? TESTBATCH : UNLABELEDBATCH;
    for (int s = 0; s < nSamples; ++s) {
      bool bg = false;
      for (int r = off[s]; r < off[s + 1]; ++r) bg = bg || keys[r] < 0;
      pics.emplace_back(new SitesPicture(nF, labels ? labels[s] : -1, bg));
      for (int r = off[s]; r < off[s + 1]; ++r) {
        if (keys[r] < 0) continue;
        pics.back()->keys.push_back(keys[r]);
        pics.back()->features.insert(pics.back()->features.end(), features + (size_t)r * nF, features + (size_t)(r + 1) * nF);
      }
      ds.pictures.push_back(pics.back().get());
    }
    // the loop of SparseConvNetCUDA::processDataset, keeping each batch's probabilities
    BatchProducer bp(cnn, ds, cnn.inputSpatialSize, batchSize);
    std::ofstream nof, nog;
    float err = 0;
    size_t at = 0;
    while (SpatiallySparseBatch *b = bp.nextBatch()) {
      cnn.processBatch(*b, 0, 0, nof, nog);
      err += b->mistakes * 1.0f / nSamples;
      for (int i = 0; i < b->batchSize; ++i, ++at)
        if (probs) std::memcpy(probs + at * cnn.nClasses, b->probabilities[i].data(), sizeof(float) * cnn.nClasses);
    }
    if (errorRate) *errorRate = err;
  });
}

int scn_host_vectorTopIndices(const float *v, int n, int k, int *out) {
  return guarded([&] {
    std::vector<float> t(v, v + n);
    std::vector<int> r = vectorTopIndices(t, k);
    std::memcpy(out, r.data(), sizeof(int) * k);
  });
}
}
