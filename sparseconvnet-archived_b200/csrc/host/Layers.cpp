// Geometry layers and the learnt layers: host-side bookkeeping around the C ABI calls.
#include <climits>
#include "Regions.h"
#include <cmath>
#include <cstring>
#include <random>
#include "ConvolutionalLayer.h"
#include "ConvolutionalTriangularLayer.h"
#include "IndexLearnerLayer.h"
#include "MaxPoolingLayer.h"
#include "MaxPoolingTriangularLayer.h"
#include "NetworkInNetworkLayer.h"
#include "NetworkInNetworkPReLULayer.h"
#include "RuleChain.h"
#include "SigmoidLayer.h"
#include "SoftmaxClassifier.h"
#include "TerminalPoolingLayer.h"

using rulechain::preprocessNow;

namespace {
// Every batch type runs the same forward kernels (a TRAINBATCH of a layer with dropout zeroes the dropped features behind them).
void requireInference(const SpatiallySparseBatch &) {}
// The 0/1 mask (one float per feature, on the device) of the features a training batch keeps at `iface`, or nullptr if it
// keeps them all: the mask of the nearest learnt layer's output at or below it.  The layers in between copy features
// through (a convolution: `copies` times, so masks apply with the period of their own length).
const float *presentMaskAt(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &iface, int &period) {
  SpatiallySparseBatchInterface *first = batch.interfaces.data();
  for (SpatiallySparseBatchInterface *i = &iface; i >= first && i < first + batch.interfaces.size(); --i) {
    if (i->learntOutput || i == first) {
      period = (int)i->presentMask.size();
      return period ? i->presentMask.dPtr() : nullptr;
    }
  }
  period = 0;
  return nullptr;
}
// The split tensor-core precision (SCN_PREC_3XTF32 or SCN_PREC_SPLIT) a layer set to `precision` runs a batch of this type
// in, or -1 if it runs in another one.  Training steps use tf32 operands throughout: the bf16 operands that SCN_PREC_SPLIT
// gives layers with long K carry 16 mantissa bits per product, and a gradient that has gone through a whole forward and
// backward pass amplifies that about 250 times.
int splitPrecision(int precision, const SpatiallySparseBatch &batch) {
  int p = precision == SCN_PREC_AUTO ? scn_conv_auto_precision() : precision;
  if (p == SCN_PREC_SPLIT && batch.type == TRAINBATCH) p = SCN_PREC_3XTF32;
  return (p == SCN_PREC_3XTF32 || p == SCN_PREC_SPLIT) ? p : -1;
}
// Zeroed device vector of n elements.
void zeroed(vectorCUDA<float> &v, int n, cudaMemStream &ms) {
  v.copyToGPU();
  v.resize(n);
  if (n) cudaSafeCall(cudaMemsetAsync(v.dPtr(), 0, sizeof(float) * (size_t)n, ms.stream));
}
// Shared body of the four region layers' finishRules().
void finishGeometry(const scn_regions_t &R, SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                    SpatiallySparseBatchInterface &output, int nFeaturesOut, int copies, const int *h) {
  output.nFeatures = nFeaturesOut;
  output.spatialSize = R.nOut;
  output.backpropErrors = input.backpropErrors;
  rulechain::finishRegions(R, output, h);
  if (copies > 1) {
    output.featuresPresent.copyToCPU();
    rulechain::convolutionFeaturesPresent(input.featuresPresent.hVector(), output.featuresPresent.hVector(), input.nFeatures,
                                          (int)input.featuresPresent.size(), copies);
  } else {
    output.featuresPresent.hVector() = input.featuresPresent.hVector();
  }
  (void)batch;
}
void checkSpatial(const SpatiallySparseBatchInterface &input, int inSpatialSize, const char *who) {
  if (input.spatialSize != inSpatialSize)
    throw ScnException(std::string(who) + ": input spatial size " + std::to_string(input.spatialSize) + " but the layer expects " +
                       std::to_string(inSpatialSize) + " (call addSoftmaxLayer / calculateInputSpatialSize first)");
}
} // namespace

// ------------------------------------------------------------------ ConvolutionalLayer
ConvolutionalLayer::ConvolutionalLayer(cudaMemStream &memStream, int filterSize, int filterStride, int dimension, int nFeaturesIn,
                                       int minActiveInputs)
    : SpatiallySparseLayer(memStream), inSpatialSize(0), outSpatialSize(0), filterSize(filterSize), filterStride(filterStride),
      dimension(dimension), nFeaturesIn(nFeaturesIn), minActiveInputs(minActiveInputs), fuseWithNext(false) {
  changesGeometry = true;
  fs = ipow(filterSize, dimension);
  nFeaturesOut = fs * nFeaturesIn;
  std::cout << "Convolution " << filterSize << "^" << dimension << "x" << nFeaturesIn << "->" << nFeaturesOut;
  if (filterStride != 1) std::cout << " stride:" << filterStride;
  if (minActiveInputs != 1) std::cout << " minActiveInputs:" << minActiveInputs;
  std::cout << std::endl;
}
long long ConvolutionalLayer::enqueueRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                                           SpatiallySparseBatchInterface &output, long long rowsInBound, int *d_result) {
  requireInference(batch);
  if (input.nFeatures != nFeaturesIn) throw ScnException("ConvolutionalLayer: wrong number of input features");
  checkSpatial(input, inSpatialSize, "ConvolutionalLayer");
  scn_regions_t R = {SCN_LATTICE_SQUARE, dimension, inSpatialSize, outSpatialSize, filterSize, filterStride, minActiveInputs};
  output.nFeatures = nFeaturesOut; output.spatialSize = outSpatialSize; // known before any count is
  return rulechain::enqueueRegions(R, batch, input, output, rowsInBound, d_result, memStream);
}
void ConvolutionalLayer::finishRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                                     SpatiallySparseBatchInterface &output, const int *h) {
  scn_regions_t R = {SCN_LATTICE_SQUARE, dimension, inSpatialSize, outSpatialSize, filterSize, filterStride, minActiveInputs};
  finishGeometry(R, batch, input, output, nFeaturesOut, fs, h);
}
void ConvolutionalLayer::preprocess(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output) {
  preprocessNow(*this, batch, input, output);
}
void ConvolutionalLayer::forwards(SpatiallySparseBatch &, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output) {
  if (fuseWithNext) { // the NetworkInNetwork layer behind this one gathers inside its kernel
    output.deferredFrom = &input;
    output.deferredCells = fs;
    return;
  }
  output.sub->features.resize(output.nSpatialSites * output.featuresPresent.size());
  propForwardToMatrixMultiply(input.sub->features.dPtr(), output.sub->features.dPtr(), output.rules.dPtr(), output.nSpatialSites * fs,
                              input.featuresPresent.size(), memStream);
}
int ConvolutionalLayer::calculateInputSpatialSize(int outputSpatialSize) {
  outSpatialSize = outputSpatialSize;
  inSpatialSize = filterSize + (outputSpatialSize - 1) * filterStride;
  std::cout << "-(C" << filterSize;
  if (filterStride != 1) std::cout << "/" << filterStride;
  std::cout << ")-" << inSpatialSize;
  return inSpatialSize;
}
void propForwardToMatrixMultiply(float *inFeatures, float *outFeatures, int *rules, int count, int nIn, cudaMemStream &memStream) {
  scnSafeCall(scn_gather_forward(inFeatures, rules, count, nIn, outFeatures, memStream.stream));
}

// ------------------------------------------------------------------ ConvolutionalTriangularLayer
ConvolutionalTriangularLayer::ConvolutionalTriangularLayer(cudaMemStream &memStream, int filterSize, int filterStride, int dimension,
                                                           int nFeaturesIn, int minActiveInputs)
    : SpatiallySparseLayer(memStream), inSpatialSize(0), outSpatialSize(0), filterSize(filterSize), filterStride(filterStride),
      dimension(dimension), nFeaturesIn(nFeaturesIn), minActiveInputs(minActiveInputs), fuseWithNext(false) {
  changesGeometry = true;
  fs = triangleSize(filterSize, dimension);
  nFeaturesOut = fs * nFeaturesIn;
  std::cout << dimension << "D ConvolutionalTriangularLayer side-length=" << filterSize << " " << nFeaturesIn << "x" << fs << "->" << nFeaturesOut;
  if (filterStride > 1) std::cout << ", stride " << filterStride;
  if (minActiveInputs != 1) std::cout << " minActiveInputs:" << minActiveInputs;
  std::cout << std::endl;
}
long long ConvolutionalTriangularLayer::enqueueRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                                                     SpatiallySparseBatchInterface &output, long long rowsInBound, int *d_result) {
  requireInference(batch);
  if (input.nFeatures != nFeaturesIn) throw ScnException("ConvolutionalTriangularLayer: wrong number of input features");
  checkSpatial(input, inSpatialSize, "ConvolutionalTriangularLayer");
  scn_regions_t R = {SCN_LATTICE_TRIANGULAR, dimension, inSpatialSize, outSpatialSize, filterSize, filterStride, minActiveInputs};
  output.nFeatures = nFeaturesOut; output.spatialSize = outSpatialSize;
  return rulechain::enqueueRegions(R, batch, input, output, rowsInBound, d_result, memStream);
}
void ConvolutionalTriangularLayer::finishRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                                               SpatiallySparseBatchInterface &output, const int *h) {
  scn_regions_t R = {SCN_LATTICE_TRIANGULAR, dimension, inSpatialSize, outSpatialSize, filterSize, filterStride, minActiveInputs};
  finishGeometry(R, batch, input, output, nFeaturesOut, fs, h);
}
void ConvolutionalTriangularLayer::preprocess(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output) {
  preprocessNow(*this, batch, input, output);
}
void ConvolutionalTriangularLayer::forwards(SpatiallySparseBatch &, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output) {
  if (fuseWithNext) { output.deferredFrom = &input; output.deferredCells = fs; return; }
  output.sub->features.resize(output.nSpatialSites * output.featuresPresent.size());
  propForwardToMatrixMultiply(input.sub->features.dPtr(), output.sub->features.dPtr(), output.rules.dPtr(), output.nSpatialSites * fs,
                              input.featuresPresent.size(), memStream);
}
int ConvolutionalTriangularLayer::calculateInputSpatialSize(int outputSpatialSize) {
  outSpatialSize = outputSpatialSize;
  inSpatialSize = filterSize + (outputSpatialSize - 1) * filterStride;
  std::cout << "-(C" << filterSize;
  if (filterStride != 1) std::cout << "/" << filterStride;
  std::cout << ")-" << inSpatialSize;
  return inSpatialSize;
}

// ------------------------------------------------------------------ MaxPoolingLayer
void maxPool(float *g1, float *g2, int *rules, int count, int sd, int nOut, int *d_choice, cudaMemStream &memStream) {
  scnSafeCall(scn_maxpool_forward(g1, rules, count, sd, nOut, g2, d_choice, memStream.stream));
}
MaxPoolingLayer::MaxPoolingLayer(cudaMemStream &memStream, int poolSize, int poolStride, int dimension)
    : SpatiallySparseLayer(memStream), inSpatialSize(0), outSpatialSize(0), poolSize(poolSize), poolStride(poolStride), dimension(dimension) {
  changesGeometry = true;
  fusedLast = false; splitEvent = nullptr; splitRecorded = false;
  sd = ipow(poolSize, dimension);
  std::cout << "MaxPooling " << poolSize << " " << poolStride << std::endl;
}
long long MaxPoolingLayer::enqueueRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                                        SpatiallySparseBatchInterface &output, long long rowsInBound, int *d_result) {
  requireInference(batch);
  checkSpatial(input, inSpatialSize, "MaxPoolingLayer");
  scn_regions_t R = {SCN_LATTICE_SQUARE, dimension, inSpatialSize, outSpatialSize, poolSize, poolStride, 1};
  output.nFeatures = input.nFeatures; output.spatialSize = outSpatialSize;
  return rulechain::enqueueRegions(R, batch, input, output, rowsInBound, d_result, memStream);
}
void MaxPoolingLayer::finishRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                                  const int *h) {
  scn_regions_t R = {SCN_LATTICE_SQUARE, dimension, inSpatialSize, outSpatialSize, poolSize, poolStride, 1};
  finishGeometry(R, batch, input, output, input.nFeatures, 1, h);
}
void MaxPoolingLayer::preprocess(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output) {
  preprocessNow(*this, batch, input, output);
}
void MaxPoolingLayer::forwards(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output) {
  fusedLast = false; splitRecorded = false;
  if (input.deferredLearnt) { // convolution + learnt layer + this pooling as one kernel, if it takes the case
    NetworkInNetworkLayer *nin = input.deferredLearnt;
    SpatiallySparseBatchInterface &ninInput = *input.deferredLearntInput;
    if (poolSize == poolStride &&
        nin->forwardsPooled(batch, *ninInput.deferredFrom, ninInput, output, ninInput.deferredCells, sd, output.nSpatialSites, nullptr,
                            input.nSpatialSites)) {
      fusedLast = true;
      return;
    }
    input.deferredLearnt = nullptr; // not taken: materialise the learnt layer's output after all, then pool it
    input.sub->reset();
    nin->forwardsNow(batch, ninInput, input);
    if (splitEvent) { cudaSafeCall(cudaEventRecord(splitEvent, memStream.stream)); splitRecorded = true; }
  }
  const int n = output.nSpatialSites * output.featuresPresent.size();
  output.sub->poolingChoices.resize(n);
  output.sub->features.resize(n);
  maxPool(input.sub->features.dPtr(), output.sub->features.dPtr(), output.rules.dPtr(), output.nSpatialSites, sd,
          output.featuresPresent.size(), output.sub->poolingChoices.dPtr(), memStream);
}
int MaxPoolingLayer::calculateInputSpatialSize(int outputSpatialSize) {
  outSpatialSize = outputSpatialSize;
  inSpatialSize = poolSize + (outputSpatialSize - 1) * poolStride;
  std::cout << "-(MP" << poolSize;
  if (poolStride != poolSize) std::cout << "/" << poolStride;
  std::cout << ")-" << inSpatialSize;
  return inSpatialSize;
}

// ------------------------------------------------------------------ fractional max-pooling
FractionalMaxPoolingLayerBase::FractionalMaxPoolingLayerBase(cudaMemStream &memStream, int poolSize, float fmpShrink, int dimension,
                                                             const char *label, const char *tag)
    : SpatiallySparseLayer(memStream), inSpatialSize(0), outSpatialSize(0), poolSize(poolSize), dimension(dimension), fmpShrink(fmpShrink),
      ticks(false, 0), tag(tag) {
  changesGeometry = true;
  sd = ipow(poolSize, dimension);
  std::cout << label << " Fractional Max Pooling " << fmpShrink << " " << poolSize << std::endl;
}
// MaxPoolingLayer.cu:171-186 (and 232-247, 293-308, 354-369): per sample new regions from the layer's
// rng, then gridRules; here the tables of the whole batch go to the device and one build does all samples.
long long FractionalMaxPoolingLayerBase::enqueueRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                                                     SpatiallySparseBatchInterface &output, long long rowsInBound, int *d_result) {
  requireInference(batch);
  checkSpatial(input, inSpatialSize, "FractionalMaxPoolingLayer");
  output.nFeatures = input.nFeatures; output.spatialSize = outSpatialSize;
  std::vector<int> &t = ticks.hVector();
  t.clear();
  for (int item = 0; item < batch.batchSize; ++item) appendSampleTables(t);
  long long full = 1;
  for (int a = 0; a < dimension; ++a) full *= outSpatialSize;
  const long long bound = std::min(rowsInBound * sd, (long long)batch.batchSize * full) + batch.batchSize;
  if (bound * sd > INT_MAX || rowsInBound > INT_MAX) throw ScnException("rule build: more than 2^31 rule cells in one batch; use smaller batches");
  SpatiallySparseBatchInterface *g = input.gridOwner;
  output.gridOwner = &output;
  output.siteKeys.resize((int)bound);
  output.sampleOffsets.resize(batch.batchSize + 1);
  output.backgroundRows.resize(batch.batchSize);
  output.rules.resize((int)(bound * sd));
  const size_t wsBytes = scn_fmp_rules_workspace_bytes(dimension, inSpatialSize, outSpatialSize, poolSize, batch.batchSize, (int)rowsInBound);
  scnSafeCall(scn_fmp_rules_build(dimension, inSpatialSize, outSpatialSize, poolSize, overlapping() ? 1 : 0, batch.batchSize, ticks.dPtr(),
                                  g->siteKeys.dPtr(), g->sampleOffsets.dPtr(), g->backgroundRows.dPtr(), (int)rowsInBound,
                                  output.siteKeys.dPtr(), output.sampleOffsets.dPtr(), output.backgroundRows.dPtr(), output.rules.dPtr(),
                                  (int)bound, d_result, memStream.deviceScratch(wsBytes), wsBytes, memStream.stream));
  return bound;
}
void FractionalMaxPoolingLayerBase::finishRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                                                SpatiallySparseBatchInterface &output, const int *h) {
  scn_regions_t R = {SCN_LATTICE_SQUARE, dimension, poolSize, 1, poolSize, 1, 1}; // rule rows of poolSize^dimension cells
  finishGeometry(R, batch, input, output, input.nFeatures, 1, h);
  output.spatialSize = outSpatialSize;
}
void FractionalMaxPoolingLayerBase::preprocess(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                                               SpatiallySparseBatchInterface &output) {
  preprocessNow(*this, batch, input, output);
}
void FractionalMaxPoolingLayerBase::forwards(SpatiallySparseBatch &, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output) {
  const int n = output.nSpatialSites * output.featuresPresent.size();
  output.sub->poolingChoices.resize(n);
  output.sub->features.resize(n);
  maxPool(input.sub->features.dPtr(), output.sub->features.dPtr(), output.rules.dPtr(), output.nSpatialSites, sd,
          output.featuresPresent.size(), output.sub->poolingChoices.dPtr(), memStream);
}
// MaxPoolingLayer.cu:216-223: int * float, + 0.5, truncated; at least one larger than the output
int FractionalMaxPoolingLayerBase::calculateInputSpatialSize(int outputSpatialSize) {
  outSpatialSize = outputSpatialSize;
  inSpatialSize = outputSpatialSize * fmpShrink + 0.5;
  if (inSpatialSize == outputSpatialSize) inSpatialSize++;
  std::cout << "-(" << tag << ")-" << inSpatialSize;
  return inSpatialSize;
}
#define SCN_FMP_LAYER(CLASS, TICKS, LABEL, TAG, OVERLAP)                                                             \
  CLASS::CLASS(cudaMemStream &memStream, int poolSize, float fmpShrink, int dimension)                               \
      : FractionalMaxPoolingLayerBase(memStream, poolSize, fmpShrink, dimension, LABEL, TAG) {}                      \
  bool CLASS::overlapping() const { return OVERLAP; }                                                                \
  void CLASS::appendSampleTables(std::vector<int> &dst) {                                                            \
    FractionalPoolingRegions<TICKS> regions(inSpatialSize, outSpatialSize, dimension, poolSize, rng);                \
    regions.appendTables(dst);                                                                                       \
  }
SCN_FMP_LAYER(PseudorandomOverlappingFractionalMaxPoolingLayer, PseudorandomOverlappingFmpTicks, "Pseudorandom overlapping", "POFMP", true)
SCN_FMP_LAYER(PseudorandomNonOverlappingFractionalMaxPoolingLayer, PseudorandomNonOverlappingFmpTicks, "Pseudorandom non-overlapping", "PDFMP", false)
SCN_FMP_LAYER(RandomOverlappingFractionalMaxPoolingLayer, RandomOverlappingFmpTicks, "Random overlapping", "ROFMP", true)
SCN_FMP_LAYER(RandomNonOverlappingFractionalMaxPoolingLayer, RandomNonOverlappingFmpTicks, "Random non-overlapping", "RDFMP", false)
#undef SCN_FMP_LAYER

// ------------------------------------------------------------------ MaxPoolingTriangularLayer
MaxPoolingTriangularLayer::MaxPoolingTriangularLayer(cudaMemStream &memStream, int poolSize, int poolStride, int dimension)
    : SpatiallySparseLayer(memStream), inSpatialSize(0), outSpatialSize(0), poolSize(poolSize), poolStride(poolStride), dimension(dimension) {
  changesGeometry = true;
  S = triangleSize(poolSize, dimension);
  std::cout << dimension << "D MaxPoolingTriangularLayer side-length=" << poolSize << " volume=" << S << " stride " << poolStride << std::endl;
}
long long MaxPoolingTriangularLayer::enqueueRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                                                  SpatiallySparseBatchInterface &output, long long rowsInBound, int *d_result) {
  requireInference(batch);
  checkSpatial(input, inSpatialSize, "MaxPoolingTriangularLayer");
  scn_regions_t R = {SCN_LATTICE_TRIANGULAR, dimension, inSpatialSize, outSpatialSize, poolSize, poolStride, 1};
  output.nFeatures = input.nFeatures; output.spatialSize = outSpatialSize;
  return rulechain::enqueueRegions(R, batch, input, output, rowsInBound, d_result, memStream);
}
void MaxPoolingTriangularLayer::finishRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                                            SpatiallySparseBatchInterface &output, const int *h) {
  scn_regions_t R = {SCN_LATTICE_TRIANGULAR, dimension, inSpatialSize, outSpatialSize, poolSize, poolStride, 1};
  finishGeometry(R, batch, input, output, input.nFeatures, 1, h);
}
void MaxPoolingTriangularLayer::preprocess(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output) {
  preprocessNow(*this, batch, input, output);
}
void MaxPoolingTriangularLayer::forwards(SpatiallySparseBatch &, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output) {
  const int n = output.nSpatialSites * output.featuresPresent.size();
  output.sub->poolingChoices.resize(n);
  output.sub->features.resize(n);
  maxPool(input.sub->features.dPtr(), output.sub->features.dPtr(), output.rules.dPtr(), output.nSpatialSites, S,
          output.featuresPresent.size(), output.sub->poolingChoices.dPtr(), memStream);
}
int MaxPoolingTriangularLayer::calculateInputSpatialSize(int outputSpatialSize) {
  outSpatialSize = outputSpatialSize;
  inSpatialSize = poolSize + (outputSpatialSize - 1) * poolStride;
  std::cout << "-(MP" << poolSize;
  if (poolStride != poolSize) std::cout << "/" << poolStride;
  std::cout << ")-" << inSpatialSize;
  return inSpatialSize;
}

// ------------------------------------------------------------------ TerminalPoolingLayer
TerminalPoolingLayer::TerminalPoolingLayer(cudaMemStream &memStream, int poolSize, int S)
    : SpatiallySparseLayer(memStream), inSpatialSize(poolSize), outSpatialSize(1), poolSize(poolSize), S(S), dimension(2), widthBuilt(0) {
  changesGeometry = true;
  std::cout << "TerminalPooling " << poolSize << " " << S << std::endl;
}
// The rule width is max(1, largest site count of a sample) (TerminalPoolingLayer.cu:89-92),
// which the host may not know yet: build with a safe width now (the forward kernel stops at
// the first -1, so any width >= the true one gives the same means) and, if the exact width
// turns out smaller, rebuild to it in finishRules so `rules` has the reference's shape.
long long TerminalPoolingLayer::enqueueRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                                             SpatiallySparseBatchInterface &output, long long rowsInBound, int *d_result) {
  requireInference(batch);
  checkSpatial(input, inSpatialSize, "TerminalPoolingLayer");
  output.nFeatures = input.nFeatures; output.spatialSize = outSpatialSize;
  long long cells = 1;
  for (int a = 0; a < dimension; ++a) cells *= inSpatialSize;
  long long width = std::max<long long>(1, std::min(cells, rowsInBound));
  if (width * batch.batchSize > 0x7fffffffll) throw ScnException("TerminalPoolingLayer: rules too large");
  SpatiallySparseBatchInterface *g = input.gridOwner;
  output.gridOwner = &output;
  output.siteKeys.resize(batch.batchSize);
  output.sampleOffsets.resize(batch.batchSize + 1);
  output.backgroundRows.resize(batch.batchSize);
  output.rules.resize((int)(width * batch.batchSize));
  size_t wsBytes = scn_terminal_rules_workspace_bytes(dimension, inSpatialSize, batch.batchSize, (int)rowsInBound);
  void *ws = memStream.deviceScratch(wsBytes);
  scnSafeCall(scn_terminal_rules_build(dimension, inSpatialSize, batch.batchSize, g->siteKeys.dPtr(), g->sampleOffsets.dPtr(),
                                       g->backgroundRows.dPtr(), (int)rowsInBound, (int)width, output.siteKeys.dPtr(),
                                       output.sampleOffsets.dPtr(), output.backgroundRows.dPtr(), output.rules.dPtr(), d_result, ws,
                                       wsBytes, memStream.stream));
  widthBuilt = (int)width;
  return batch.batchSize;
}
void TerminalPoolingLayer::finishRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                                       const int *h) {
  if (h[2]) throw ScnException("terminal pooling rule build reported device error bits " + std::to_string(h[2]));
  output.nFeatures = input.nFeatures;
  output.featuresPresent.hVector() = input.featuresPresent.hVector();
  output.spatialSize = outSpatialSize;
  output.nSpatialSites = batch.batchSize;
  output.maxSitesPerSample = 1;
  output.backpropErrors = input.backpropErrors;
  const int exact = std::max(1, input.gridOwner->maxSitesPerSample);
  if (exact != widthBuilt) {
    SpatiallySparseBatchInterface *g = input.gridOwner;
    output.rules.resize(exact * batch.batchSize);
    size_t wsBytes = scn_terminal_rules_workspace_bytes(dimension, inSpatialSize, batch.batchSize, input.nSpatialSites);
    void *ws = memStream.deviceScratch(wsBytes);
    scnSafeCall(scn_terminal_rules_build(dimension, inSpatialSize, batch.batchSize, g->siteKeys.dPtr(), g->sampleOffsets.dPtr(),
                                         g->backgroundRows.dPtr(), input.nSpatialSites, exact, output.siteKeys.dPtr(),
                                         output.sampleOffsets.dPtr(), output.backgroundRows.dPtr(), output.rules.dPtr(),
                                         memStream.deviceResult(), ws, wsBytes, memStream.stream));
    widthBuilt = exact;
  }
}
void TerminalPoolingLayer::preprocess(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output) {
  preprocessNow(*this, batch, input, output);
}
void TerminalPoolingLayer::forwards(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output) {
  const int n = output.nSpatialSites * output.featuresPresent.size();
  output.sub->poolingChoices.resize(n);
  output.sub->features.resize(n);
  scnSafeCall(scn_terminal_pool_forward(input.sub->features.dPtr(), output.rules.dPtr(), output.nSpatialSites,
                                        output.rules.size() / batch.batchSize, output.featuresPresent.size(),
                                        output.sub->features.dPtr(), memStream.stream));
}
int TerminalPoolingLayer::calculateInputSpatialSize(int outputSpatialSize) {
  if (outputSpatialSize != 1) throw ScnException("TerminalPoolingLayer must produce a 1x1 grid");
  std::cout << "-(TP)-" << inSpatialSize;
  return inSpatialSize;
}

// ------------------------------------------------------------------ NetworkInNetworkLayer
NetworkInNetworkLayer::NetworkInNetworkLayer(cudaMemStream &memStream, cublasHandle_t &, int nFeaturesIn, int nFeaturesOut, float dropout,
                                             ActivationFunction fn, float alpha)
    : SpatiallySparseLayer(memStream), W(false, nFeaturesIn * nFeaturesOut), MW(false, 0), B(false, nFeaturesOut), MB(false, 0), fn(fn),
      nFeaturesIn(nFeaturesIn), nFeaturesOut(nFeaturesOut), dropout(dropout), precision(SCN_PREC_AUTO), fusePoolNext(false), precisionFallback(false), packedT(nullptr), packedTBytes(0), packed(nullptr),
      packedBytes(0), packedPrecision(-100), packedFs(0) {
  // uniform(+-sqrt(6/(nIn + nOut*alpha))) as NetworkInNetworkLayer.cu:135-137, from a fixed
  // seed (the reference seeds from the clock); real runs load weights.
  const float scale = std::pow(6.0f / (nFeaturesIn + nFeaturesOut * alpha), 0.5f);
  std::mt19937 gen(1234567u + 31u * nFeaturesIn + nFeaturesOut);
  std::uniform_real_distribution<float> u(-scale, scale);
  for (auto &w : W.hVector()) w = u(gen);
  B.setZero();
  std::cout << "Learn " << nFeaturesIn << "->" << nFeaturesOut << " dropout=" << dropout << " " << sigmoidNames[fn] << std::endl;
}
NetworkInNetworkLayer::~NetworkInNetworkLayer() {
  if (packed) cudaFree(packed);
  if (packedT) cudaFree(packedT);
}
float *NetworkInNetworkLayer::slopes() { return nullptr; }
float *NetworkInNetworkLayer::slopeGradient() { return nullptr; }
void NetworkInNetworkLayer::updateSlopes(float, float, const float *) {}
void NetworkInNetworkLayer::weightsChanged() { packedPrecision = -100; }
// NetworkInNetworkLayer.cu:203-220 (and NetworkInNetworkPReLULayer.cu:175-191, the same): after this layer's forwards on
// a RESCALEBATCH, weights and biases are scaled so that the mean absolute output moves towards 1 (by its -0.1th power)
// and the scale applied underneath is taken out of the weights again; the top layer is left at scale 1.
void NetworkInNetworkLayer::scaleWeights(SpatiallySparseBatchInterface &, SpatiallySparseBatchInterface &output, float &scalingUnderneath, bool topLayer) {
  if (output.sub->features.size() == 0) throw ScnException("scaleWeights: call after forwards() on a RESCALEBATCH");
  cudaSafeCall(cudaStreamSynchronize(memStream.stream));
  float scale = output.sub->features.meanAbs();
  if (scale != scale) throw ScnException("scaleWeights: the layer's output holds a NaN");
  std::cout << "featureScale:" << scale << std::endl;
  scale = topLayer ? 1.0f : std::pow(scale, -0.1f);
  W.multiplicativeRescale(scale / scalingUnderneath);
  B.multiplicativeRescale(scale);
  MW.multiplicativeRescale(scale / scalingUnderneath);
  MB.multiplicativeRescale(scale);
  scalingUnderneath = scale;
  weightsChanged();
}
const void *NetworkInNetworkLayer::packedWeights(int fs, int nIn, int prec) {
  if (prec == SCN_PREC_FP32) return nullptr;
  size_t need = scn_conv_packed_weight_bytes(nFeaturesIn, nFeaturesOut, prec);
  if (need == 0) return nullptr;
  if (packed && packedPrecision == prec && packedFs == fs) return packed;
  if (need > packedBytes) {
    if (packed) cudaSafeCall(cudaFree(packed));
    packed = nullptr;
    cudaSafeCall(cudaMalloc(&packed, need));
    packedBytes = need;
  }
  scnSafeCall(scn_conv_pack_weights(W.dPtr(), nFeaturesIn, nFeaturesOut, prec, packed, memStream.stream));
  packedPrecision = prec; packedFs = fs;
  (void)nIn;
  return packed;
}
long long NetworkInNetworkLayer::enqueueRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                                              SpatiallySparseBatchInterface &output, long long rowsInBound, int *) {
  (void)batch;
  if (input.nFeatures != nFeaturesIn) throw ScnException("NetworkInNetworkLayer: wrong number of input features");
  output.nFeatures = nFeaturesOut;
  output.spatialSize = input.spatialSize;
  output.gridOwner = input.gridOwner; // same geometry: the grids are shared, not copied
  return rowsInBound;
}
void NetworkInNetworkLayer::finishRules(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                                        const int *) {
  requireInference(batch);
  if (input.nFeatures != nFeaturesIn) throw ScnException("NetworkInNetworkLayer: wrong number of input features");
  output.nFeatures = nFeaturesOut;
  output.spatialSize = input.spatialSize;
  output.nSpatialSites = input.nSpatialSites;
  output.maxSitesPerSample = input.maxSitesPerSample;
  output.gridOwner = input.gridOwner; // same geometry: the grids are shared, not copied
  output.featuresPresent.hVector() = range(nFeaturesOut); // the matrices keep their full width; see presentSubset
  output.backpropErrors = true;
  output.learntOutput = true;
  output.presentSubset.clear();
  output.presentMask.resize(0);
  if (batch.type == TRAINBATCH && dropout > 0) { // NetworkInNetworkLayer.cu:152-154
    const int keep = nFeaturesOut * (1.0f - dropout);
    std::lock_guard<std::mutex> lock(rngMutex);
    if (!forcedPresent.empty()) {
      for (size_t i = 0; i < forcedPresent.size(); ++i)
        if (forcedPresent[i] < 0 || forcedPresent[i] >= nFeaturesOut || (i && forcedPresent[i] <= forcedPresent[i - 1]))
          throw ScnException("NetworkInNetworkLayer: forcedPresent must hold ascending feature indices below nFeaturesOut");
      output.presentSubset = forcedPresent;
    } else {
      output.presentSubset = rng.NchooseM(nFeaturesOut, keep);
    }
    if ((int)output.presentSubset.size() < nFeaturesOut) {
      output.presentMask.copyToCPU();
      std::vector<float> &m = output.presentMask.hVector();
      m.assign(nFeaturesOut, 0.f);
      for (int f : output.presentSubset) m[f] = 1.f;
      output.presentMask.copyToGPU();
    }
  }
}
void NetworkInNetworkLayer::preprocess(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output) {
  enqueueRules(batch, input, output, input.nSpatialSites, nullptr);
  finishRules(batch, input, output, nullptr);
}
bool NetworkInNetworkLayer::forwardsEarly(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &source, SpatiallySparseBatchInterface &input,
                                          SpatiallySparseBatchInterface &output, int cells, long long rowsBound, const int *d_rows) {
  if (batch.type == TRAINBATCH || batch.type == RESCALEBATCH || rowsBound < 1 || rowsBound * (long long)nFeaturesOut > INT_MAX) return false;
  const int sp = splitPrecision(precision, batch);
  if (sp < 0) return false;
  if (fn == SOFTMAX || nFeaturesOut % 4 != 0 || nFeaturesIn % cells != 0) return false;
  const int nIn = nFeaturesIn / cells;
  const void *pk = packedWeights(cells, nIn, sp);
  if (!pk) return false;
  output.sub->features.resize((int)(rowsBound * nFeaturesOut));
  const float p = 1.0f - (batch.type != RESCALEBATCH ? dropout : 0.0f);
  const int rc = scn_conv_nin_forward_dyn(source.sub->features.dPtr(), input.rules.dPtr(), (int)rowsBound, d_rows, cells, nIn, pk, B.dPtr(), slopes(),
                                          nFeaturesOut, p, (int)fn, output.sub->features.dPtr(), sp, memStream.stream);
  if (rc == SCN_ERR_UNSUPPORTED) return false; // e.g. so few rows that K would be split
  scnSafeCall(rc);
  return true;
}
void NetworkInNetworkLayer::countMultiplyAdds(SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output) {
  multiplyAddCount += (__int128_t)output.nSpatialSites * input.featuresPresent.size() * output.featuresPresent.size();
}
void NetworkInNetworkLayer::finishEarly(SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output) {
  output.sub->features.resize(output.nSpatialSites * output.featuresPresent.size());
  countMultiplyAdds(input, output);
}
bool NetworkInNetworkLayer::forwardsPooled(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &source, SpatiallySparseBatchInterface &input,
                                           SpatiallySparseBatchInterface &poolOutput, int convCells, int poolCells, long long rowsPoolBound,
                                           const int *d_rowsPool, int rowsUnpooled) {
  if (batch.type == TRAINBATCH || batch.type == RESCALEBATCH || rowsPoolBound < 1 || rowsPoolBound * (long long)nFeaturesOut > INT_MAX) return false;
  const int sp = splitPrecision(precision, batch);
  if (sp < 0) return false;
  if (fn == SOFTMAX || nFeaturesOut % 4 != 0 || nFeaturesIn % convCells != 0) return false;
  const int nIn = nFeaturesIn / convCells;
  const void *pk = packedWeights(convCells, nIn, sp);
  if (!pk) return false;
  const int n = (int)(rowsPoolBound * nFeaturesOut);
  poolOutput.sub->features.resize(n);
  poolOutput.sub->poolingChoices.resize(n);
  const float p = 1.0f - (batch.type != RESCALEBATCH ? dropout : 0.0f);
  // a layer of few tiles keeps its K split: the pooling then runs where the partial sums are added
  void *ws = nullptr;
  const size_t wsBytes = (rowsUnpooled > 0 && !d_rowsPool) ? scn_conv_nin_workspace_bytes(rowsUnpooled, convCells, nIn, nFeaturesOut, sp) : 0;
  if (wsBytes) {
    splitScratch.resize((int)((wsBytes + sizeof(float) - 1) / sizeof(float)));
    ws = splitScratch.dPtr();
  }
  const int rc = scn_conv_nin_maxpool_forward(source.sub->features.dPtr(), input.rules.dPtr(), convCells, nIn, pk, B.dPtr(), slopes(), nFeaturesOut, p,
                                              (int)fn, poolOutput.rules.dPtr(), poolCells, (int)rowsPoolBound, d_rowsPool, rowsUnpooled,
                                              poolOutput.sub->features.dPtr(), poolOutput.sub->poolingChoices.dPtr(), ws, wsBytes, sp, memStream.stream);
  if (rc == SCN_ERR_UNSUPPORTED) return false; // e.g. so few rows that K would be split
  scnSafeCall(rc);
  return true;
}
bool NetworkInNetworkLayer::forwardsWithNext(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                                             NetworkInNetworkLayer &next, SpatiallySparseBatchInterface &nextOutput) {
  if (batch.type == TRAINBATCH || batch.type == RESCALEBATCH || fusePoolNext || next.fusePoolNext) return false;
  const int sp = splitPrecision(precision, batch);
  if (sp < 0) return false;
  if (next.precision != SCN_PREC_AUTO && next.precision != SCN_PREC_FP32) return false;
  if (fn == SOFTMAX || nFeaturesOut % 4 != 0 || next.nFeaturesOut > 16 || next.nFeaturesIn != nFeaturesOut) return false;
  const float *src;
  const int *rules = nullptr;
  int fs = 1, nIn = nFeaturesIn;
  if (input.deferredFrom) { // fused gather
    src = input.deferredFrom->sub->features.dPtr();
    rules = input.rules.dPtr();
    fs = input.deferredCells;
    nIn = nFeaturesIn / fs;
  } else {
    src = input.sub->features.dPtr();
  }
  const int rows = output.nSpatialSites;
  const size_t wsBytes = rows > 0 ? scn_conv_nin_workspace_bytes(rows, fs, nIn, nFeaturesOut, sp) : 0;
  if (!wsBytes) return false; // the layer would not split K
  const void *pk = packedWeights(fs, nIn, sp);
  if (!pk) return false;
  splitScratch.resize((int)((wsBytes + sizeof(float) - 1) / sizeof(float)));
  output.sub->features.resize(rows * output.featuresPresent.size());
  nextOutput.sub->features.resize(rows * nextOutput.featuresPresent.size());
  const bool rescale = batch.type == RESCALEBATCH;
  const float p = 1.0f - (!rescale ? dropout : 0.0f), p2 = 1.0f - (!rescale ? next.dropout : 0.0f);
  const int rc = scn_conv_nin_nin_forward(src, rules, rows, fs, nIn, pk, B.dPtr(), slopes(), nFeaturesOut, p, (int)fn, next.W.dPtr(), next.B.dPtr(),
                                          next.slopes(), next.nFeaturesOut, p2, (int)next.fn, output.sub->features.dPtr(),
                                          nextOutput.sub->features.dPtr(), splitScratch.dPtr(), wsBytes, sp, memStream.stream);
  if (rc == SCN_ERR_UNSUPPORTED) return false;
  scnSafeCall(rc);
  countMultiplyAdds(input, output);
  next.countMultiplyAdds(output, nextOutput);
  return true;
}
void NetworkInNetworkLayer::forwards(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output) {
  if (fusePoolNext && input.deferredFrom && batch.type != TRAINBATCH && batch.type != RESCALEBATCH) { // the pooling layer behind this one runs all three steps
    output.deferredLearnt = this;
    output.deferredLearntInput = &input;
    countMultiplyAdds(input, output);
    return;
  }
  forwardsNow(batch, input, output);
  countMultiplyAdds(input, output);
}
void NetworkInNetworkLayer::forwardsNow(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output) {
  requireInference(batch);
  output.sub->features.resize(output.nSpatialSites * output.featuresPresent.size());
  float p = 1.0f - (batch.type != RESCALEBATCH ? dropout : 0.0f); // NetworkInNetworkLayer.cu:188
  int inPeriod = 0;
  // a training batch that drops features on either side of this layer runs on the kept ones unscaled (NetworkInNetworkLayer.cu:162-186)
  if (batch.type == TRAINBATCH && (output.presentMask.size() || presentMaskAt(batch, input, inPeriod))) p = 1.0f;
  const float *src;
  const int *rules = nullptr;
  int fs = 1, nIn = nFeaturesIn;
  if (input.deferredFrom) { // fused gather
    src = input.deferredFrom->sub->features.dPtr();
    rules = input.rules.dPtr();
    fs = input.deferredCells;
    nIn = nFeaturesIn / fs;
  } else {
    src = input.sub->features.dPtr();
  }
  const bool wasAuto = precision == SCN_PREC_AUTO;
  int prec = wasAuto ? scn_conv_auto_precision() : precision;
  if (splitPrecision(precision, batch) >= 0) prec = splitPrecision(precision, batch); // (tf32 operands for training steps)
  const void *pk = nullptr;
  if (prec != SCN_PREC_FP32) {
    pk = packedWeights(fs, nIn, prec);
    if (nFeaturesOut % 4 != 0) pk = nullptr; // the tensor-core kernels store whole float4 columns
    if (!pk) {
      if (!wasAuto && !precisionFallback) throw ScnException("NetworkInNetworkLayer: layer shape has no tensor-core path; use SCN_PREC_AUTO or SCN_PREC_FP32");
      prec = SCN_PREC_FP32;
    }
  }
  void *ws = nullptr;
  size_t wsBytes = pk ? scn_conv_nin_workspace_bytes(output.nSpatialSites, fs, nIn, nFeaturesOut, prec) : 0;
  if (wsBytes) { // few output tiles: split K over more CTAs, partial sums in a per-layer scratch vector
    splitScratch.resize((int)((wsBytes + sizeof(float) - 1) / sizeof(float)));
    ws = splitScratch.dPtr();
  }
  scnSafeCall(scn_conv_nin_forward_ws(src, rules, output.nSpatialSites, fs, nIn, W.dPtr(), pk, B.dPtr(), slopes(), nFeaturesOut, p,
                                      (int)fn, prec, output.sub->features.dPtr(), ws, wsBytes, memStream.stream));
  if (output.presentMask.size()) // the dropped features: zeros in place of the columns the reference's narrow matrix leaves out
    scnSafeCall(scn_mask_columns(output.sub->features.dPtr(), output.nSpatialSites, nFeaturesOut, output.presentMask.dPtr(), memStream.stream));
}
// Weight files: raw fp32 W then B (then momentum copies) per layer (NetworkInNetworkLayer.cu:290-328).
void NetworkInNetworkLayer::loadWeightsFromStream(std::ifstream &f, bool momentum) {
  std::vector<float> &w = W.hVector(), &b = B.hVector();
  f.read((char *)w.data(), sizeof(float) * w.size());
  f.read((char *)b.data(), sizeof(float) * b.size());
  if (momentum) f.seekg((std::streamoff)(sizeof(float) * (w.size() + b.size())), std::ios::cur);
  if (!f) throw ScnException("weight file ends early");
  weightsChanged();
}
void NetworkInNetworkLayer::putWeightsToStream(std::ofstream &f, bool momentum) {
  const bool wOn = W.onGPU, bOn = B.onGPU;
  std::vector<float> &w = W.hVector(), &b = B.hVector();
  f.write((char *)w.data(), sizeof(float) * w.size());
  f.write((char *)b.data(), sizeof(float) * b.size());
  if (momentum) { std::vector<float> z(w.size() + b.size(), 0.f); f.write((char *)z.data(), sizeof(float) * z.size()); }
  if (wOn) W.copyToGPU();
  if (bOn) B.copyToGPU();
}
int NetworkInNetworkLayer::calculateInputSpatialSize(int outputSpatialSize) { return outputSpatialSize; }
void replicateArray(float *src, float *dst, int nRows, int nColumns, cudaMemStream &memStream) {
  for (int r = 0; r < nRows; ++r)
    cudaSafeCall(cudaMemcpyAsync(dst + (size_t)r * nColumns, src, sizeof(float) * nColumns, cudaMemcpyDeviceToDevice, memStream.stream));
}

// ------------------------------------------------------------------ NetworkInNetworkPReLULayer
NetworkInNetworkPReLULayer::NetworkInNetworkPReLULayer(cudaMemStream &memStream, cublasHandle_t &h, int nFeaturesIn, int nFeaturesOut,
                                                       float dropout, float alpha)
    : NetworkInNetworkLayer(memStream, h, nFeaturesIn, nFeaturesOut, dropout, PRELU, alpha), PReLU(false, nFeaturesOut), MPReLU(false, 0) {
  PReLU.setConstant(0.25f);
}
float *NetworkInNetworkPReLULayer::slopes() { return PReLU.dPtr(); }
void NetworkInNetworkPReLULayer::loadWeightsFromStream(std::ifstream &f, bool momentum) {
  std::vector<float> &w = W.hVector(), &b = B.hVector(), &s = PReLU.hVector();
  f.read((char *)w.data(), sizeof(float) * w.size());
  f.read((char *)b.data(), sizeof(float) * b.size());
  f.read((char *)s.data(), sizeof(float) * s.size());
  if (momentum) f.seekg((std::streamoff)(sizeof(float) * (w.size() + b.size() + s.size())), std::ios::cur);
  if (!f) throw ScnException("weight file ends early");
  weightsChanged();
}
void NetworkInNetworkPReLULayer::putWeightsToStream(std::ofstream &f, bool momentum) {
  std::vector<float> &w = W.hVector(), &b = B.hVector(), &s = PReLU.hVector();
  f.write((char *)w.data(), sizeof(float) * w.size());
  f.write((char *)b.data(), sizeof(float) * b.size());
  f.write((char *)s.data(), sizeof(float) * s.size());
  if (momentum) { std::vector<float> z(w.size() + b.size() + s.size(), 0.f); f.write((char *)z.data(), sizeof(float) * z.size()); }
}

// ------------------------------------------------------------------ applySigmoid / SoftmaxClassifier
void applySigmoid(SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output, ActivationFunction fn, cudaMemStream &memStream) {
  if (fn == PRELU) throw ScnException("applySigmoid: PReLU needs its layer's slopes");
  scnSafeCall(scn_activation_forward(input.sub->features.dPtr(), output.sub->features.dPtr(), output.nSpatialSites,
                                     output.featuresPresent.size(), (int)fn, nullptr, memStream.stream));
}

// SigmoidLayer.cu:224-267.  (PReLU has its own layer class there too; SOFTMAX hands the gradient through unchanged: the
// classifier's gradient is already taken with respect to the softmax input.)
void applySigmoidBackProp(SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output, ActivationFunction fn,
                          cudaMemStream &memStream) {
  if (fn == PRELU) throw ScnException("applySigmoidBackProp: PReLU needs its layer's slopes");
  const int rows = output.nSpatialSites, N = output.featuresPresent.size();
  if ((int)output.sub->dfeatures.size() != rows * N) throw ScnException("applySigmoidBackProp: the output's gradient is missing");
  float *d = output.sub->dfeatures.dPtr();
  if (input.sub != output.sub) {
    input.sub->dfeatures.resize(rows * N);
    cudaSafeCall(cudaMemcpyAsync(input.sub->dfeatures.dPtr(), d, sizeof(float) * (size_t)rows * N, cudaMemcpyDeviceToDevice, memStream.stream));
    d = input.sub->dfeatures.dPtr();
  }
  scnSafeCall(scn_activation_backward(output.sub->features.dPtr(), d, rows, N, (int)fn, nullptr, nullptr, memStream.stream));
}
void maxPoolBackProp(float *d1, float *d2, int count, int nOut, int *d_choice, cudaMemStream &memStream) {
  scnSafeCall(scn_maxpool_backward(d2, d_choice, (long long)count * nOut, d1, 0, memStream.stream)); // (0: nothing is zeroed)
}
void propBackwardFromMatrixMultiply(float *inDFeatures, float *outDFeatures, int *rules, int count, int nIn, cudaMemStream &memStream) {
  scnSafeCall(scn_gather_backward(outDFeatures, rules, count, nIn, inDFeatures, 0, memStream.stream)); // (0: nothing is zeroed)
}

// SigmoidLayer.cu:269-310: a layer that only applies an activation.
SigmoidLayer::SigmoidLayer(cudaMemStream &memStream, ActivationFunction fn) : SpatiallySparseLayer(memStream), fn(fn) {
  std::cout << sigmoidNames[fn] << std::endl;
  changesGeometry = false;
}
long long SigmoidLayer::enqueueRules(SpatiallySparseBatch &, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                                     long long rowsInBound, int *) {
  output.nFeatures = input.nFeatures;
  output.spatialSize = input.spatialSize;
  output.gridOwner = input.gridOwner;
  return rowsInBound;
}
void SigmoidLayer::finishRules(SpatiallySparseBatch &, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output, const int *) {
  output.nFeatures = input.nFeatures;
  output.featuresPresent.hVector() = input.featuresPresent.hVector();
  output.spatialSize = input.spatialSize;
  output.nSpatialSites = input.nSpatialSites;
  output.maxSitesPerSample = input.maxSitesPerSample;
  output.gridOwner = input.gridOwner;
  output.backpropErrors = input.backpropErrors;
}
void SigmoidLayer::preprocess(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output) {
  enqueueRules(batch, input, output, input.nSpatialSites, nullptr);
  finishRules(batch, input, output, nullptr);
}
void SigmoidLayer::forwards(SpatiallySparseBatch &, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output) {
  output.sub->features.resize(output.nSpatialSites * output.featuresPresent.size());
  applySigmoid(input, output, fn, memStream);
}
void SigmoidLayer::backwards(SpatiallySparseBatch &, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output, float, float) {
  if (input.backpropErrors) applySigmoidBackProp(input, output, fn, memStream);
}
int SigmoidLayer::calculateInputSpatialSize(int outputSpatialSize) { return outputSpatialSize; }

// The classifier's device half and the one copy that brings its results to the host: probabilities, the nTop classes
// per row and the error word of the tensor-core kernels travel as one block (scn_classifier_result).  Returns the
// block in the stream's page-locked staging memory; throws if a tensor-core kernel gave up a wait.
const char *fetchClassifierResult(SpatiallySparseBatchInterface &input, int n, int nTop, cudaMemStream &memStream) {
  const int C = input.nFeatures;
  static thread_local vectorCUDA<int> block;
  const size_t bytes = scn_classifier_result_bytes(n, C, nTop);
  block.resize((int)(bytes / sizeof(int)));
  scnSafeCall(scn_classifier_result(input.sub->features.dPtr(), n, C, nTop, block.dPtr(), memStream.stream));
  char *stage = (char *)memStream.staging(bytes);
  cudaSafeCall(cudaMemcpyAsync(stage, block.dPtr(), bytes, cudaMemcpyDeviceToHost, memStream.stream));
  cudaSafeCall(cudaStreamSynchronize(memStream.stream));
  const int tcError = *(const int *)(stage + bytes - sizeof(int));
  if (tcError) throw ScnException("a tensor-core kernel gave up a time-limited wait (code " + std::to_string(tcError) +
                                  ": 1 gather, 2 epilogue, 3 weight copy, 4 MMA); this batch's features are not valid");
  return stage;
}

// SoftmaxClassifier.cu:16-58 without the training branch: probabilities and the nTop
// predictions come back in one staged copy; NLL and mistakes are scored on the host.
void SoftmaxClassifier(SpatiallySparseBatchInterface &input, SpatiallySparseBatch &batch, int nTop, cudaMemStream &memStream) {
  requireInference(batch);
  if (batch.batchSize != input.nSpatialSites) throw ScnException("SoftmaxClassifier: the top layer must hold one row per sample");
  const int n = batch.batchSize, C = input.nFeatures;
  const size_t pb = sizeof(float) * (size_t)n * C;
  if (batch.type == TRAINBATCH) { // the backward pass starts here: d cost / d (softmax input), SoftmaxClassifier.cu:24-33
    if (batch.labels.size() != (unsigned)n) throw ScnException("SoftmaxClassifier: a TRAINBATCH needs one label per sample");
    input.sub->dfeatures.resize(n * C);
    scnSafeCall(scn_softmax_nll_backward(input.sub->features.dPtr(), batch.labels.dPtr(), n, C, input.sub->dfeatures.dPtr(), memStream.stream));
  }
  const char *stage = fetchClassifierResult(input, n, nTop, memStream);
  const float *probs = (const float *)stage;
  const int *pred = (const int *)(stage + pb);
  for (int i = 0; i < n; ++i) { // refill the vectors that reset() set aside, where there are any
    if (!batch.spareProbabilities.empty()) { batch.probabilities.emplace_back(std::move(batch.spareProbabilities.back())); batch.spareProbabilities.pop_back(); }
    else batch.probabilities.emplace_back();
    batch.probabilities.back().assign(probs + (size_t)i * C, probs + (size_t)(i + 1) * C);
    if (!batch.sparePredictions.empty()) { batch.predictions.emplace_back(std::move(batch.sparePredictions.back())); batch.sparePredictions.pop_back(); }
    else batch.predictions.emplace_back();
    batch.predictions.back().assign(pred + (size_t)i * nTop, pred + (size_t)(i + 1) * nTop);
  }
  if (batch.type != UNLABELEDBATCH && batch.labels.size() == (unsigned)n) {
    std::vector<int> &labels = batch.labels.hVector();
    batch.mistakes += n;
    for (int i = 0; i < n; ++i) {
      batch.negativeLogLikelihood -= std::log(std::max(batch.probabilities[i][labels[i]], 1.0e-15f));
      for (int j = 0; j < nTop; ++j)
        if (batch.predictions[i][j] == labels[i]) batch.mistakes--;
    }
  }
}

// ------------------------------------------------------------------ backward pass (training step)
// ConvolutionalLayer.cu:134-146.  Behind a fused gather the learnt layer's backwards() has already scattered its input
// gradient through the rulebook onto this layer's input, so nothing is left to do here.
void ConvolutionalLayer::backwards(SpatiallySparseBatch &, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output, float, float) {
  if (!input.backpropErrors || output.deferredFrom) return;
  const int nIn = input.featuresPresent.size();
  input.sub->dfeatures.resize(input.nSpatialSites * nIn);
  scnSafeCall(scn_gather_backward(output.sub->dfeatures.dPtr(), output.rules.dPtr(), (long long)output.nSpatialSites * fs, nIn,
                                  input.sub->dfeatures.dPtr(), input.nSpatialSites, memStream.stream));
}
void ConvolutionalTriangularLayer::backwards(SpatiallySparseBatch &, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output, float,
                                             float) {
  if (!input.backpropErrors || output.deferredFrom) return;
  const int nIn = input.featuresPresent.size();
  input.sub->dfeatures.resize(input.nSpatialSites * nIn);
  scnSafeCall(scn_gather_backward(output.sub->dfeatures.dPtr(), output.rules.dPtr(), (long long)output.nSpatialSites * fs, nIn,
                                  input.sub->dfeatures.dPtr(), input.nSpatialSites, memStream.stream));
}
// MaxPoolingLayer.cu:134-146 (and MaxPoolingTriangularLayer.cu:49-61).
static void poolBackwards(SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output, cudaMemStream &ms) {
  if (!input.backpropErrors) return;
  const long long nIn = (long long)input.nSpatialSites * input.featuresPresent.size();
  const long long n = (long long)output.nSpatialSites * output.featuresPresent.size();
  if (output.sub->poolingChoices.size() != (unsigned)n) throw ScnException("max pooling backwards: no pooling choices (run forwards first)");
  input.sub->dfeatures.resize((int)nIn);
  scnSafeCall(scn_maxpool_backward(output.sub->dfeatures.dPtr(), output.sub->poolingChoices.dPtr(), n, input.sub->dfeatures.dPtr(), nIn, ms.stream));
}
void MaxPoolingLayer::backwards(SpatiallySparseBatch &, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output, float, float) {
  poolBackwards(input, output, memStream);
}
void MaxPoolingTriangularLayer::backwards(SpatiallySparseBatch &, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output, float,
                                          float) {
  poolBackwards(input, output, memStream);
}
// MaxPoolingLayer.cu:187-199 and its three siblings: the same gradient routing through the pooling choices.
void FractionalMaxPoolingLayerBase::backwards(SpatiallySparseBatch &, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output, float,
                                              float) {
  poolBackwards(input, output, memStream);
}
// TerminalPoolingLayer.cu:112-125.
void TerminalPoolingLayer::backwards(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output, float,
                                     float) {
  if (!input.backpropErrors) return;
  const int C = output.featuresPresent.size();
  input.sub->dfeatures.resize(input.nSpatialSites * C);
  scnSafeCall(scn_terminal_pool_backward(output.sub->dfeatures.dPtr(), output.rules.dPtr(), output.nSpatialSites, output.rules.size() / batch.batchSize,
                                         C, input.sub->dfeatures.dPtr(), input.nSpatialSites, memStream.stream));
}
// NetworkInNetworkLayer.cu:221-289: activation derivative in place on the output's gradient;
// dW = X^T d and dB = column sums (X read through the rulebook where the convolution in front is fused); the input's
// gradient d W^T with the weights as they were in the forward pass, scattered through the rulebook onto the
// convolution's input where fused; then the SGD update of W, B (and the PReLU slopes).  Where the batch drops features
// (on this layer's output, or on the learnt layer's below) the gradients of the dropped columns are zeroed on both sides
// and the update leaves the weights that touch a dropped feature, and their momentum, alone
// (dGradientDescentShrunkMatrix, NetworkInNetworkLayer.cu:43-61).
void NetworkInNetworkLayer::backwards(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                                      float learningRate, float momentum) {
  const int rows = output.nSpatialSites, N = nFeaturesOut, K = nFeaturesIn;
  cudaStream_t s = memStream.stream;
  if ((int)output.sub->dfeatures.size() != rows * N) throw ScnException("NetworkInNetworkLayer::backwards: the output's gradient is missing");
  if ((int)output.sub->features.size() != rows * N) throw ScnException("NetworkInNetworkLayer::backwards: the output's features are missing (run forwards on a TRAINBATCH)");
  float *d = output.sub->dfeatures.dPtr();
  int inPeriod = 0;
  const float *inMask = presentMaskAt(batch, input, inPeriod);
  const float *outMask = output.presentMask.size() ? output.presentMask.dPtr() : nullptr;
  if (outMask) scnSafeCall(scn_mask_columns(d, rows, N, outMask, s));
  scnSafeCall(scn_activation_backward(output.sub->features.dPtr(), d, rows, N, (int)fn, slopes(), slopeGradient(), s));
  const float *src;
  const int *rules = nullptr;
  int fs = 1, nIn = K;
  SpatiallySparseBatchInterface *target = &input; // whose dfeatures receive the input gradient
  if (input.deferredFrom) {
    target = input.deferredFrom;
    src = target->sub->features.dPtr();
    rules = input.rules.dPtr();
    fs = input.deferredCells;
    nIn = K / fs;
  } else {
    src = input.sub->features.dPtr();
  }
  dw.copyToGPU(); db.copyToGPU();
  dw.resize(K * N); db.resize(N);
  // the weight gradient: on the tensor cores (three tf32 products, the forward kernel with the roles turned) where the
  // shape has a form for it and the layer does not ask for plain fp32, else the CUDA-core kernel
  bool onTensorCores = false;
  if (precision != SCN_PREC_FP32 && rows > 0) {
    const size_t need = scn_conv_nin_backward_weights_tc_bytes(rows, fs, nIn, N);
    if (need) {
      const int st = scn_conv_nin_backward_weights_tc(src, rules, rows, fs, nIn, d, N, dw.dPtr(), db.dPtr(), memStream.deviceScratch(need), need, s);
      if (st == SCN_OK) onTensorCores = true;
      else if (st != SCN_ERR_UNSUPPORTED) scnSafeCall(st);
    }
  }
  if (!onTensorCores) scnSafeCall(scn_conv_nin_backward_weights(src, rules, rows, fs, nIn, d, N, dw.dPtr(), db.dPtr(), s));
  if (input.backpropErrors && rows > 0) {
    Wt.copyToGPU();
    Wt.resize(K * N);
    scnSafeCall(scn_transpose_weights(W.dPtr(), K, N, Wt.dPtr(), s));
    if ((int)zeroBias.size() != K) zeroed(zeroBias, K, memStream);
    // the forward kernel on the transposed weights: [rows x N] times [N x K]
    int prec = precision == SCN_PREC_AUTO ? scn_conv_auto_precision() : precision;
    if (prec == SCN_PREC_SPLIT) prec = SCN_PREC_3XTF32; // gradients keep tf32 operands (see splitPrecision)
    const void *pk = nullptr;
    if (prec != SCN_PREC_FP32 && K % 4 == 0) {
      const size_t need = scn_conv_packed_weight_bytes(N, K, prec);
      if (need) {
        if (need > packedTBytes) {
          if (packedT) cudaSafeCall(cudaFree(packedT));
          packedT = nullptr;
          cudaSafeCall(cudaMalloc(&packedT, need));
          packedTBytes = need;
        }
        scnSafeCall(scn_conv_pack_weights(Wt.dPtr(), N, K, prec, packedT, s));
        pk = packedT;
      }
    }
    if (!pk) prec = SCN_PREC_FP32;
    float *dX;
    if (rules) {
      dGathered.copyToGPU();
      dGathered.resize(rows * K);
      dX = dGathered.dPtr();
    } else {
      input.sub->dfeatures.resize(rows * K);
      dX = input.sub->dfeatures.dPtr();
    }
    void *ws = nullptr;
    const size_t wsBytes = pk ? scn_conv_nin_workspace_bytes(rows, 1, N, K, prec) : 0;
    if (wsBytes) {
      splitScratch.resize((int)((wsBytes + sizeof(float) - 1) / sizeof(float)));
      ws = splitScratch.dPtr();
    }
    scnSafeCall(scn_conv_nin_forward_ws(d, nullptr, rows, 1, N, Wt.dPtr(), pk, zeroBias.dPtr(), nullptr, K, 1.0f, SCN_NOSIGMOID, prec, dX, ws, wsBytes, s));
    multiplyAddCount += (__int128_t)rows * K * N;
    if (inMask) scnSafeCall(scn_mask_columns(dX, (long long)rows * (K / inPeriod), inPeriod, inMask, s));
    if (rules) {
      target->sub->dfeatures.resize(target->nSpatialSites * nIn);
      scnSafeCall(scn_gather_backward(dX, rules, (long long)rows * fs, nIn, target->sub->dfeatures.dPtr(), target->nSpatialSites, s));
    }
  }
  multiplyAddCount += (__int128_t)rows * K * N;
  if ((int)MW.size() != K * N) { zeroed(MW, K * N, memStream); zeroed(MB, N, memStream); }
  if (inMask || outMask) {
    scnSafeCall(scn_sgd_update_masked(W.dPtr(), MW.dPtr(), dw.dPtr(), K, N, inMask, inPeriod, outMask, learningRate, momentum, 0, s));
    scnSafeCall(scn_sgd_update_masked(B.dPtr(), MB.dPtr(), db.dPtr(), 1, N, nullptr, 1, outMask, learningRate, momentum, 0, s));
  } else {
    scnSafeCall(scn_sgd_update(W.dPtr(), MW.dPtr(), dw.dPtr(), (long long)K * N, learningRate, momentum, 0, s));
    scnSafeCall(scn_sgd_update(B.dPtr(), MB.dPtr(), db.dPtr(), N, learningRate, momentum, 0, s));
  }
  updateSlopes(learningRate, momentum, outMask);
  weightsChanged();
}
float *NetworkInNetworkPReLULayer::slopeGradient() {
  dprelu.copyToGPU();
  dprelu.resize(nFeaturesOut);
  return dprelu.dPtr();
}
// A batch that drops features updates the slopes of the kept ones only.  (The reference means to,
// NetworkInNetworkPReLULayer.cu:199-207, but its test `size() < size()` never holds, so it runs the full-width update on a
// narrow gradient vector and reads past its end: training a PReLU layer with dropout has no defined reference result.)
void NetworkInNetworkPReLULayer::updateSlopes(float learningRate, float momentum, const float *presentMask) {
  if ((int)MPReLU.size() != nFeaturesOut) zeroed(MPReLU, nFeaturesOut, memStream);
  if (presentMask) {
    scnSafeCall(scn_sgd_update_masked(PReLU.dPtr(), MPReLU.dPtr(), dprelu.dPtr(), 1, nFeaturesOut, nullptr, 1, presentMask, learningRate, momentum, 1,
                                      memStream.stream));
    return;
  }
  scnSafeCall(scn_sgd_update(PReLU.dPtr(), MPReLU.dPtr(), dprelu.dPtr(), nFeaturesOut, learningRate, momentum, 1, memStream.stream));
}

// ------------------------------------------------------------------ IndexLearnerLayer (index learning: every picture its own class)
IndexLearnerLayer::IndexLearnerLayer(cudaMemStream &memStream, cublasHandle_t &, int nFeaturesIn, int nFeaturesOut)
    : SpatiallySparseLayer(memStream), W(true, 0), nFeaturesIn(nFeaturesIn), nFeaturesOut(nFeaturesOut), indices(false, 0) {
  std::cout << "IndexLearnerLayer" << std::endl;
  zeroed(W, nFeaturesIn * nFeaturesOut, memStream); // IndexLearnerLayer.cu:29-31: the weights start at zero
  changesGeometry = false;
}
// IndexLearnerLayer.cu:35-45: only a TRAINBATCH runs this layer (processIndexLearnerBatch stops one layer early otherwise).
long long IndexLearnerLayer::enqueueRules(SpatiallySparseBatch &, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                                          long long rowsInBound, int *) {
  if (input.nFeatures != nFeaturesIn) throw ScnException("IndexLearnerLayer: wrong number of input features");
  output.nFeatures = nFeaturesOut;
  output.spatialSize = input.spatialSize;
  output.gridOwner = input.gridOwner;
  return rowsInBound;
}
void IndexLearnerLayer::finishRules(SpatiallySparseBatch &, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output, const int *) {
  output.nFeatures = nFeaturesOut;
  output.spatialSize = input.spatialSize;
  output.nSpatialSites = input.nSpatialSites;
  output.maxSitesPerSample = input.maxSitesPerSample;
  output.gridOwner = input.gridOwner;
  output.backpropErrors = true;
  output.learntOutput = true;
}
void IndexLearnerLayer::preprocess(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output) {
  enqueueRules(batch, input, output, input.nSpatialSites, nullptr);
  finishRules(batch, input, output, nullptr);
}
// IndexLearnerLayer.cu:47-70: softmax(X w) with w the batch's columns of W; no bias.
void IndexLearnerLayer::forwards(SpatiallySparseBatch &, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output) {
  const int n = (int)indexLearnerIndices.size(), rows = output.nSpatialSites;
  if (n < 1 || n > 1024) throw ScnException("IndexLearnerLayer: a batch of 1..1024 pictures is needed (set indexLearnerIndices)");
  for (int i : indexLearnerIndices)
    if (i < 0 || i >= nFeaturesOut) throw ScnException("IndexLearnerLayer: a picture's index exceeds the layer's width (the size of the training set)");
  output.featuresPresent.hVector() = indexLearnerIndices;
  indices.copyToCPU();
  indices.hVector() = indexLearnerIndices;
  output.sub->features.resize(rows * n);
  output.sub->dfeatures.resize(rows * n);
  w.copyToGPU();
  w.resize(nFeaturesIn * n);
  cudaStream_t s = memStream.stream;
  scnSafeCall(scn_gather_columns(W.dPtr(), nFeaturesIn, nFeaturesOut, indices.dPtr(), n, w.dPtr(), s));
  if ((int)zeroBias.size() < std::max(n, nFeaturesIn)) zeroed(zeroBias, std::max(n, nFeaturesIn), memStream);
  scnSafeCall(scn_conv_nin_forward_ws(input.sub->features.dPtr(), nullptr, rows, 1, nFeaturesIn, w.dPtr(), nullptr, zeroBias.dPtr(), nullptr, n, 1.0f,
                                      SCN_SOFTMAX, SCN_PREC_FP32, output.sub->features.dPtr(), nullptr, 0, s));
  multiplyAddCount += (__int128_t)rows * nFeaturesIn * n;
}
// IndexLearnerLayer.cu:71-100: dw = X^T d, the input's gradient d w^T, and the update of the batch's columns without momentum.
void IndexLearnerLayer::backwards(SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output,
                                  float learningRate, float) {
  const int n = (int)indexLearnerIndices.size(), rows = output.nSpatialSites, K = nFeaturesIn;
  cudaStream_t s = memStream.stream;
  if ((int)output.sub->dfeatures.size() != rows * n) throw ScnException("IndexLearnerLayer::backwards: the output's gradient is missing");
  float *d = output.sub->dfeatures.dPtr();
  dw.copyToGPU(); db.copyToGPU();
  dw.resize(K * n); db.resize(n);
  scnSafeCall(scn_conv_nin_backward_weights(input.sub->features.dPtr(), nullptr, rows, 1, K, d, n, dw.dPtr(), db.dPtr(), s));
  if (input.backpropErrors && rows > 0) {
    wt.copyToGPU();
    wt.resize(K * n);
    scnSafeCall(scn_transpose_weights(w.dPtr(), K, n, wt.dPtr(), s));
    input.sub->dfeatures.resize(rows * K);
    scnSafeCall(scn_conv_nin_forward_ws(d, nullptr, rows, 1, n, wt.dPtr(), nullptr, zeroBias.dPtr(), nullptr, K, 1.0f, SCN_NOSIGMOID, SCN_PREC_FP32,
                                        input.sub->dfeatures.dPtr(), nullptr, 0, s));
    int period = 0;
    if (const float *mask = presentMaskAt(batch, input, period)) // features the batch dropped below this layer
      scnSafeCall(scn_mask_columns(input.sub->dfeatures.dPtr(), (long long)rows * (K / period), period, mask, s));
    multiplyAddCount += (__int128_t)rows * K * n;
  }
  multiplyAddCount += (__int128_t)rows * K * n;
  // (a dropped input feature's column of X is zero, so its row of dw is zero and its weights stay as they are)
  scnSafeCall(scn_scatter_columns_axpy(W.dPtr(), K, nFeaturesOut, indices.dPtr(), n, dw.dPtr(), -learningRate, s));
}
void IndexLearnerLayer::loadWeightsFromStream(std::ifstream &f, bool) { // IndexLearnerLayer.cu:101-103: the weights alone
  std::vector<float> &h = W.hVector();
  f.read((char *)h.data(), sizeof(float) * h.size());
  if (!f) throw ScnException("weight file ends early");
}
void IndexLearnerLayer::putWeightsToStream(std::ofstream &f, bool) {
  const bool on = W.onGPU;
  std::vector<float> &h = W.hVector();
  f.write((char *)h.data(), sizeof(float) * h.size());
  if (on) W.copyToGPU();
}
int IndexLearnerLayer::calculateInputSpatialSize(int outputSpatialSize) { return outputSpatialSize; }

void IndexLearner(SpatiallySparseBatchInterface &input, SpatiallySparseBatch &batch, int nTop, cudaMemStream &memStream) {
  const int n = batch.batchSize;
  if (n != input.nSpatialSites || (size_t)n * n != input.sub->features.size()) throw ScnException("IndexLearner: the top layer must hold one row per picture and one column per picture of the batch");
  if (batch.type != TRAINBATCH) throw ScnException("IndexLearner: a TRAINBATCH is needed");
  // the backward pass starts here: d cost / d (softmax input) with picture i's class = column i (IndexLearnerLayer.cu:129-141)
  vectorCUDA<int> own(false, 0);
  own.hVector() = range(n);
  input.sub->dfeatures.resize(n * n);
  scnSafeCall(scn_softmax_nll_backward(input.sub->features.dPtr(), own.dPtr(), n, n, input.sub->dfeatures.dPtr(), memStream.stream));
  std::vector<float> probs((size_t)n * n);
  cudaSafeCall(cudaMemcpyAsync(probs.data(), input.sub->features.dPtr(), sizeof(float) * probs.size(), cudaMemcpyDeviceToHost, memStream.stream));
  cudaSafeCall(cudaStreamSynchronize(memStream.stream)); // (also: `own` is read before it goes out of scope)
  for (int i = 0; i < n; ++i) {
    batch.probabilities.emplace_back(probs.begin() + (size_t)i * n, probs.begin() + (size_t)(i + 1) * n);
    batch.predictions.push_back(vectorTopIndices(batch.probabilities.back(), nTop));
  }
  batch.mistakes += n;
  for (int i = 0; i < n; ++i) {
    batch.negativeLogLikelihood -= std::log(std::max(batch.probabilities[i][i], 1.0e-15f));
    for (int j = 0; j < nTop; ++j)
      if (batch.predictions[i][j] == i) batch.mistakes--;
  }
}
