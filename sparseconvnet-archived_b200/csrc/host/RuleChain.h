// Helpers shared by the geometry layers (convolution, pooling): enqueue a batch-wide rule
// build on the device and finish the interface once the counts are on the host.
#pragma once
#include "SpatiallySparseLayer.h"

namespace rulechain {
// (The device scratch of the rule builds belongs to the network's cudaMemStream: cudaMemStream::deviceScratch.)
// While a list is installed (this thread), enqueueRegions() sizes the output buffers but records
// the build instead of launching it, so that the caller can hand the whole chain to one kernel.
struct DeferredBuild {
  scn_regions_t R;
  const int *inKeys, *inOff, *inBg;
  int rowsInBound;
  scn_chain_layer_t out;
};
void beginDeferred(std::vector<DeferredBuild> *list);
void endDeferred();
// Run recorded builds: one fused kernel when the samples are small enough, else one
// scn_rules_build per layer.  rowsHint as in scn_rules_chain_build; returns true if the fused
// kernel ran with a hint (so a capacity error means "retry with rowsHint = 0").
// resident: how a network that owns its chain state runs the fused kernel without stream operations in front of it
// (scn_rules_chain_build_resident): the phase of this batch's result records, the records of the next batch, and
// whether the input's background rows are still to be found (then they are written to list[0].inBg by the kernel,
// or by scn_background_rows where the fused kernel does not apply).
struct ResidentChain { int phase; int *resultNext; int nResultNext; bool findBackground; };
bool runDeferred(std::vector<DeferredBuild> &list, int batch, int maxRowsPerSample, int rowsHint, cudaMemStream &ms,
                 const ResidentChain *resident = nullptr);

long long enqueueRegions(const scn_regions_t &R, SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                         SpatiallySparseBatchInterface &output, long long rowsInBound, int *d_result, cudaMemStream &ms);
void finishRegions(const scn_regions_t &R, SpatiallySparseBatchInterface &output, const int *h_result);
// Run enqueue + finish for one layer with a blocking read of the counts (the per-layer
// preprocess() path of the reference API).
void preprocessNow(SpatiallySparseLayer &layer, SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                   SpatiallySparseBatchInterface &output);
// featuresPresent of a gather: the input's list repeated per filter cell with an offset of
// nFeatures per cell (ConvolutionalLayer.cu:74-80).
void convolutionFeaturesPresent(std::vector<int> &src, std::vector<int> &dst, int nf, int nfp, int nCopies);
} // namespace rulechain
