// Helpers shared by the geometry layers (convolution, pooling): enqueue a batch-wide rule
// build on the device and finish the interface once the counts are on the host.
#pragma once
#include "SpatiallySparseLayer.h"

namespace rulechain {
// Device scratch shared by all rule builds of a stream (grown on demand, never shrunk).
void *workspace(size_t bytes);
// A small device record array for callers that build one layer at a time.
int *scratchResult();

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
