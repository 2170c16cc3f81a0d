#include "RuleChain.h"
#include <climits>

namespace rulechain {
namespace { thread_local std::vector<DeferredBuild> *g_deferred = nullptr; }
void beginDeferred(std::vector<DeferredBuild> *list) { g_deferred = list; }
void endDeferred() { g_deferred = nullptr; }

bool runDeferred(std::vector<DeferredBuild> &list, int batch, int maxRowsPerSample, int rowsHint, cudaMemStream &ms,
                 const ResidentChain *resident) {
  if (list.empty()) return false;
  std::vector<scn_chain_layer_t> layers;
  for (auto &d : list) layers.push_back(d.out);
  const int n = (int)layers.size();
  if (rowsHint > 0 && !scn_rules_chain_supported(layers.data(), n, batch, maxRowsPerSample, rowsHint)) rowsHint = 0;
  const bool chain = scn_rules_chain_supported(layers.data(), n, batch, maxRowsPerSample, rowsHint) != 0;
  if (chain && resident) {
    const size_t bytes = scn_rules_chain_resident_workspace_bytes(n, batch);
    void *ws = ms.chainWorkspace(bytes);
    scnSafeCall(scn_rules_chain_build_resident(ms.chainState(), layers.data(), n, batch, list[0].inKeys, list[0].inOff,
                                               resident->findBackground ? nullptr : list[0].inBg, const_cast<int *>(list[0].inBg),
                                               maxRowsPerSample, rowsHint, ws, bytes, resident->phase, resident->resultNext, resident->nResultNext, ms.stream));
    return rowsHint > 0;
  }
  if (resident && resident->findBackground)
    scnSafeCall(scn_background_rows(list[0].inKeys, list[0].inOff, batch, const_cast<int *>(list[0].inBg), ms.stream));
  if (chain) {
    size_t bytes = scn_rules_chain_workspace_bytes(n, batch);
    void *ws = ms.deviceScratch(bytes);
    scnSafeCall(scn_rules_chain_build(layers.data(), n, batch, list[0].inKeys, list[0].inOff, list[0].inBg, maxRowsPerSample,
                                      rowsHint, ws, bytes, ms.stream));
    return rowsHint > 0;
  }
  for (auto &d : list) {
    size_t bytes = scn_rules_workspace_bytes(&d.R, batch, d.rowsInBound);
    void *ws = ms.deviceScratch(bytes);
    scnSafeCall(scn_rules_build(&d.R, batch, d.inKeys, d.inOff, d.inBg, d.rowsInBound, d.out.d_out_keys, d.out.d_out_off,
                                d.out.d_out_bg, d.out.d_rules, d.out.rows_out_capacity, d.out.d_result, ws, bytes, ms.stream));
  }
  return false;
}

long long enqueueRegions(const scn_regions_t &R, SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                         SpatiallySparseBatchInterface &output, long long rowsInBound, int *d_result, cudaMemStream &ms) {
  const int sd = scn_regions_cells(&R);
  if (sd < 0) throw ScnException(std::string("rule build: ") + scn_last_error());
  long long T = 1, full = 1;
  if (R.minActive != -1) for (int a = 0; a < R.dim; ++a) T *= (R.size + R.stride - 1) / R.stride;
  if (R.lattice == SCN_LATTICE_SQUARE) for (int a = 0; a < R.dim; ++a) full *= R.nOut;
  else full = triangleSize(R.nOut, R.dim);
  long long bound = std::min(rowsInBound * T, (long long)batch.batchSize * full) + batch.batchSize;
  if (bound * sd > INT_MAX || rowsInBound > INT_MAX) throw ScnException("rule build: more than 2^31 rule cells in one batch; use smaller batches");
  SpatiallySparseBatchInterface *g = input.gridOwner;
  output.gridOwner = &output;
  output.siteKeys.resize((int)bound);
  output.sampleOffsets.resize(batch.batchSize + 1);
  output.backgroundRows.resize(batch.batchSize);
  output.rules.resize((int)(bound * sd));
  if (g_deferred) {
    DeferredBuild d;
    d.R = R;
    d.inKeys = g->siteKeys.dPtr(); d.inOff = g->sampleOffsets.dPtr(); d.inBg = g->backgroundRows.dPtr();
    d.rowsInBound = (int)rowsInBound;
    d.out.regions = R;
    d.out.d_out_keys = output.siteKeys.dPtr(); d.out.d_out_off = output.sampleOffsets.dPtr();
    d.out.d_out_bg = output.backgroundRows.dPtr(); d.out.d_rules = output.rules.dPtr();
    d.out.rows_out_capacity = (int)bound; d.out.d_result = d_result;
    g_deferred->push_back(d);
    return bound;
  }
  size_t wsBytes = scn_rules_workspace_bytes(&R, batch.batchSize, (int)rowsInBound);
  void *ws = ms.deviceScratch(wsBytes);
  scnSafeCall(scn_rules_build(&R, batch.batchSize, g->siteKeys.dPtr(), g->sampleOffsets.dPtr(), g->backgroundRows.dPtr(),
                              (int)rowsInBound, output.siteKeys.dPtr(), output.sampleOffsets.dPtr(), output.backgroundRows.dPtr(),
                              output.rules.dPtr(), (int)bound, d_result, ws, wsBytes, ms.stream));
  return bound;
}

void finishRegions(const scn_regions_t &R, SpatiallySparseBatchInterface &output, const int *h) {
  if (h[2]) throw ScnException("rule build reported device error bits " + std::to_string(h[2]) +
                               " (1 capacity, 2 key outside the grid, 4 duplicate key)");
  const int sd = scn_regions_cells(&R);
  output.nSpatialSites = h[0];
  output.maxSitesPerSample = h[3];
  output.siteKeys.resize(h[0]);
  output.rules.resize(h[0] * sd);
}

void preprocessNow(SpatiallySparseLayer &layer, SpatiallySparseBatch &batch, SpatiallySparseBatchInterface &input,
                   SpatiallySparseBatchInterface &output) {
  int *d_res = layer.memStream.deviceResult();
  layer.enqueueRules(batch, input, output, input.nSpatialSites, d_res);
  int h[4] = {0, 0, 0, 0};
  if (layer.changesGeometry) {
    cudaSafeCall(cudaMemcpyAsync(h, d_res, sizeof(h), cudaMemcpyDeviceToHost, layer.memStream.stream));
    cudaSafeCall(cudaStreamSynchronize(layer.memStream.stream));
  }
  layer.finishRules(batch, input, output, h);
}

void convolutionFeaturesPresent(std::vector<int> &src, std::vector<int> &dst, int nf, int nfp, int nCopies) {
  dst.resize((size_t)nfp * nCopies);
  for (int c = 0; c < nCopies; ++c)
    for (int i = 0; i < nfp; ++i) dst[(size_t)c * nfp + i] = src[i] + nf * c;
}
} // namespace rulechain
