// The data contract between layers (SpatiallySparseBatchInterface.h:8-46), extended with
// the device-resident form of the grids.
#pragma once
#include <vector>
#include "SparseGrid.h"
#include "vectorCUDA.h"

// The large vectors that stay on the device.
class SpatiallySparseBatchSubInterface {
public:
  vectorCUDA<float> features;     // [nSpatialSites x featuresPresent.size()]
  vectorCUDA<float> dfeatures;    // backward pass: d cost / d features, same shape
  vectorCUDA<int> poolingChoices; // argmax of max pooling, flat input index
  SpatiallySparseBatchSubInterface();
  void reset();
};

class SpatiallySparseBatchInterface {
public:
  SpatiallySparseBatchSubInterface *sub; // not owned
  int nFeatures;                         // features per site
  vectorCUDA<int> featuresPresent;       // features not dropped out (all of them at test time)
  int nSpatialSites;                     // rows in the whole batch, background rows included
  int spatialSize;                       // side of the grid
  bool backpropErrors;
  std::vector<SparseGrid> grids;         // host maps; see materializeGrids()
  vectorCUDA<int> rules;                 // [nSpatialSites x cells], filled by preprocess()

  // ---- device form of `grids` (no reference counterpart)
  vectorCUDA<int> siteKeys;       // [nSpatialSites] site key per row, -1 for background rows
  vectorCUDA<int> sampleOffsets;  // [batchSize+1] first row of each sample
  vectorCUDA<int> backgroundRows; // [batchSize] SparseGrid::backgroundCol per sample
  int maxSitesPerSample;          // largest number of sites (background excluded) in a sample
  // The interface whose three arrays above describe this interface's grids: itself, or,
  // behind a layer that keeps the geometry (NetworkInNetwork), the interface it copies.
  SpatiallySparseBatchInterface *gridOwner;
  // A gather that ConvolutionalLayer::forwards left for the next NetworkInNetwork layer to
  // fuse: when `deferredFrom` is set, features are NOT materialised and
  // out[r] = concat_f in[rules[r*fs+f]] is implied.
  SpatiallySparseBatchInterface *deferredFrom;
  int deferredCells;
  // The same one step later: a NetworkInNetworkLayer that is followed by a non-overlapping max-pooling layer
  // leaves its output unmaterialised (`deferredLearnt` = the layer, `deferredLearntInput` = its input interface)
  // and the pooling layer runs convolution, learnt layer and pooling as one kernel.
  class NetworkInNetworkLayer *deferredLearnt;
  SpatiallySparseBatchInterface *deferredLearntInput;

  // Training-time dropout.  The reference narrows `features` to the features a training batch keeps and lists them in
  // featuresPresent (NetworkInNetworkLayer.cu:152-154); here `features` keeps its full width, the dropped features'
  // columns hold zeros, featuresPresent lists every feature, and the subset drawn for the batch is in `presentSubset`
  // with `presentMask` its 0/1 form on the device (both empty: nothing dropped).  `learntOutput`: written by a learnt layer.
  std::vector<int> presentSubset;
  vectorCUDA<float> presentMask;
  bool learntOutput;

  explicit SpatiallySparseBatchInterface(SpatiallySparseBatchSubInterface *s);
  SpatiallySparseBatchInterface(SpatiallySparseBatchInterface &&o) noexcept; // pointers into a moved-from interface are dropped
  void summary();
  void reset();
  // Upload `grids` (as filled by Picture::codifyInputData-style code) into the device form.
  void uploadGrids(cudaMemStream &memStream);
  // Download the device form into `grids` (blocking).
  void materializeGrids(cudaMemStream &memStream);
};
