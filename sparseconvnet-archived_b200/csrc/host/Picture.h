// The input contract (Picture.h:6-19): a picture writes its active sites into a SparseGrid
// and appends one feature row per site, plus one zero "background" row per sample whose id
// goes into grid.backgroundCol (e.g. OpenCVPicture.cpp:373-375).  Rows of one picture must
// be consecutive.  Decoding and augmentation of real datasets is not part of this library;
// SitesPicture is the concrete class used by the synthetic workloads and tests.
#pragma once
#include <string>
#include <vector>
#include "SparseGrid.h"
#include "types.h"

class Picture {
public:
  virtual void codifyInputData(SparseGrid &grid, std::vector<float> &features, int &nSpatialSites, int spatialSize) = 0;
  virtual Picture *distort(int /*unused seed source*/, batchType) { return this; }
  virtual std::string identify() { return std::string(); }
  int label; // -1 for unknown
  Picture(int label = -1) : label(label) {}
  virtual ~Picture() {}
};

// A picture given directly as site keys (row-major index in the spatialSize^dim cube) and
// per-site features.  Emits the background row first, then the sites in the order given.
class SitesPicture : public Picture {
public:
  std::vector<int64_t> keys;
  std::vector<float> features; // keys.size() x nFeatures
  int nFeatures;
  bool backgroundRow;
  SitesPicture(int nFeatures, int label = -1, bool backgroundRow = true) : Picture(label), nFeatures(nFeatures), backgroundRow(backgroundRow) {}
  void codifyInputData(SparseGrid &grid, std::vector<float> &out, int &nSpatialSites, int spatialSize) override;
};
