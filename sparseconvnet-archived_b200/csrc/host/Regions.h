// Region descriptions with the reference's names (Regions.h) and the host-callable
// gridRules() entry points.  The geometry classes are plain data: the builders run on the
// GPU (scn_rules_build); gridRules() here is a convenience that ships ONE sample's grid to
// the device, builds, and brings the result back -- the layers never use it, they build whole
// batches on the device.  Fractional max-pooling regions are not built.
#pragma once
#include <vector>
#include "SparseGrid.h"
#include "utilities.h"

class RectangularRegions {
public:
  int nIn, nOut, dimension, s, sd;
  RectangularRegions(int nIn, int nOut, int dimension, int s);
  virtual ~RectangularRegions();
  virtual int inputL(int axis, int j) = 0;  // first input coordinate of output j's field
  virtual int inputR(int axis, int j) = 0;  // one past the last
  virtual int outputL(int axis, int i) = 0; // first output coordinate input i reaches
  virtual int outputR(int axis, int i) = 0; // one past the last
};

class RegularSquareRegions : public RectangularRegions {
public:
  int poolSize, poolStride;
  RegularSquareRegions(int nIn, int nOut, int dimension, int poolSize, int poolStride);
  ~RegularSquareRegions();
  int inputL(int axis, int j);
  int inputR(int axis, int j);
  int outputL(int axis, int i);
  int outputR(int axis, int i);
};

class RegularTriangularRegions {
public:
  int poolSize, poolStride, nIn, nOut, dimension;
  int s;                // side of the filter
  int S;                // cells of the filter: triangleSize(s, dimension)
  std::vector<int> ord; // cube cell -> filter cell, -1 outside the simplex
  RegularTriangularRegions(int nIn, int nOut, int dimension, int poolSize, int poolStride);
  int inputL(int j);
  int outputL(int i);
  int outputR(int i);
};

// One sample, through the device (Regions.h:84-87).  uniformSizeRegions must be true.
void gridRules(SparseGrid &inputGrid, SparseGrid &outputGrid, RegularSquareRegions &regions, int &nOutputSpatialSites,
               std::vector<int> &rules, bool uniformSizeRegions, int minActiveInputs = 1);
// Regions.h:120-127.
void gridRules(SparseGrid &inputGrid, SparseGrid &outputGrid, RegularTriangularRegions &regions,
               int &nOutputSpatialSites, std::vector<int> &rules, int minActiveInputs = 1);
