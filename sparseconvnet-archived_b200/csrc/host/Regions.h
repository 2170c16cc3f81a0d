// Region descriptions with the reference's names (Regions.h) and the host-callable
// gridRules() entry points.  The geometry classes are plain data: the builders run on the
// GPU (scn_rules_build); gridRules() here is a convenience that ships ONE sample's grid to
// the device, builds, and brings the result back -- the layers never use it, they build whole
// batches on the device.  The fractional max-pooling tick classes draw their random region bounds on
// the host (a few hundred integers per sample); the rules are built on the device from those tables
// (scn_fmp_rules_build).
#pragma once
#include <vector>
#include "Rng.h"
#include "SparseGrid.h"
#include "utilities.h"

void fmpGridRulesOneSample(int dimension, int nIn, int nOut, int poolSize, bool overlapping, const std::vector<int> &tables,
                           SparseGrid &inputGrid, SparseGrid &outputGrid, int &nOutputSpatialSites, std::vector<int> &rules);

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

// Region bounds of one axis of a fractional max-pooling layer (Regions.h:48-72): output j pools the
// inputs [inputL[j], inputR[j]); input i is pooled by the outputs [outputL[i], outputR[i]).
class FractionalMaxPoolingTicks {
public:
  std::vector<int> inputL, inputR, outputL, outputR;

protected:
  void fillOutputRanges(int nIn, int nOut);
};
class PseudorandomOverlappingFmpTicks : public FractionalMaxPoolingTicks {
public:
  PseudorandomOverlappingFmpTicks(int nIn, int nOut, int poolSize, RNG &rng);
};
class PseudorandomNonOverlappingFmpTicks : public FractionalMaxPoolingTicks {
public:
  PseudorandomNonOverlappingFmpTicks(int nIn, int nOut, int poolSize, RNG &rng);
};
class RandomOverlappingFmpTicks : public FractionalMaxPoolingTicks {
public:
  RandomOverlappingFmpTicks(int nIn, int nOut, int poolSize, RNG &rng);
};
class RandomNonOverlappingFmpTicks : public FractionalMaxPoolingTicks {
public:
  RandomNonOverlappingFmpTicks(int nIn, int nOut, int poolSize, RNG &rng);
};

// One tick object per axis (Regions.h:74-86, Regions.cu:127-157).
template <typename ticks> class FractionalPoolingRegions : public RectangularRegions {
  std::vector<ticks> pb;

public:
  FractionalPoolingRegions(int nIn, int nOut, int dimension, int poolSize, RNG &rng) : RectangularRegions(nIn, nOut, dimension, poolSize) {
    for (int i = 0; i < dimension; ++i) pb.push_back(ticks(nIn, nOut, poolSize, rng));
    if (nIn < nOut + poolSize - 1) throw ScnException("FractionalPoolingRegions: nIn < nOut + poolSize - 1");
  }
  int inputL(int axis, int j) { return pb[axis].inputL[j]; }
  int inputR(int axis, int j) { return pb[axis].inputR[j]; }
  int outputL(int axis, int i) { return pb[axis].outputL[i]; }
  int outputR(int axis, int i) { return pb[axis].outputR[i]; }
  // the four tables of every axis in the layout scn_fmp_rules_build reads: per axis inputL[nOut],
  // inputR[nOut], outputL[nIn], outputR[nIn]
  void appendTables(std::vector<int> &dst) {
    for (auto &t : pb) {
      dst.insert(dst.end(), t.inputL.begin(), t.inputL.end());
      dst.insert(dst.end(), t.inputR.begin(), t.inputR.end());
      dst.insert(dst.end(), t.outputL.begin(), t.outputL.end());
      dst.insert(dst.end(), t.outputR.begin(), t.outputR.end());
    }
  }
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
// The same for fractional max-pooling regions: uniformSizeRegions = true selects the overlapping
// builder, false the non-overlapping one (Regions.cu:782-802).
template <typename ticks>
void gridRules(SparseGrid &inputGrid, SparseGrid &outputGrid, FractionalPoolingRegions<ticks> &regions, int &nOutputSpatialSites,
               std::vector<int> &rules, bool uniformSizeRegions, int minActiveInputs = 1) {
  if (minActiveInputs != 1) throw ScnException("gridRules: fractional max-pooling regions take minActiveInputs = 1");
  std::vector<int> tables;
  regions.appendTables(tables);
  fmpGridRulesOneSample(regions.dimension, regions.nIn, regions.nOut, regions.s, uniformSizeRegions, tables, inputGrid, outputGrid,
                        nOutputSpatialSites, rules);
}
// Regions.h:120-127.
void gridRules(SparseGrid &inputGrid, SparseGrid &outputGrid, RegularTriangularRegions &regions,
               int &nOutputSpatialSites, std::vector<int> &rules, int minActiveInputs = 1);
