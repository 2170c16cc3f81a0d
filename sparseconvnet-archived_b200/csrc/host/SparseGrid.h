// Host view of one sample's grid: site key -> row id, plus the row of the sample's
// background ("null") vector (SparseGrid.h:68-77).  Iteration is in ascending key, which is
// the order of the reference's vectorHash backend and the order that fixes row numbering.
// On the device a grid is the keys[row] / offsets / background-row arrays of
// SpatiallySparseBatchInterface; these host maps are filled for the input layer and, for
// later layers, only when materializeGrids() is called.
#pragma once
#include <cstdint>
#include <map>

typedef std::map<int64_t, int> SparseGridMap;
class SparseGrid {
public:
  int backgroundCol; // -1: no null vector needed
  SparseGridMap mp;
  SparseGrid() : backgroundCol(-1) {}
};
