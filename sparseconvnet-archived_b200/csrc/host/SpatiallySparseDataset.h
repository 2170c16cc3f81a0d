// A list of pictures with its metadata (SpatiallySparseDataset.h).  The file readers of the
// reference (CIFAR, MNIST, CASIA, ...) are not part of this library.
#pragma once
#include <string>
#include <vector>
#include "Picture.h"
#include "types.h"

class SpatiallySparseDataset {
public:
  std::string name;
  std::string header;
  std::vector<Picture *> pictures; // not owned
  int nFeatures;
  int nClasses;
  batchType type;
  SpatiallySparseDataset() : nFeatures(0), nClasses(0), type(TESTBATCH) {}
  void summary();
};
