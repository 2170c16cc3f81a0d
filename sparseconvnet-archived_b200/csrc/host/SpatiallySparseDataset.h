// A list of pictures with its metadata and the helpers that cut and resample it (SpatiallySparseDataset.h).  The
// file readers of the reference (CIFAR, MNIST, CASIA, ...) are not part of this library.
#pragma once
#include <string>
#include <vector>
#include "Picture.h"
#include "Rng.h"
#include "types.h"

class SpatiallySparseDataset {
  RNG rng;

public:
  std::string name;
  std::string header;
  std::vector<Picture *> pictures; // shared with the data sets cut from this one; see subsetOfClasses for the one deletion
  int nFeatures;
  int nClasses;
  batchType type;
  SpatiallySparseDataset() : nFeatures(0), nClasses(0), type(TESTBATCH) {}
  void summary();
  void shuffle();
  // Moves floor(size * p) pictures into a new TESTBATCH set, after a shuffle with a fixed seed; renames both sets.
  SpatiallySparseDataset extractValidationSet(float p = 0.1);
  // Keeps the pictures whose label is listed, relabels them by position in the list and DELETES the others.
  void subsetOfClasses(std::vector<int> activeClasses);
  SpatiallySparseDataset subset(int n);         // n pictures drawn without replacement, in their order
  SpatiallySparseDataset balancedSample(int n); // n pictures of every class (a class with fewer is sampled again and again)
  void repeatSamples(int reps);                 // the list repeated: small sets then give epochs of a useful length
};

// The files that match a shell pattern, sorted.
std::vector<std::string> globVector(const std::string &pattern);
