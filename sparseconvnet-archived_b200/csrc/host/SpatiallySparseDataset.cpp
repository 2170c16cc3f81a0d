// The helpers that cut and resample a data set.  What each one must do is fixed by the reference
// (SpatiallySparseDataset.cpp): which pictures move, in which order, under which names.
#include "SpatiallySparseDataset.h"
#include <glob.h>
#include <algorithm>
#include <iomanip>
#include <iostream>
#include <random>

namespace {
// An empty data set that inherits the metadata of `from` under the name "<from> <suffix>".
SpatiallySparseDataset emptyLike(const SpatiallySparseDataset &from, const char *suffix, batchType type) {
  SpatiallySparseDataset d;
  d.name = from.name + " " + suffix;
  d.nFeatures = from.nFeatures;
  d.nClasses = from.nClasses;
  d.type = type;
  return d;
}
} // namespace

// One "key: value" line per fact, keys padded to 17 columns, then the class histogram of a labelled set
// (SpatiallySparseDataset.cpp:7-23).
void SpatiallySparseDataset::summary() {
  const std::pair<const char *, std::string> facts[] = {{"Name:", name},
                                                        {"Type:", batchTypeNames[type]},
                                                        {"nFeatures:", std::to_string(nFeatures)},
                                                        {"nPictures:", std::to_string(pictures.size())},
                                                        {"nClasses:", std::to_string(nClasses)}};
  for (const auto &f : facts) std::cout << std::left << std::setw(17) << f.first << f.second << std::endl;
  if (type == UNLABELEDBATCH) return;
  std::vector<int> histogram(std::max(nClasses, 0), 0);
  for (const Picture *pic : pictures)
    if (pic->label >= 0 && pic->label < nClasses) histogram[pic->label] += 1;
  std::cout << "nPictures/class:";
  for (int n : histogram) std::cout << ' ' << n;
  std::cout << std::endl;
}

// The split repeats from run to run: the shuffle in front of it always starts from seed 123, and the validation
// pictures are taken off the END of the shuffled list, last one first (SpatiallySparseDataset.cpp:24-40).
SpatiallySparseDataset SpatiallySparseDataset::extractValidationSet(float p) {
  SpatiallySparseDataset val = emptyLike(*this, "Validation set", TESTBATCH);
  name += " minus Validation set";
  std::mt19937 fixed(123);
  std::shuffle(pictures.begin(), pictures.end(), fixed);
  const size_t take = (size_t)std::max(0, (int)(pictures.size() * p));
  val.pictures.assign(pictures.rbegin(), pictures.rbegin() + std::min(take, pictures.size()));
  pictures.resize(pictures.size() - val.pictures.size());
  return val;
}

// Class activeClasses[k] becomes class k; pictures of other classes are deleted (SpatiallySparseDataset.cpp:41-56).
void SpatiallySparseDataset::subsetOfClasses(std::vector<int> activeClasses) {
  nClasses = (int)activeClasses.size();
  auto newLabel = [&](int old) {
    const auto at = std::find(activeClasses.begin(), activeClasses.end(), old);
    return at == activeClasses.end() ? -1 : (int)(at - activeClasses.begin());
  };
  size_t kept = 0;
  for (Picture *pic : pictures) {
    const int l = newLabel(pic->label);
    if (l < 0) { delete pic; continue; }
    pic->label = l;
    pictures[kept++] = pic;
  }
  pictures.resize(kept);
}

// n pictures of every class that has any (SpatiallySparseDataset.cpp:58-88): passes over fresh permutations of the set; a
// picture is taken while its class has been met fewer than n times, a class is complete in the pass in which it is met
// for the n-th time, and the search ends when every class is complete or a whole pass took nothing.
SpatiallySparseDataset SpatiallySparseDataset::balancedSample(int n) {
  SpatiallySparseDataset sample = emptyLike(*this, "sample", type);
  std::vector<int> met(nClasses, 0);
  int complete = 0;
  for (bool took = true; took && complete < nClasses;) {
    took = false;
    for (int i : rng.permutation((int)pictures.size())) {
      if (complete >= nClasses) break;
      int &seen = met[pictures[i]->label];
      if (seen < n) { sample.pictures.push_back(pictures[i]); took = true; }
      if (++seen == n) ++complete;
    }
  }
  return sample;
}

// n pictures without replacement, in the order they have in this set (SpatiallySparseDataset.cpp:90-101).
SpatiallySparseDataset SpatiallySparseDataset::subset(int n) {
  SpatiallySparseDataset sub = emptyLike(*this, "subset", type);
  const std::vector<int> chosen = rng.NchooseM((int)pictures.size(), n);
  sub.pictures.reserve(chosen.size());
  std::transform(chosen.begin(), chosen.end(), std::back_inserter(sub.pictures), [&](int i) { return pictures[i]; });
  return sub;
}

void SpatiallySparseDataset::shuffle() { std::shuffle(pictures.begin(), pictures.end(), rng.gen); }

// The list followed by reps - 1 copies of itself (SpatiallySparseDataset.cpp:106-113).
void SpatiallySparseDataset::repeatSamples(int reps) {
  std::cout << "Repeating each sample in " << name << " " << reps << " times" << std::endl;
  const std::vector<Picture *> once = pictures;
  for (int r = 1; r < reps; ++r) pictures.insert(pictures.end(), once.begin(), once.end());
}

std::vector<std::string> globVector(const std::string &pattern) {
  std::vector<std::string> files;
  glob_t found = {};
  if (glob(pattern.c_str(), GLOB_TILDE, nullptr, &found) == 0) {
    files.assign(found.gl_pathv, found.gl_pathv + found.gl_pathc);
    globfree(&found);
  }
  std::sort(files.begin(), files.end());
  return files;
}
