#include "SpatiallySparseDataset.h"
#include <glob.h>
#include <algorithm>
#include <iostream>
#include <random>

// SpatiallySparseDataset.cpp:7-23
void SpatiallySparseDataset::summary() {
  std::cout << "Name:            " << name << "\nType:            " << batchTypeNames[type] << "\nnFeatures:       " << nFeatures
            << "\nnPictures:       " << pictures.size() << "\nnClasses:        " << nClasses << std::endl;
  if (type == UNLABELEDBATCH) return;
  std::vector<int> perClass(nClasses > 0 ? nClasses : 0, 0);
  for (Picture *pic : pictures)
    if (pic->label >= 0 && pic->label < nClasses) ++perClass[pic->label];
  std::cout << "nPictures/class:";
  for (int c : perClass) std::cout << " " << c;
  std::cout << std::endl;
}
// SpatiallySparseDataset.cpp:24-40: the generator is seeded with 123 every time, so the split repeats.
SpatiallySparseDataset SpatiallySparseDataset::extractValidationSet(float p) {
  SpatiallySparseDataset val;
  val.name = name + " Validation set";
  name += " minus Validation set";
  val.nClasses = nClasses;
  val.nFeatures = nFeatures;
  val.type = TESTBATCH;
  std::mt19937 gen(123);
  std::shuffle(pictures.begin(), pictures.end(), gen);
  for (int take = (int)(pictures.size() * p); take > 0; --take) {
    val.pictures.push_back(pictures.back());
    pictures.pop_back();
  }
  return val;
}
// SpatiallySparseDataset.cpp:41-56
void SpatiallySparseDataset::subsetOfClasses(std::vector<int> activeClasses) {
  nClasses = (int)activeClasses.size();
  std::vector<Picture *> all;
  all.swap(pictures);
  for (Picture *pic : all) {
    auto at = std::find(activeClasses.begin(), activeClasses.end(), pic->label);
    if (at == activeClasses.end()) { delete pic; continue; }
    pic->label = (int)(at - activeClasses.begin());
    pictures.push_back(pic);
  }
}
// SpatiallySparseDataset.cpp:58-88: passes over a fresh permutation until every class has n pictures or a pass adds nothing.
// (The per-class counters keep counting past n, as in the reference: a class is done in the pass its counter reaches n.)
SpatiallySparseDataset SpatiallySparseDataset::balancedSample(int n) {
  SpatiallySparseDataset bs;
  bs.name = name + " sample";
  bs.nFeatures = nFeatures;
  bs.nClasses = nClasses;
  bs.type = type;
  std::vector<int> count(nClasses, 0);
  int classesDone = 0;
  while (classesDone < nClasses) {
    const std::vector<int> order = rng.permutation((int)pictures.size());
    bool progress = false;
    for (size_t i = 0; i < pictures.size() && classesDone < nClasses; ++i) {
      Picture *pic = pictures[order[i]];
      if (count[pic->label]++ < n) { bs.pictures.push_back(pic); progress = true; }
      if (count[pic->label] == n) ++classesDone;
    }
    if (!progress) break;
  }
  return bs;
}
// SpatiallySparseDataset.cpp:90-101
SpatiallySparseDataset SpatiallySparseDataset::subset(int n) {
  SpatiallySparseDataset sub;
  sub.name = name + " subset";
  sub.nFeatures = nFeatures;
  sub.nClasses = nClasses;
  sub.type = type;
  for (int i : rng.NchooseM((int)pictures.size(), n)) sub.pictures.push_back(pictures[i]);
  return sub;
}
void SpatiallySparseDataset::shuffle() { std::shuffle(pictures.begin(), pictures.end(), rng.gen); }
// SpatiallySparseDataset.cpp:106-113
void SpatiallySparseDataset::repeatSamples(int reps) {
  std::cout << "Repeating each sample in " << name << " " << reps << " times" << std::endl;
  const size_t n = pictures.size();
  pictures.reserve(n * (reps > 1 ? reps : 1));
  for (int r = 1; r < reps; ++r)
    for (size_t j = 0; j < n; ++j) pictures.push_back(pictures[j]);
}
std::vector<std::string> globVector(const std::string &pattern) {
  glob_t found = {};
  std::vector<std::string> files;
  if (glob(pattern.c_str(), GLOB_TILDE, nullptr, &found) == 0) {
    for (size_t i = 0; i < found.gl_pathc; ++i) files.emplace_back(found.gl_pathv[i]);
    globfree(&found);
  }
  std::sort(files.begin(), files.end());
  return files;
}
