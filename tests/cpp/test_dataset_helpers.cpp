// Host-only checks of SpatiallySparseDataset's helpers (SpatiallySparseDataset.h:18-30): runs without a GPU.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include "SpatiallySparseDataset.h"

#define CHECK(c) do { if (!(c)) { std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #c); std::exit(1); } } while (0)

int main() {
  SpatiallySparseDataset all;
  all.name = "helpers"; all.nFeatures = 3; all.nClasses = 4; all.type = TRAINBATCH;
  for (int i = 0; i < 20; ++i) all.pictures.push_back(new SitesPicture(3, i % 4));
  const std::vector<Picture *> original = all.pictures;
  all.summary();
  SpatiallySparseDataset val = all.extractValidationSet(0.25f);
  CHECK(val.pictures.size() == 5 && all.pictures.size() == 15 && val.type == TESTBATCH && val.nClasses == 4 && val.nFeatures == 3);
  CHECK(val.name == "helpers Validation set" && all.name == "helpers minus Validation set");
  { // the split repeats: a second set built the same way gives the same pictures by position
    SpatiallySparseDataset again;
    again.name = "again"; again.nFeatures = 3; again.nClasses = 4; again.type = TRAINBATCH;
    again.pictures = original;
    SpatiallySparseDataset val2 = again.extractValidationSet(0.25f);
    CHECK(val2.pictures == val.pictures && again.pictures == all.pictures);
  }
  SpatiallySparseDataset six = all.subset(6);
  CHECK(six.pictures.size() == 6 && six.type == TRAINBATCH && six.name == "helpers minus Validation set subset");
  for (size_t i = 0; i + 1 < 6; ++i) { // in the order of the set, no picture twice
    auto a = std::find(all.pictures.begin(), all.pictures.end(), six.pictures[i]);
    auto b = std::find(all.pictures.begin(), all.pictures.end(), six.pictures[i + 1]);
    CHECK(a != all.pictures.end() && a < b);
  }
  SpatiallySparseDataset two = all.balancedSample(2);
  int perClass[4] = {0, 0, 0, 0};
  for (auto p : two.pictures) ++perClass[p->label];
  CHECK(two.pictures.size() == 8 && perClass[0] == 2 && perClass[1] == 2 && perClass[2] == 2 && perClass[3] == 2);
  SpatiallySparseDataset many = all.balancedSample(100); // more than any class has: the passes repeat pictures until every class has 100
  int perClassMany[4] = {0, 0, 0, 0};
  for (auto p : many.pictures) ++perClassMany[p->label];
  CHECK(many.pictures.size() == 400 && perClassMany[0] == 100 && perClassMany[1] == 100 && perClassMany[2] == 100 && perClassMany[3] == 100);
  std::vector<Picture *> a = all.pictures;
  all.shuffle();
  std::vector<Picture *> b = all.pictures;
  std::sort(a.begin(), a.end()); std::sort(b.begin(), b.end());
  CHECK(a == b);
  all.repeatSamples(3);
  CHECK(all.pictures.size() == 45 && all.pictures[0] == all.pictures[15] && all.pictures[14] == all.pictures[44]);
  all.pictures.resize(15);
  int kept = 0;
  for (auto p : all.pictures) kept += (p->label == 1 || p->label == 3);
  std::vector<int> was;
  for (auto p : all.pictures) if (p->label == 1 || p->label == 3) was.push_back(p->label);
  all.subsetOfClasses({3, 1}); // classes 3 and 1 become 0 and 1; the other pictures are deleted
  CHECK((int)all.pictures.size() == kept && all.nClasses == 2);
  for (size_t i = 0; i < all.pictures.size(); ++i) CHECK(all.pictures[i]->label == (was[i] == 3 ? 0 : 1));
  for (auto p : all.pictures) delete p;
  for (auto p : val.pictures) delete p;
  CHECK(globVector("/nonexistent-dir-for-this-test/*").empty());
  std::vector<std::string> here = globVector("/proc/self/s*");
  CHECK(!here.empty() && std::is_sorted(here.begin(), here.end()));
  std::printf("ALL OK\n");
  return 0;
}
