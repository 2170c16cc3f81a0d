// Exercises the C++ classes that keep the reference's names the way a program written against
// the reference would: builders, per-layer preprocess()/forwards(), processBatch(), the host
// gridRules() entry point, vectorCUDA migration, fused against unfused convolution.
// Built and run by tests/test_gpu_cpp_api.py on a B200; prints "OK" lines and exits 0 on success.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <sstream>
#include <cstdlib>
#include <random>
#include <vector>
#include "BatchProducer.h"
#include "ConvolutionalLayer.h"
#include "MaxPoolingLayer.h"
#include "NetworkArchitectures.h"
#include "NetworkInNetworkLayer.h"
#include "Regions.h"
#include "Rng.h"
#include "SigmoidLayer.h"
#include "SparseConvNetCUDA.h"

#define CHECK(cond)                                                                   \
  do {                                                                                \
    if (!(cond)) { std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); return 1; } \
  } while (0)

static void fillWeights(SparseConvNetCUDA &cnn, unsigned seed) {
  std::mt19937 gen(seed);
  for (auto L : cnn.layers)
    if (auto n = dynamic_cast<NetworkInNetworkLayer *>(L)) {
      std::normal_distribution<float> nd(0.f, std::sqrt(2.0f / n->nFeaturesIn));
      for (auto &w : n->W.hVector()) w = nd(gen);
      for (auto &b : n->B.hVector()) b = 0.01f * nd(gen);
      n->weightsChanged();
    }
}

static SitesPicture *randomPicture(int S, int nF, int label, std::mt19937 &gen, double density) {
  SitesPicture *p = new SitesPicture(nF, label);
  std::uniform_real_distribution<double> u(0, 1);
  std::normal_distribution<float> nd(0.f, 1.f);
  for (int x = 0; x < S; ++x)
    for (int y = 0; y < S; ++y)
      if (u(gen) < density) {
        p->keys.push_back((int64_t)x * S + y);
        for (int f = 0; f < nF; ++f) p->features.push_back(nd(gen));
      }
  return p;
}

int main() {
  try {
    // ---- 1. the host gridRules(): the hand-checkable 8x8 example (conv3 then MP2)
    {
      SparseGrid in, mid, out;
      in.backgroundCol = 0;
      const int pts[5][2] = {{5, 5}, {1, 2}, {2, 2}, {3, 4}, {6, 1}};
      for (int i = 0; i < 5; ++i) in.mp[pts[i][0] * 8 + pts[i][1]] = i + 1;
      RegularSquareRegions conv(8, 6, 2, 3, 1), pool(6, 3, 2, 2, 2);
      int n1 = 0, n2 = 0;
      std::vector<int> r1, r2;
      gridRules(in, mid, conv, n1, r1, true, 1);
      gridRules(mid, out, pool, n2, r2, true, 1);
      CHECK(n1 == 28 && mid.backgroundCol == 27 && r1.size() == 28 * 9);
      const int row0[9] = {0, 0, 0, 0, 0, 2, 0, 0, 3}, row5[9] = {2, 0, 0, 3, 0, 0, 0, 0, 4};
      for (int c = 0; c < 9; ++c) CHECK(r1[c] == row0[c] && r1[5 * 9 + c] == row5[c]);
      const int p0[4] = {0, 1, 3, 4}, p1[4] = {2, 27, 5, 9};
      for (int c = 0; c < 4; ++c) CHECK(r2[c] == p0[c] && r2[4 + c] == p1[c]);
      CHECK(n2 == 9 && out.backgroundCol == -1);
      RegularTriangularRegions tri(5, 4, 3, 2, 1);
      CHECK(tri.S == 4 && tri.ord.size() == 8);
      std::printf("OK gridRules\n");
    }
    // ---- 2. builder arithmetic of the named architectures
    {
      DeepCNet a(2, 5, 100, VLEAKYRELU, 3, 10, 0.5f);
      CHECK(a.cnn->inputSpatialSize == 127 && a.cnn->layers.size() == 18);
    }
    {
      DeepC2 b(3, 2, 32, RELU, 1, 20);
      int s = 1; // walk back: C2 (no pool), then twice MP3/2 + C2
      s = s + 1;
      for (int i = 0; i < 2; ++i) { s = 3 + (s - 1) * 2; s = s + 1; }
      CHECK(b.cnn->inputSpatialSize == s);
      std::printf("OK builders\n");
    }
    // ---- 3. a small network three ways: processDataset (BatchProducer threads + fused rule chain),
    //         per-layer preprocess()/forwards() with fused convolutions, and with the gather materialised
    SparseConvNet net(2, 3, 5);
    net.addLeNetLayerMP(32, 3, 1, 2, 2, VLEAKYRELU, 0.1f);
    net.addLeNetLayerMP(64, 2, 1, 2, 2, VLEAKYRELU, 0.2f);
    net.addLeNetLayerMP(96, 2, 1, 1, 1, VLEAKYRELU, 0.0f);
    net.addSoftmaxLayer();
    SparseConvNetCUDA &cnn = *net.cnn;
    const int S = cnn.inputSpatialSize; // 1 <-C2- 2 <-MP2/2- 4 <-C2- 5 <-MP2/2- 10 <-C3- 12
    CHECK(S == 12);
    fillWeights(cnn, 5);
    std::mt19937 gen(11);
    SpatiallySparseDataset ds;
    ds.name = "cpp-test"; ds.nFeatures = 3; ds.nClasses = 5; ds.type = TESTBATCH;
    std::vector<SitesPicture *> pics;
    for (int i = 0; i < 7; ++i) { pics.push_back(randomPicture(S, 3, i % 5, gen, i == 3 ? 0.0 : 0.4)); ds.pictures.push_back(pics.back()); }
    std::vector<std::vector<float>> viaDataset;
    {
      BatchProducer bp(cnn, ds, S, 3); // batches of 3, 3, 1
      std::ofstream nof, nog;
      while (SpatiallySparseBatch *b = bp.nextBatch()) {
        cnn.processBatch(*b, 0, 0, nof, nog);
        for (auto &p : b->probabilities) viaDataset.push_back(p);
      }
    }
    CHECK(viaDataset.size() == 7);
    float nll = cnn.processDataset(ds, 4); // mean negative log-likelihood (SparseConvNetCUDA.cu:325)
    CHECK(nll > 0.f && nll < 10.f);
    cnn.processDatasetRepeatTest(ds, 4, 2);

    for (int variant = 0; variant < 2; ++variant) { // 0: fused conv+NiN, 1: ConvolutionalLayer writes the gathered matrix
      for (auto L : cnn.layers)
        if (auto c = dynamic_cast<ConvolutionalLayer *>(L)) c->fuseWithNext = (variant == 0);
      SpatiallySparseBatch &b = cnn.batchPool[0];
      cnn.prepareBatch(b);
      b.reset();
      b.type = TESTBATCH;
      SpatiallySparseBatchInterface &in = b.interfaces[0];
      in.nFeatures = 3; in.spatialSize = S; in.featuresPresent.hVector() = range(3);
      std::vector<float> &feat = in.sub->features.hVector();
      feat.clear();
      for (auto p : pics) {
        b.batchSize++;
        in.grids.push_back(SparseGrid());
        b.labels.hVector().push_back(p->label);
        p->codifyInputData(in.grids.back(), feat, in.nSpatialSites, S);
      }
      in.uploadGrids(cnn.memStream);
      for (size_t i = 0; i < cnn.layers.size(); ++i) cnn.layers[i]->preprocess(b, b.interfaces[i], b.interfaces[i + 1]); // one layer at a time, as BatchProducer.cu:72-75
      CHECK(b.interfaces.back().nSpatialSites == 7 && b.interfaces.back().nFeatures == 5);
      b.interfaces[2].materializeGrids(cnn.memStream);
      CHECK(b.interfaces[2].grids.size() == 7 && b.interfaces[2].grids[3].mp.empty()); // the empty picture stays empty
      CHECK((int)b.interfaces[1].rules.size() == b.interfaces[1].nSpatialSites * 9);
      std::ofstream nof, nog;
      cnn.processBatch(b, 0, 0, nof, nog);
      CHECK(b.probabilities.size() == 7);
      for (int i = 0; i < 7; ++i) {
        float sum = 0;
        for (int k = 0; k < 5; ++k) {
          sum += b.probabilities[i][k];
          CHECK(std::fabs(b.probabilities[i][k] - viaDataset[i][k]) < 2e-5f);
        }
        CHECK(std::fabs(sum - 1.f) < 1e-5f);
      }
      if (variant == 1) CHECK((int)b.interfaces[1].sub->features.size() == b.interfaces[1].nSpatialSites * 27);
      CHECK(b.mistakes >= 0 && b.mistakes <= 7);
    }
    std::printf("OK network three ways\n");
    // ---- 4. vectorCUDA migration and applySigmoid
    {
      vectorCUDA<float> v(false, 0);
      v.hVector() = {-3.f, -1.f, 0.f, 2.f};
      float *d = v.dPtr(); // uploads
      CHECK(v.onGPU && d != nullptr && v.size() == 4);
      SpatiallySparseBatchSubInterface sub;
      SpatiallySparseBatchInterface I(&sub);
      I.nSpatialSites = 1; I.nFeatures = 4; I.featuresPresent.hVector() = range(4);
      sub.features.hVector() = v.hVector(); // downloads v again
      CHECK(!v.onGPU);
      applySigmoid(I, I, VLEAKYRELU, cnn.memStream);
      cudaStreamSynchronize(cnn.memStream.stream);
      std::vector<float> &o = sub.features.hVector();
      CHECK(std::fabs(o[0] + 0.999f) < 1e-6f && std::fabs(o[1] + 0.333f) < 1e-6f && o[2] == 0.f && o[3] == 2.f);
      v.resize(0);
      std::printf("OK vectorCUDA/applySigmoid\n");
    }
    // ---- 5. what the library refuses
    {
      bool threw = false;
      try { cnn.loadWeights("/nonexistent/w", 1, false); } catch (const ScnException &) { threw = true; }
      CHECK(threw);
      std::printf("OK refusals\n");
    }
    // ---- 5b. training: a few passes over the (shuffled) TRAINBATCH dataset lower its negative log-likelihood
    {
      for (auto L : cnn.layers)
        if (auto c = dynamic_cast<ConvolutionalLayer *>(L)) c->fuseWithNext = true;
      ds.type = TRAINBATCH;
      const float first = cnn.processDataset(ds, 4, 0.01f, 0.9f);
      float last = first;
      for (int epoch = 0; epoch < 12; ++epoch) last = cnn.processDataset(ds, 4, 0.01f, 0.9f);
      CHECK(std::isfinite(first) && std::isfinite(last) && last < 0.8f * first);
      ds.type = TESTBATCH;
      std::printf("OK training (NLL %.3f -> %.3f)\n", first, last);
    }
    // ---- 5c. training with dropout: each TRAINBATCH keeps a drawn subset of a learnt layer's output features
    //          (NetworkInNetworkLayer.cu:152-154), zeros stand in the dropped columns, test batches keep every feature
    {
      SparseConvNet dnet(2, 3, 5);
      dnet.addLeNetLayerMP(32, 3, 1, 2, 2, VLEAKYRELU, 0.0f);
      dnet.addLeNetLayerMP(128, 2, 1, 2, 2, VLEAKYRELU, 0.5f); // keeps 64 of 128
      dnet.addLeNetLayerMP(96, 2, 1, 1, 1, VLEAKYRELU, 0.5f);  // 48 rounds to 64 of 96: dropout 1/3 (SparseConvNetCUDA.cu:56-60)
      dnet.addSoftmaxLayer();
      SparseConvNetCUDA &d = *dnet.cnn;
      CHECK(d.inputSpatialSize == S);
      fillWeights(d, 6);
      ds.type = TRAINBATCH;
      const float first = d.processDataset(ds, 4, 0.01f, 0.9f);
      float last = first;
      for (int epoch = 0; epoch < 12; ++epoch) last = d.processDataset(ds, 4, 0.01f, 0.9f);
      CHECK(std::isfinite(first) && std::isfinite(last) && last < first);
      {
        BatchProducer bp(d, ds, S, 4);
        std::ofstream nof, nog;
        SpatiallySparseBatch *b = bp.nextBatch();
        CHECK(b != nullptr);
        d.processBatch(*b, 0.01f, 0.9f, nof, nog);
        int withDropout = 0;
        for (size_t l = 0; l < d.layers.size(); ++l) {
          auto nin = dynamic_cast<NetworkInNetworkLayer *>(d.layers[l]);
          if (!nin || nin->dropout == 0.f) continue;
          SpatiallySparseBatchInterface &I = b->interfaces[l + 1];
          CHECK((int)I.presentSubset.size() == 64 && (int)I.featuresPresent.size() == nin->nFeaturesOut);
          std::vector<float> &f = I.sub->features.hVector();
          std::vector<char> kept(nin->nFeaturesOut, 0);
          for (int k : I.presentSubset) kept[k] = 1;
          for (int r = 0; r < I.nSpatialSites; ++r)
            for (int k = 0; k < nin->nFeaturesOut; ++k)
              if (!kept[k]) CHECK(f[(size_t)r * nin->nFeaturesOut + k] == 0.f);
          ++withDropout;
        }
        CHECK(withDropout == 2);
        while (bp.nextBatch()) {}
      }
      ds.type = TESTBATCH;
      const float test = d.processDataset(ds, 4);
      CHECK(std::isfinite(test));
      std::printf("OK training with dropout (NLL %.3f -> %.3f)\n", first, last);
    }
    // ---- 5e. input regularising constants (SparseConvNetCUDA.cu:537-566) and the dump of the features under the top layer
    {
      SparseConvNet rnet(2, 3, 5);
      rnet.addLeNetLayerMP(32, 3, 1, 2, 2, VLEAKYRELU, 0.0f);
      rnet.addLeNetLayerMP(64, 2, 1, 2, 2, VLEAKYRELU, 0.0f);
      rnet.addLeNetLayerMP(96, 2, 1, 1, 1, VLEAKYRELU, 0.0f);
      rnet.addSoftmaxLayer();
      fillWeights(*rnet.cnn, 12);
      ds.type = TESTBATCH;
      float largest[3] = {0.f, 0.f, 0.f};
      for (auto p : pics) {
        SparseGrid g; std::vector<float> f; int rows = 0;
        p->codifyInputData(g, f, rows, S);
        for (size_t i = 0; i < f.size(); ++i) largest[i % 3] = std::max(largest[i % 3], std::fabs(f[i]));
      }
      const float before = rnet.processDataset(ds, 4);
      rnet.calculateInputRegularizingConstants(ds);
      CHECK(rnet.cnn->inputNormalizingConstants.size() == 3);
      for (int c = 0; c < 3; ++c) CHECK(std::fabs(rnet.cnn->inputNormalizingConstants[c] * largest[c] - 1.f) < 1e-6f);
      const float after = rnet.processDataset(ds, 4); // the same pictures, inputs now scaled into [-1, 1]
      CHECK(std::isfinite(after) && after != before);
      ds.name = "cpp-test-dump";
      rnet.processDatasetDumpTopLevelFeatures(ds, 3, 2);
      std::ifstream ff("cpp-test-dump.features");
      int lines = 0;
      std::string line;
      while (std::getline(ff, line)) {
        std::istringstream is(line);
        int number, label, count = 0;
        float v;
        is >> number >> label;
        while (is >> v) ++count;
        CHECK(count == 96 && number == lines % (int)ds.pictures.size() && label == pics[number]->label);
        ++lines;
      }
      CHECK(lines == 2 * (int)ds.pictures.size());
      std::remove("cpp-test-dump.features");
      ds.name = "cpp-test";
      std::printf("OK regularising constants and feature dump\n");
    }
    // ---- 5d. index learning (SparseConvNet.h:50, 57-60): every picture its own class; a data set that is not a training
    //          set writes "<name>.features" (sample number, label, the features under the index learner)
    {
      SparseConvNet inet(2, 3, (int)ds.pictures.size());
      inet.addLeNetLayerMP(32, 3, 1, 2, 2, VLEAKYRELU, 0.0f);
      inet.addLeNetLayerMP(64, 2, 1, 2, 2, VLEAKYRELU, 0.0f);
      inet.addLeNetLayerMP(96, 2, 1, 1, 1, VLEAKYRELU, 0.0f);
      inet.addIndexLearnerLayer();
      CHECK(inet.cnn->inputSpatialSize == S);
      fillWeights(*inet.cnn, 8); // (leaves the index learner's weights at zero: it is no NetworkInNetworkLayer)
      ds.type = TRAINBATCH;
      const float first = inet.processIndexLearnerDataset(ds, 4, 0.01f, 0.9f);
      float last = first;
      for (int epoch = 0; epoch < 15; ++epoch) last = inet.processIndexLearnerDataset(ds, 4, 0.01f, 0.9f);
      CHECK(std::isfinite(first) && std::isfinite(last) && last < first);
      ds.type = TESTBATCH;
      ds.name = "cpp-test-index";
      inet.processIndexLearnerDataset(ds, 4);
      std::ifstream ff("cpp-test-index.features");
      int lines = 0;
      std::string line;
      while (std::getline(ff, line)) {
        std::istringstream is(line);
        int number, label, count = 0;
        float v;
        is >> number >> label;
        while (is >> v) ++count;
        CHECK(count == 96 && number == lines);
        ++lines;
      }
      CHECK(lines == (int)ds.pictures.size());
      std::remove("cpp-test-index.features");
      ds.name = "cpp-test";
      std::printf("OK index learning (NLL %.3f -> %.3f)\n", first, last);
    }
    // ---- 6. fractional max-pooling: a named FMP network, and the host gridRules over FractionalPoolingRegions
    {
      POFMPSparseConvNet fmp(2, 3, 32, 1.414f, VLEAKYRELU, 2, 5);
      CHECK(fmp.cnn->inputSpatialSize == 11); // 1 <-C2- 2 <-FMP- 3 <-C2- 4 <-FMP- 6 <-C2- 7 <-FMP- 10 <-C2- 11
      fillWeights(*fmp.cnn, 9);
      SpatiallySparseDataset fds;
      fds.name = "cpp-fmp"; fds.nFeatures = 2; fds.nClasses = 5; fds.type = TESTBATCH;
      std::vector<SitesPicture *> fp;
      for (int i = 0; i < 5; ++i) { fp.push_back(randomPicture(11, 2, i % 5, gen, 0.4)); fds.pictures.push_back(fp.back()); }
      float e1 = fmp.processDataset(fds, 2); // mean negative log-likelihood
      CHECK(e1 > 0.f && e1 < 20.f);
      for (auto q : fp) delete q;

      RNG rng;
      rng.gen.seed(42);
      FractionalPoolingRegions<PseudorandomNonOverlappingFmpTicks> regions(7, 5, 2, 2, rng);
      int covered = 0;
      for (int j = 0; j < 5; ++j) { CHECK(regions.inputR(0, j) - regions.inputL(0, j) >= 1 && regions.inputR(0, j) - regions.inputL(0, j) <= 2); covered += regions.inputR(0, j) - regions.inputL(0, j); }
      CHECK(covered == 7 && regions.inputL(0, 0) == 0 && regions.inputR(0, 4) == 7); // disjoint regions tile the axis
      SparseGrid gin, gout;
      gin.backgroundCol = 0;
      for (int k = 0; k < 49; k += 3) gin.mp[k] = 1 + k / 3;
      int nSites = 0;
      std::vector<int> rls;
      gridRules(gin, gout, regions, nSites, rls, false);
      CHECK(nSites >= 1 && (int)rls.size() == nSites * 4);
      int placed = 0;
      for (int v : rls) placed += v > 0;
      CHECK(placed == 17); // every input site appears exactly once: the regions do not overlap
      std::printf("OK fractional max-pooling\n");
    }
    // ---- 8. the data set helpers (SpatiallySparseDataset.h:18-30)
    {
      SpatiallySparseDataset all;
      all.name = "helpers"; all.nFeatures = 3; all.nClasses = 4; all.type = TRAINBATCH;
      for (int i = 0; i < 20; ++i) all.pictures.push_back(new SitesPicture(3, i % 4));
      all.summary();
      SpatiallySparseDataset val = all.extractValidationSet(0.25f);
      CHECK(val.pictures.size() == 5 && all.pictures.size() == 15 && val.type == TESTBATCH && val.nClasses == 4);
      CHECK(val.name == "helpers Validation set" && all.name == "helpers minus Validation set");
      SpatiallySparseDataset six = all.subset(6);
      CHECK(six.pictures.size() == 6 && six.type == TRAINBATCH);
      for (size_t i = 0; i < 6; ++i)
        for (size_t j = i + 1; j < 6; ++j) CHECK(six.pictures[i] != six.pictures[j]);
      SpatiallySparseDataset two = all.balancedSample(2);
      int perClass[4] = {0, 0, 0, 0};
      for (auto p : two.pictures) ++perClass[p->label];
      CHECK(two.pictures.size() == 8 && perClass[0] == 2 && perClass[1] == 2 && perClass[2] == 2 && perClass[3] == 2);
      std::vector<Picture *> order = all.pictures;
      all.shuffle();
      std::vector<Picture *> a = order, b = all.pictures;
      std::sort(a.begin(), a.end()); std::sort(b.begin(), b.end());
      CHECK(a == b);
      all.repeatSamples(3);
      CHECK(all.pictures.size() == 45 && all.pictures[0] == all.pictures[15] && all.pictures[14] == all.pictures[44]);
      all.pictures.resize(15);
      int kept = 0;
      for (auto p : all.pictures) kept += (p->label == 1 || p->label == 3);
      all.subsetOfClasses({3, 1}); // keeps classes 3 and 1 as 0 and 1, deletes the other pictures
      CHECK((int)all.pictures.size() == kept && all.nClasses == 2);
      for (auto p : all.pictures) CHECK(p->label == 0 || p->label == 1);
      for (auto p : all.pictures) delete p;
      for (auto p : val.pictures) delete p;
      CHECK(globVector("/nonexistent-dir-for-this-test/*").empty());
      std::printf("OK data set helpers\n");
    }
    // ---- 9. the stand-alone backward passes (MaxPoolingLayer.h:8, ConvolutionalLayer.h:41, SigmoidLayer.h:7) and SigmoidLayer
    {
      vectorCUDA<float> d1(false, 0), d2(false, 0);
      vectorCUDA<int> choice(false, 0), rules(false, 0);
      d1.hVector() = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f};
      d2.hVector() = {1.f, 2.f, 3.f, 4.f};
      choice.hVector() = {0, 5, 0, 2};
      maxPoolBackProp(d1.dPtr(), d2.dPtr(), 2, 2, choice.dPtr(), cnn.memStream); // adds onto what d1 holds
      cudaStreamSynchronize(cnn.memStream.stream);
      CHECK((d1.hVector() == std::vector<float>{5.f, 1.f, 5.f, 1.f, 1.f, 3.f}));
      vectorCUDA<float> in(false, 0), out(false, 0);
      in.hVector() = {1.f, 1.f, 1.f, 1.f};
      out.hVector() = {1.f, 2.f, 3.f, 4.f, 5.f, 6.f};
      rules.hVector() = {1, -1, 0};
      propBackwardFromMatrixMultiply(in.dPtr(), out.dPtr(), rules.dPtr(), 3, 2, cnn.memStream);
      cudaStreamSynchronize(cnn.memStream.stream);
      CHECK((in.hVector() == std::vector<float>{6.f, 7.f, 2.f, 3.f}));
      SpatiallySparseBatchSubInterface subIn, subOut;
      SpatiallySparseBatchInterface I(&subIn), O(&subOut);
      I.nSpatialSites = O.nSpatialSites = 1; I.nFeatures = O.nFeatures = 4;
      I.featuresPresent.hVector() = range(4); O.featuresPresent.hVector() = range(4);
      I.backpropErrors = true;
      subIn.features.hVector() = {-3.f, -1.f, 0.5f, 2.f};
      SpatiallySparseBatch &none = cnn.batchPool[0]; // (the layer does not read it)
      SigmoidLayer leaky(cnn.memStream, VLEAKYRELU);
      leaky.forwards(none, I, O);
      cudaStreamSynchronize(cnn.memStream.stream);
      std::vector<float> f = subOut.features.hVector();
      CHECK(std::fabs(f[0] + 0.999f) < 1e-6f && std::fabs(f[1] + 0.333f) < 1e-6f && f[2] == 0.5f && f[3] == 2.f);
      subOut.dfeatures.hVector() = {10.f, 10.f, 10.f, 10.f};
      leaky.backwards(none, I, O, 0.f, 0.f);
      cudaStreamSynchronize(cnn.memStream.stream);
      std::vector<float> g = subIn.dfeatures.hVector();
      CHECK(std::fabs(g[0] - 3.33f) < 1e-5f && std::fabs(g[1] - 3.33f) < 1e-5f && g[2] == 10.f && g[3] == 10.f);
      CHECK(leaky.calculateInputSpatialSize(7) == 7);
      // the cuBLAS wrappers' signatures (utilities.h:82-102): C[2 x 2] = A^t B with A stored 3 x 2, B 3 x 2
      vectorCUDA<float> mA(false, 0), mB(false, 0), mC(false, 0);
      mA.hVector() = {1.f, 2.f, 3.f, 4.f, 5.f, 6.f};
      mB.hVector() = {1.f, 0.f, 0.f, 1.f, 1.f, 1.f};
      mC.hVector() = {100.f, 100.f, 100.f, 100.f};
      d_rowMajorSGEMM_alphaAtB_betaC(cnn.cublasHandle, mA.dPtr(), mB.dPtr(), mC.dPtr(), 2, 3, 2, 1.0f, 0.5f, __FILE__, __LINE__);
      cudaDeviceSynchronize();
      CHECK((mC.hVector() == std::vector<float>{56.f, 58.f, 58.f, 60.f}));
      std::printf("OK stand-alone backward passes\n");
    }
    for (auto p : pics) delete p;
  } catch (const std::exception &e) {
    std::printf("FAILED with exception: %s\n", e.what());
    return 1;
  }
  std::printf("ALL OK\n");
  return 0;
}
