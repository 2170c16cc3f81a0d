// TEST INFRASTRUCTURE ONLY -- the parity oracle.  A CPU restatement, in independent code, of
// the forward (inference) path of btgraham/SparseConvNet-archived.  Only tests/, the smoke
// check and the benchmark's CPU-baseline legs may load this library; the product never
// does, and has no CPU fallback.
//
// Pinning status:
//   * rule construction and the scalar helpers are PINNED: tests compare them with the
//     reference's own Regions.cu / utilities.cu compiled here (oracle/_ref, see
//     oracle/Makefile) on random grids, and with golden vectors generated from that build;
//   * the floating-point layers restate CUDA kernels and a cuBLAS SGEMM that cannot run in a
//     GPU-less container and that no reference test pins: FLOAT PARITY UNPINNED.  They
//     follow the reference source line by line in meaning (citations below).
//
// All citations are paths inside the reference project (SparseConvNet/...).
#include <random>
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

namespace orc {

// ------------------------------------------------------------------ scalar helpers
// utilities.cu:14-26 (integer power by squaring).
static int ipow(int base, int exp) {
  int r = 1;
  for (; exp; exp >>= 1, base *= base)
    if (exp & 1) r *= base;
  return r;
}
// utilities.cu:27-32: binomial(linearSize+dimension-1, dimension), evaluated with the same
// left-to-right integer arithmetic.
static int triangleSize(int linearSize, int dimension) {
  int fs = 1;
  for (int i = 1; i <= dimension; ++i) fs = fs * (linearSize + dimension - i) / i;
  return fs;
}
// utilities.cu:103.
static int intRound(int a, int d) { return (int)(std::round(a * 1.0 / d) * d); }

enum Act { NOSIGMOID = 0, RELU, VLEAKYRELU, LEAKYRELU, TANH, SOFTMAX, PRELU, SIGMOID }; // types.h:20-29

// ------------------------------------------------------------------ grids
// A SparseGrid (SparseGrid.h:68-77) held as its ascending-key iteration order, which is what
// the vectorHash backend yields (vectorHash.cpp:40-55).
struct Grid {
  std::vector<std::pair<int64_t, int>> sites; // (key, row), ascending key
  int bg = -1;                                 // backgroundCol
  int find(int64_t key) const {
    auto it = std::lower_bound(sites.begin(), sites.end(), std::make_pair(key, INT32_MIN));
    return (it != sites.end() && it->first == key) ? it->second : INT32_MIN;
  }
};

struct Regions { // RegularSquareRegions (Regions.cu:13-29) / RegularTriangularRegions (804-832)
  int kind, dim, nIn, nOut, size, stride;
  int sd;               // cells per rule row: size^dim, or triangleSize(size, dim)
  int cube;             // size^dim
  std::vector<int> ord; // triangular: cube cell -> rule column, -1 outside the simplex
  Regions(int kind, int dim, int nIn, int nOut, int size, int stride)
      : kind(kind), dim(dim), nIn(nIn), nOut(nOut), size(size), stride(stride) {
    cube = ipow(size, dim);
    ord.assign(cube, -1);
    int S = 0;
    for (int c = 0; c < cube; ++c) {
      int j = c, J = 0;
      while (j > 0) { J += j % size; j /= size; }
      if (kind == 0 || J < size) ord[c] = S++;
    }
    sd = S;
  }
  int inputL(int j) const { return j * stride; }
  int outputL(int i) const { return std::max(0, (i - size + stride) / stride); }
  int outputR(int i) const { return std::min(i / stride + 1, nOut); }
  long long fullSize() const { return kind == 0 ? ipow(nOut, dim) : triangleSize(nOut, dim); }
};

static void decode(int64_t key, int n, int dim, int *c) {
  for (int a = dim - 1; a >= 0; --a) { c[a] = (int)(key % n); key /= n; }
}
static int64_t encode(const int *c, int n, int dim) {
  int64_t k = 0;
  for (int a = 0; a < dim; ++a) k = k * n + c[a];
  return k;
}

// Visit the box [lo, hi) in lexicographic order (axis 0 most significant).
template <class F> static void forBox(int dim, const int *lo, const int *hi, F f) {
  int c[4];
  for (int a = 0; a < dim; ++a) { if (lo[a] >= hi[a]) return; c[a] = lo[a]; }
  for (;;) {
    f(c);
    int a = dim - 1;
    while (a >= 0 && ++c[a] >= hi[a]) { c[a] = lo[a]; --a; }
    if (a < 0) return;
  }
}

// One sample of gridRules (dispatch Regions.cu:782-802 and 1166-1174).
//   minActive == 1 : OverlappingNoMin (528-653) / triangular NoMin (834-970)
//   minActive  > 1 : OverlappingMin   (338-526) / triangular Min   (972-1164)
//   minActive == -1: Valid (658-780), square lattices only
static void gridRules(const Grid &in, Grid &out, const Regions &R, int &nOutSites,
                      std::vector<int> &rules, int minActive) {
  const int dim = R.dim;
  std::unordered_map<int64_t, int> created; // output key -> row, or -2 for a rejected site
  std::vector<std::pair<int64_t, int>> outSites;
  int i[4], lo[4], hi[4];
  const bool tri = R.kind == 1;

  auto fieldRow = [&](const int *j, int &active) { // push one rule row by probing the field
    int flo[4], fhi[4];
    for (int a = 0; a < dim; ++a) { flo[a] = R.inputL(j[a]); fhi[a] = flo[a] + R.size; }
    active = 0;
    int cell = 0;
    forBox(dim, flo, fhi, [&](const int *ii) {
      if (R.ord[cell++] < 0) return; // outside the triangular filter: no column
      int r = in.find(encode(ii, R.nIn, dim));
      if (r == INT32_MIN) rules.push_back(in.bg);
      else { rules.push_back(r); ++active; }
    });
  };

  if (minActive == -1) { // Regions.cu:688-712: output sites are the interior input sites
    for (auto &s : in.sites) {
      decode(s.first, R.nIn, dim, i);
      bool interior = true;
      int j[4];
      for (int a = 0; a < dim; ++a) { interior = interior && i[a] >= 1 && i[a] <= R.nOut; j[a] = i[a] - 1; }
      if (!interior) continue;
      int active;
      outSites.emplace_back(encode(j, R.nOut, dim), nOutSites++);
      fieldRow(j, active);
    }
  } else {
    for (auto &s : in.sites) {
      decode(s.first, R.nIn, dim, i);
      for (int a = 0; a < dim; ++a) { lo[a] = R.outputL(i[a]); hi[a] = R.outputR(i[a]); }
      forBox(dim, lo, hi, [&](const int *j) {
        if (tri) { int sum = 0; for (int a = 0; a < dim; ++a) sum += j[a]; if (sum >= R.nOut) return; }
        int64_t outKey = encode(j, R.nOut, dim);
        auto f = created.find(outKey);
        if (minActive == 1) {
          if (f == created.end()) {
            f = created.emplace(outKey, nOutSites++).first;
            outSites.emplace_back(outKey, f->second);
            rules.resize((size_t)nOutSites * R.sd, in.bg);
          }
          int cell = 0;
          for (int a = 0; a < dim; ++a) cell = cell * R.size + (i[a] - R.inputL(j[a]));
          int col = R.ord[cell];
          if (col > -1) rules[(size_t)f->second * R.sd + col] = s.second;
        } else if (f == created.end()) {
          int active;
          fieldRow(j, active);
          if (active >= minActive) {
            created.emplace(outKey, nOutSites);
            outSites.emplace_back(outKey, nOutSites++);
          } else {
            created.emplace(outKey, -2);
            rules.resize((size_t)nOutSites * R.sd);
          }
        }
      });
    }
  }
  std::sort(outSites.begin(), outSites.end());
  out.sites = outSites;
  out.bg = -1;
  if ((long long)outSites.size() < R.fullSize()) { // e.g. Regions.cu:647-652
    for (int c = 0; c < R.sd; ++c) rules.push_back(in.bg);
    out.bg = nOutSites++;
  }
}

// ------------------------------------------------------------------ fractional max-pooling
// The reference's RNG (Rng.h, Rng.cpp:16-21, 59-61): a std::mt19937 behind a double-valued
// uniform_real_distribution whose result passes through float, and std::shuffle.
struct FmpRng {
  std::mt19937 gen;
  std::uniform_real_distribution<> uniform01{0, 1};
  float uniform(float a = 0, float b = 1) { return a + (b - a) * uniform01(gen); }
};
// FractionalMaxPoolingTicks of one axis (Regions.h:48-54).  kind: 0 pseudorandom overlapping
// (Regions.cu:31-52), 1 pseudorandom non-overlapping (54-74), 2 random overlapping (76-100),
// 3 random non-overlapping (102-125).
struct Ticks { std::vector<int> inputL, inputR, outputL, outputR; };
static Ticks makeTicks(int kind, int nIn, int nOut, int poolSize, FmpRng &rng) {
  Ticks t;
  if (kind == 0 || kind == 1) {
    const double alpha = kind == 0 ? (nIn - poolSize) * 1.0 / (nOut - 1) : nIn * 1.0 / nOut;
    const double u = rng.uniform(0, 1);
    for (int j = 0; j < nOut; ++j) {
      const int i = (int)((j + u) * alpha) - (int)(u * alpha);
      t.inputL.push_back(i);
      t.inputR.push_back(kind == 0 ? i + poolSize : (int)((j + 1 + u) * alpha) - (int)(u * alpha));
    }
  } else {
    const int alpha = (int)(nIn * 1.0 / nOut);
    std::vector<int> inc;
    inc.resize(nOut * (alpha + 1) - nIn, alpha);
    inc.resize(kind == 2 ? nOut - 1 : nOut, alpha + 1);
    std::shuffle(inc.begin(), inc.end(), rng.gen);
    t.inputL.push_back(0);
    t.inputR.push_back(kind == 2 ? poolSize : inc[0]);
    for (int i = 0; i < nOut - 1; ++i) {
      t.inputL.push_back(t.inputL.back() + inc[i]);
      t.inputR.push_back(kind == 2 ? t.inputL.back() + poolSize : t.inputR.back() + inc[i + 1]);
    }
  }
  t.outputL.assign(nIn, nOut);
  t.outputR.assign(nIn, 0);
  for (int i = 0; i < nOut; ++i)
    for (int j = t.inputL[i]; j < t.inputR[i] && j < nIn; ++j) {
      t.outputL[j] = std::min(t.outputL[j], i);
      t.outputR[j] = std::max(t.outputR[j], i + 1);
    }
  return t;
}
// gridRules with tick tables: gridRulesOverlappingNoMin (Regions.cu:528-653) when overlapping,
// gridRulesNonOverlapping (159-336) otherwise; the two differ in what a new rule row holds outside
// the (variable-size) pooling region: the background row, or -1.
static void gridRulesFmp(const Grid &in, Grid &out, const Ticks *pb, int dim, int nIn, int nOut, int s, bool overlapping,
                         int &nOutSites, std::vector<int> &rules) {
  const int sd = ipow(s, dim);
  std::unordered_map<int64_t, int> created;
  std::vector<std::pair<int64_t, int>> outSites;
  int i[4], lo[4], hi[4];
  for (auto &site : in.sites) {
    decode(site.first, nIn, dim, i);
    for (int a = 0; a < dim; ++a) { lo[a] = pb[a].outputL[i[a]]; hi[a] = pb[a].outputR[i[a]]; }
    forBox(dim, lo, hi, [&](const int *j) {
      const int64_t outKey = encode(j, nOut, dim);
      auto f = created.find(outKey);
      if (f == created.end()) {
        f = created.emplace(outKey, nOutSites++).first;
        outSites.emplace_back(outKey, f->second);
        rules.resize((size_t)nOutSites * sd, overlapping ? in.bg : -1);
        if (!overlapping) { // Regions.cu:206-215: the cells of this site's own region start as background
          int zero[4] = {0, 0, 0, 0}, ext[4];
          for (int a = 0; a < dim; ++a) ext[a] = pb[a].inputR[j[a]] - pb[a].inputL[j[a]];
          forBox(dim, zero, ext, [&](const int *cc) {
            int k = 0;
            for (int a = 0; a < dim; ++a) k = k * s + cc[a];
            rules[(size_t)f->second * sd + k] = in.bg;
          });
        }
      }
      int off = 0;
      for (int a = 0; a < dim; ++a) off = off * s + (i[a] - pb[a].inputL[j[a]]);
      rules[(size_t)f->second * sd + off] = site.second;
    });
  }
  std::sort(outSites.begin(), outSites.end());
  out.sites = outSites;
  out.bg = -1;
  if ((long long)outSites.size() < ipow(nOut, dim)) { // Regions.cu:330-335, 647-652
    for (int c = 0; c < sd; ++c) rules.push_back(in.bg);
    out.bg = nOutSites++;
  }
}

// TerminalPoolingLayer.cu:8-20.
static void terminalRules(const Grid &in, Grid &out, int S, int &nOutSites, std::vector<int> &rules) {
  if (in.sites.empty()) rules.push_back(in.bg);
  else for (auto &s : in.sites) rules.push_back(s.second);
  out.sites.assign(1, std::make_pair((int64_t)0, nOutSites++));
  out.bg = -1;
  rules.resize((size_t)S * nOutSites, -1);
}

// ------------------------------------------------------------------ float layers
// ConvolutionalLayer.cu:12-31: row gather.  The reference does not test for a negative rule;
// here -1 yields a zero row (the only defined reading).
static void gather(const float *feat, const int *rules, long long count, int nIn, float *out) {
  for (long long c = 0; c < count; ++c) {
    if (rules[c] >= 0) std::memcpy(out + c * nIn, feat + (long long)rules[c] * nIn, sizeof(float) * nIn);
    else std::memset(out + c * nIn, 0, sizeof(float) * nIn);
  }
}

static inline float activate(float v, int act, float slope) {
  switch (act) {
  case RELU: return v > 0 ? v : 0;                         // SigmoidLayer.cu:9
  case VLEAKYRELU: return v > 0 ? v : v * 0.333f;          // SigmoidLayer.cu:121, 209-213
  case LEAKYRELU: return v > 0 ? v : v * 0.01f;            // SigmoidLayer.cu:121, 204-208
  case TANH: return std::tanh(v);                          // SigmoidLayer.cu:83
  case SIGMOID: return 1.0f / (1.0f + std::exp(-v));       // SigmoidLayer.cu:46
  case PRELU: return v > 0 ? v : v * slope;                // NetworkInNetworkPReLULayer.cu:12-13
  default: return v;
  }
}

// NetworkInNetworkLayer.cu:187-195 (test branch): out = p*(X W) + p*B, then applySigmoid.
// Acc = float restates the fp32 arithmetic; Acc = double is the high-precision checker.
template <class Acc>
static void ninForward(const float *X, long long rows, int K, const float *W, const float *B,
                       const float *prelu, int N, float p, int act, float *out) {
  std::vector<Acc> acc(N);
  for (long long r = 0; r < rows; ++r) {
    std::fill(acc.begin(), acc.end(), (Acc)0);
    const float *x = X + r * K;
    for (int k = 0; k < K; ++k) {
      const Acc xv = x[k];
      if (xv == 0) continue;
      const float *w = W + (long long)k * N;
      for (int n = 0; n < N; ++n) acc[n] += xv * (Acc)w[n];
    }
    float *o = out + r * N;
    for (int n = 0; n < N; ++n) o[n] = (float)((Acc)p * acc[n] + (Acc)p * (Acc)B[n]);
    if (act == SOFTMAX) { // SigmoidLayer.cu:160-176 (max starts at -10000)
      float mx = -10000.0f, sum = 0.0f;
      for (int n = 0; n < N; ++n) if (o[n] > mx) mx = o[n];
      for (int n = 0; n < N; ++n) { o[n] = std::exp(o[n] - mx); sum += o[n]; }
      for (int n = 0; n < N; ++n) o[n] /= sum;
    } else if (act != NOSIGMOID) {
      for (int n = 0; n < N; ++n) o[n] = activate(o[n], act, prelu ? prelu[n] : 0.0f);
    }
  }
}

// MaxPoolingLayer.cu:9-35: negative rules are skipped, the first maximum wins (strict '<'),
// the choice is the flat input index rule*C + channel.  A row with no usable rule is left
// at 0 / -1 here (the reference stores uninitialised registers).
static void maxPool(const float *in, const int *rules, long long rowsOut, int sd, int C, float *out, int *choice) {
  for (long long r = 0; r < rowsOut; ++r)
    for (int j = 0; j < C; ++j) {
      bool none = true; float t = 0; int c = -1;
      for (int p = 0; p < sd; ++p) {
        int rp = rules[r * sd + p];
        if (rp < 0) continue;
        float s = in[(long long)rp * C + j];
        if (none || t < s) { none = false; t = s; c = rp * C + j; }
      }
      out[r * C + j] = t; choice[r * C + j] = c;
    }
}

// TerminalPoolingLayer.cu:22-34: mean over the rules up to the first negative one.
static void terminalPool(const float *in, const int *rules, int count, int S, int C, float *out) {
  for (int b = 0; b < count; ++b)
    for (int j = 0; j < C; ++j) {
      float t = 0; int p = 0;
      for (; p < S && rules[b * S + p] >= 0; ++p) t += in[(long long)rules[b * S + p] * C + j];
      out[b * C + j] = t / p;
    }
}

// utilities.cu:35-56 (insertion top-k; needs n >= k >= 1).
static void topIndices(const float *test, int n, int k, int *indices) {
  std::vector<float> q(k);
  for (int i = 0; i < k; ++i) indices[i] = 0;
  q[0] = test[0];
  for (int i = 1; i < n; i++) {
    int j = std::min(i, k);
    if (test[i] > q[j - 1]) {
      if (i >= k) --j;
      for (; j > 0 && test[i] > q[j - 1]; --j) { q[j] = q[j - 1]; indices[j] = indices[j - 1]; }
    }
    if (j < k) { q[j] = test[i]; indices[j] = i; }
  }
}

// ------------------------------------------------------------------ network
enum LayerType { L_CONV = 0, L_CONV_TRI, L_NIN, L_MAXPOOL, L_MAXPOOL_TRI, L_TERMINAL, L_FMP };

struct Layer {
  int type;
  int size = 1, stride = 1, minActive = 1; // geometry layers
  int nIn = 0, nOut = 0;                    // features in/out
  int fs = 1;                               // cells per rule row
  int act = NOSIGMOID; float dropout = 0;   // NiN
  int S = 0;                                // terminal pooling constructor argument
  int fmpKind = 0; float fmpShrink = 1;     // fractional max-pooling: tick kind (see makeTicks), shrink factor
  int inSpatial = 0, outSpatial = 0;
  std::vector<float> W, B, prelu;
  std::vector<float> MW, MB, Mprelu; // momentum of the training step (zero until the first one)
  // Training-time dropout (NetworkInNetworkLayer.cu:152-154): the output features the next training step keeps, ascending;
  // empty = all of them.  The reference draws them at random per batch; here the caller names them (orc_net_set_dropout_features),
  // so that two implementations can run the same step.
  std::vector<int> present;
};

// 0/1 per output feature of learnt layer `l` for a training step, or empty when the step keeps them all.
static std::vector<char> keptMask(const Layer &L) {
  std::vector<char> m;
  if (L.present.empty() || (int)L.present.size() >= L.nOut) return m;
  m.assign(L.nOut, 0);
  for (int f : L.present) m[f] = 1;
  return m;
}

struct Iface { // SpatiallySparseBatchInterface.h:19-46, host side only
  int nFeatures = 0, spatialSize = 0, nSpatialSites = 0;
  std::vector<Grid> grids;
  std::vector<int> rules;
  std::vector<float> features;
  std::vector<int> choices;
  std::vector<float> dfeatures; // training step only: d cost / d features
};

struct Net {
  int dim, nInputFeatures, nClasses, nTop;
  int nOutputFeatures;
  int inputSpatialSize = 0;
  std::vector<Layer> layers;
  std::vector<Iface> kept; // last forward (keep=1): interface i+1 is layer i's output
  unsigned fmpSeed = 1;    // each forward re-seeds FMP layer l's RNG with fmpSeed + l (the reference seeds from the clock)

  // SparseConvNetCUDA.cu:50-70.
  void addLearntLayer(int nFeatures, int act, float dropout) {
    if (act != SOFTMAX) nFeatures = std::max(32, intRound(nFeatures, 32));
    if (dropout > 0) dropout = 1 - (intRound(nFeatures * (1 - dropout), 32) + 0.01f) * 1.0f / nFeatures;
    if (dropout < 0) dropout = 0;
    Layer L; L.type = L_NIN; L.nIn = nOutputFeatures; L.nOut = nFeatures; L.act = act; L.dropout = dropout;
    L.W.assign((size_t)L.nIn * L.nOut, 0.0f); L.B.assign(L.nOut, 0.0f);
    if (act == PRELU) L.prelu.assign(L.nOut, 0.25f); // NetworkInNetworkPReLULayer.cu:6
    layers.push_back(L);
    nOutputFeatures = nFeatures;
  }
  // SparseConvNetCUDA.cu:75-98 (the disabled ReallyConvolutionalLayer branch is dead code).
  void addConvolutionalLayer(int nFeatures, int fsz, int fstride, int act, float dropout, int minActive) {
    if (fsz > 1) {
      Layer L; L.type = L_CONV; L.size = fsz; L.stride = fstride; L.minActive = minActive;
      L.nIn = nOutputFeatures; L.fs = ipow(fsz, dim); L.nOut = L.fs * L.nIn;
      layers.push_back(L);
      nOutputFeatures *= L.fs;
    }
    addLearntLayer(nFeatures, act, dropout);
  }
  // SparseConvNetCUDA.cu:99-111.
  void addLeNetLayerMP(int nFeatures, int fsz, int fstride, int ps, int pstride, int act, float dropout, int minActive) {
    addConvolutionalLayer(nFeatures, fsz, fstride, act, dropout, minActive);
    if (ps > 1) { Layer L; L.type = L_MAXPOOL; L.size = ps; L.stride = pstride; L.fs = ipow(ps, dim); L.nIn = L.nOut = nOutputFeatures; layers.push_back(L); }
  }
  // SparseConvNetCUDA.cu:165-181.
  void addTriangularConvolutionalLayer(int nFeatures, int fsz, int fstride, int act, float dropout, int minActive) {
    if (fsz > 1) {
      Layer L; L.type = L_CONV_TRI; L.size = fsz; L.stride = fstride; L.minActive = minActive;
      L.nIn = nOutputFeatures; L.fs = triangleSize(fsz, dim); L.nOut = L.fs * L.nIn;
      layers.push_back(L);
      nOutputFeatures *= L.fs;
    }
    addLearntLayer(nFeatures, act, dropout);
  }
  // SparseConvNetCUDA.cu:182-194: poolSize is handed over in the minActiveInputs slot (and
  // minActiveInputs in the poolingToFollow slot, which only affects weight initialisation).
  void addTriangularLeNetLayerMP(int nFeatures, int fsz, int fstride, int ps, int pstride, int act, float dropout, int minActive) {
    (void)minActive;
    addTriangularConvolutionalLayer(nFeatures, fsz, fstride, act, dropout, /*minActiveInputs=*/ps);
    if (ps > 1) { Layer L; L.type = L_MAXPOOL_TRI; L.size = ps; L.stride = pstride; L.fs = triangleSize(ps, dim); L.nIn = L.nOut = nOutputFeatures; layers.push_back(L); }
  }
  // SparseConvNetCUDA.cu:112-163 (addLeNetLayer{PO,PD,RO,RD}FMP): convolution block, then the FMP layer
  // if it shrinks at all.
  void addLeNetLayerFMP(int kind, int nFeatures, int fsz, int fstride, int ps, float shrink, int act, float dropout, int minActive) {
    addConvolutionalLayer(nFeatures, fsz, fstride, act, dropout, minActive);
    if (shrink > 1) { Layer L; L.type = L_FMP; L.fmpKind = kind; L.fmpShrink = shrink; L.size = ps; L.fs = ipow(ps, dim); L.nIn = L.nOut = nOutputFeatures; layers.push_back(L); }
  }
  // SparseConvNetCUDA.cu:196-199.
  void addTerminalPoolingLayer(int poolSize, int S) {
    Layer L; L.type = L_TERMINAL; L.size = poolSize; L.S = S; L.nIn = L.nOut = nOutputFeatures; layers.push_back(L);
  }
  // SparseConvNetCUDA.cu:200-213 with each layer's calculateInputSpatialSize
  // (ConvolutionalLayer.cu:148-156, MaxPoolingLayer.cu:147-155, TerminalPoolingLayer.cu:126-130).
  void addSoftmaxLayer() {
    addLearntLayer(nClasses, SOFTMAX, 0.0f);
    int s = 1;
    for (int i = (int)layers.size() - 1; i >= 0; --i) {
      Layer &L = layers[i];
      L.outSpatial = s;
      if (L.type == L_NIN) L.inSpatial = s;
      else if (L.type == L_TERMINAL) L.inSpatial = L.size;
      else if (L.type == L_FMP) { // MaxPoolingLayer.cu:216-223: int * float, + 0.5, truncated
        const float prod = s * L.fmpShrink;
        L.inSpatial = (int)(prod + 0.5);
        if (L.inSpatial == s) L.inSpatial++;
      }
      else L.inSpatial = L.size + (s - 1) * L.stride;
      s = L.inSpatial;
    }
    inputSpatialSize = s;
  }
};

// ------------------------------------------------------------------------------------------ backward pass
// The reference's training step for one batch (SparseConvNetCUDA.cu:247-251: every layer's backwards() in
// reverse order behind SoftmaxClassifier), restated for layers without training-time dropout.

// SoftmaxClassifier.cu:7-14: d cost / d (softmax input) = probabilities - one_hot(label), not averaged over the batch.
static void softmaxNllBackward(const float *probs, const int *labels, int rows, int N, float *d) {
  for (int r = 0; r < rows; ++r)
    for (int n = 0; n < N; ++n) d[(size_t)r * N + n] = probs[(size_t)r * N + n] - (n == labels[r] ? 1.0f : 0.0f);
}
// applySigmoidBackProp in place on the output's dfeatures, from the output's (activated) features
// (SigmoidLayer.cu:224-268 and the kernels it dispatches to; softmax and NOSIGMOID pass through).  PReLU:
// NetworkInNetworkPReLULayer.cu:25-38, which also accumulates the slope gradient sum_rows d * (b > 0 ? 0 : b / slope).
template <class Acc>
static void activationBackward(const float *b, float *d, long long rows, int N, int act, const float *prelu, float *dprelu) {
  std::vector<Acc> ds(act == PRELU ? N : 0, (Acc)0);
  for (long long r = 0; r < rows; ++r)
    for (int n = 0; n < N; ++n) {
      const size_t i = (size_t)r * N + n;
      switch (act) {
      case RELU: d[i] = b[i] > 0 ? d[i] : 0; break;
      case VLEAKYRELU: d[i] = b[i] > 0 ? d[i] : d[i] * 0.333f; break;
      case LEAKYRELU: d[i] = b[i] > 0 ? d[i] : d[i] * 0.01f; break;
      case TANH: d[i] = d[i] * (1 + b[i]) * (1 - b[i]); break;
      case SIGMOID: d[i] = d[i] * b[i] * (1 - b[i]); break;
      case PRELU:
        ds[n] += (Acc)d[i] * (b[i] > 0 ? (Acc)0 : (Acc)(b[i] / prelu[n]));
        d[i] = b[i] > 0 ? d[i] : d[i] * prelu[n];
        break;
      default: break;
      }
    }
  if (act == PRELU) for (int n = 0; n < N; ++n) dprelu[n] = (float)ds[n];
}
// NetworkInNetworkLayer.cu:226-239, 266-277 (no dropout): dW = X^T d, dB = column sums of d, dX = d W^T.
template <class Acc>
static void ninBackward(const float *X, const float *d, long long rows, int K, int N, const float *W, float *dW, float *dB, float *dX) {
  std::vector<Acc> aw((size_t)K * N, (Acc)0), ab(N, (Acc)0);
  for (long long r = 0; r < rows; ++r) {
    const float *x = X + r * K, *dr = d + r * N;
    for (int n = 0; n < N; ++n) ab[n] += dr[n];
    for (int k = 0; k < K; ++k) {
      const Acc xv = x[k];
      if (xv == 0) continue;
      Acc *a = aw.data() + (size_t)k * N;
      for (int n = 0; n < N; ++n) a[n] += xv * (Acc)dr[n];
    }
  }
  for (size_t i = 0; i < aw.size(); ++i) dW[i] = (float)aw[i];
  for (int n = 0; n < N; ++n) dB[n] = (float)ab[n];
  if (dX) {
    std::vector<Acc> ax(K);
    for (long long r = 0; r < rows; ++r) {
      const float *dr = d + r * N;
      for (int k = 0; k < K; ++k) {
        const float *w = W + (size_t)k * N;
        Acc t = 0;
        for (int n = 0; n < N; ++n) t += (Acc)dr[n] * (Acc)w[n];
        dX[r * K + k] = (float)t;
      }
    }
  }
}
// NetworkInNetworkLayer.cu:26-40 ("NAG light"), one parameter array; keepPositive: the PReLU slopes' variant
// (NetworkInNetworkPReLULayer.cu:67-84).
static void sgdUpdate(float *w, float *m, const float *d, size_t n, float lr, float momentum, bool keepPositive = false) {
  for (size_t i = 0; i < n; ++i) {
    float wi = w[i], mi = m[i];
    wi -= mi * momentum;
    mi = momentum * mi - lr * (1 - momentum) * d[i];
    wi += mi * (1 + momentum);
    if (keepPositive) wi = (wi > 0.001) ? wi : 0.001f;
    w[i] = wi; m[i] = mi;
  }
}
// ConvolutionalLayer.cu:42-59: the gathered matrix's gradient added back onto the rows it was gathered from.
template <class Acc>
static void gatherBackward(const float *dConv, const int *rules, long long count, int nIn, long long rowsIn, float *dIn) {
  std::vector<Acc> acc((size_t)rowsIn * nIn, (Acc)0);
  for (long long c = 0; c < count; ++c)
    if (rules[c] >= 0)
      for (int j = 0; j < nIn; ++j) acc[(size_t)rules[c] * nIn + j] += dConv[c * nIn + j];
  for (size_t i = 0; i < acc.size(); ++i) dIn[i] = (float)acc[i];
}
// MaxPoolingLayer.cu:74-80: the pooled gradient added onto the inputs the forward pass chose.
template <class Acc>
static void maxPoolBackward(const float *dOut, const int *choice, long long n, long long nIn, float *dIn) {
  std::vector<Acc> acc((size_t)nIn, (Acc)0);
  for (long long i = 0; i < n; ++i) if (choice[i] >= 0) acc[choice[i]] += dOut[i];
  for (long long i = 0; i < nIn; ++i) dIn[i] = (float)acc[i];
}
// TerminalPoolingLayer.cu:48-62: every pooled input row receives the gradient divided by the number of rows pooled (stored, not added).
static void terminalPoolBackward(const float *dOut, const int *rules, int count, int S, int C, long long rowsIn, float *dIn) {
  std::fill(dIn, dIn + rowsIn * C, 0.0f);
  for (int b = 0; b < count; ++b) {
    int maxP = 0;
    while (maxP < S && rules[b * S + maxP] >= 0) ++maxP;
    for (int j = 0; j < C; ++j) {
      const float t = dOut[b * C + j] / maxP;
      for (int p = 0; p < maxP; ++p) dIn[(long long)rules[b * S + p] * C + j] = t;
    }
  }
}

// Every layer's preprocess() then forwards(), in the order BatchProducer.cu:72-75 and
// SparseConvNetCUDA.cu:242-246 run them.  Input rows of sample b are [off[b], off[b+1]);
// keys[row] is the site key, or -1 for the sample's background ("null vector") row.
static void forwardChunk(const Net &net, int batch, const int64_t *keys, const int *off, const float *features,
                         bool accum64, std::vector<Iface> &ifs, double *tRules,
                         const std::vector<std::vector<Ticks>> &fmpTicks, int firstSample, bool training = false) {
  auto t0 = std::chrono::steady_clock::now();
  ifs.assign(net.layers.size() + 1, Iface());
  Iface &I0 = ifs[0];
  const int base = off[0];
  I0.nFeatures = net.nInputFeatures; I0.spatialSize = net.inputSpatialSize; I0.nSpatialSites = off[batch] - base;
  I0.grids.resize(batch);
  for (int b = 0; b < batch; ++b) {
    for (int r = off[b]; r < off[b + 1]; ++r) {
      if (keys[r] < 0) I0.grids[b].bg = r - base;
      else I0.grids[b].sites.emplace_back(keys[r], r - base);
    }
    std::sort(I0.grids[b].sites.begin(), I0.grids[b].sites.end());
  }
  // geometry chain (the reference's host hot loop)
  for (size_t l = 0; l < net.layers.size(); ++l) {
    const Layer &L = net.layers[l];
    Iface &in = ifs[l], &out = ifs[l + 1];
    out.nFeatures = L.nOut;
    if (L.type == L_NIN) { // NetworkInNetworkLayer.cu:145-156
      out.spatialSize = in.spatialSize; out.nSpatialSites = in.nSpatialSites; out.grids = in.grids;
    } else if (L.type == L_TERMINAL) { // TerminalPoolingLayer.cu:81-99
      out.spatialSize = 1; out.grids.resize(batch);
      size_t s = 1;
      for (int b = 0; b < batch; ++b) s = std::max(s, in.grids[b].sites.size());
      for (int b = 0; b < batch; ++b) terminalRules(in.grids[b], out.grids[b], (int)s, out.nSpatialSites, out.rules);
    } else if (L.type == L_FMP) { // MaxPoolingLayer.cu:171-186 and its three siblings
      out.spatialSize = L.outSpatial; out.grids.resize(batch);
      for (int b = 0; b < batch; ++b)
        gridRulesFmp(in.grids[b], out.grids[b], &fmpTicks[l][(size_t)(firstSample + b) * net.dim], net.dim, L.inSpatial, L.outSpatial, L.size,
                     L.fmpKind == 0 || L.fmpKind == 2, out.nSpatialSites, out.rules);
    } else {
      const bool tri = (L.type == L_CONV_TRI || L.type == L_MAXPOOL_TRI);
      const bool pool = (L.type == L_MAXPOOL || L.type == L_MAXPOOL_TRI);
      out.spatialSize = (in.spatialSize - L.size) / L.stride + 1;
      out.grids.resize(batch);
      Regions R(tri ? 1 : 0, net.dim, L.inSpatial, L.outSpatial, L.size, L.stride);
      for (int b = 0; b < batch; ++b)
        gridRules(in.grids[b], out.grids[b], R, out.nSpatialSites, out.rules, pool ? 1 : L.minActive);
    }
  }
  auto t1 = std::chrono::steady_clock::now();
  if (tRules) *tRules = std::chrono::duration<double>(t1 - t0).count();
  // feature chain
  I0.features.assign(features + (size_t)base * net.nInputFeatures, features + (size_t)off[batch] * net.nInputFeatures);
  for (size_t l = 0; l < net.layers.size(); ++l) {
    const Layer &L = net.layers[l];
    Iface &in = ifs[l], &out = ifs[l + 1];
    out.features.resize((size_t)out.nSpatialSites * L.nOut);
    switch (L.type) {
    case L_CONV: case L_CONV_TRI:
      gather(in.features.data(), out.rules.data(), (long long)out.nSpatialSites * L.fs, L.nIn, out.features.data());
      break;
    case L_NIN: {
      // A training step that drops features on either side of the layer runs on the kept ones without the test-time
      // scaling (NetworkInNetworkLayer.cu:162-186); the dropped inputs are zero columns here, the dropped outputs are zeroed.
      float p = 1.0f - L.dropout;
      std::vector<char> outMask;
      if (training) {
        outMask = keptMask(L);
        bool inDropped = false;
        for (int k = (int)l - 1; k >= 0; --k)
          if (net.layers[k].type == L_NIN) { inDropped = !keptMask(net.layers[k]).empty(); break; }
        if (!outMask.empty() || inDropped) p = 1.0f;
      }
      if (accum64) ninForward<double>(in.features.data(), out.nSpatialSites, L.nIn, L.W.data(), L.B.data(), L.prelu.empty() ? nullptr : L.prelu.data(), L.nOut, p, L.act, out.features.data());
      else ninForward<float>(in.features.data(), out.nSpatialSites, L.nIn, L.W.data(), L.B.data(), L.prelu.empty() ? nullptr : L.prelu.data(), L.nOut, p, L.act, out.features.data());
      if (!outMask.empty())
        for (long long r = 0; r < out.nSpatialSites; ++r)
          for (int n = 0; n < L.nOut; ++n)
            if (!outMask[n]) out.features[(size_t)r * L.nOut + n] = 0.f;
      break;
    }
    case L_MAXPOOL: case L_MAXPOOL_TRI: case L_FMP:
      out.choices.resize(out.features.size());
      maxPool(in.features.data(), out.rules.data(), out.nSpatialSites, L.fs, L.nOut, out.features.data(), out.choices.data());
      break;
    case L_TERMINAL:
      terminalPool(in.features.data(), out.rules.data(), out.nSpatialSites, (int)(out.rules.size() / batch), L.nOut, out.features.data());
      break;
    }
  }
}

// Join the interfaces of consecutive sample chunks (each numbered from row 0) into those of the whole
// batch.  Rule cells name rows of the interface in front, choices flat indices row*C + channel into its
// features; terminal-pooling rule rows are re-padded to the widest chunk's width, which is the whole
// batch's (the maximum of the per-sample site counts).
static std::vector<Iface> joinChunks(const Net &net, std::vector<std::vector<Iface>> &chunks) {
  const size_t nI = net.layers.size() + 1;
  std::vector<Iface> all(nI);
  std::vector<std::vector<long long>> rowsOf(chunks.size(), std::vector<long long>(nI, 0));
  for (size_t t = 0; t < chunks.size(); ++t)
    for (size_t i = 0; i < nI && !chunks[t].empty(); ++i) rowsOf[t][i] = chunks[t][i].nSpatialSites;
  for (size_t i = 0; i < nI; ++i) {
    const int type = i ? net.layers[i - 1].type : -1;
    int width = 0; // terminal pooling: cells per rule row of the whole batch
    if (type == L_TERMINAL)
      for (auto &c : chunks) if (!c.empty() && c[i].nSpatialSites) width = std::max(width, (int)(c[i].rules.size() / c[i].nSpatialSites));
    Iface &A = all[i];
    std::vector<long long> inBase(chunks.size(), 0);
    long long rowsIn = 0, rowsOut = 0;
    for (size_t t = 0; t < chunks.size(); ++t) { // rows in front of chunk t in the interface that feeds this one
      inBase[t] = rowsIn;
      if (i) rowsIn += rowsOf[t][i - 1];
    }
    for (size_t t = 0; t < chunks.size(); ++t) {
      if (chunks[t].empty()) continue;
      Iface &C = chunks[t][i];
      A.nFeatures = C.nFeatures; A.spatialSize = C.spatialSize;
      for (Grid g : C.grids) {
        for (auto &sr : g.sites) sr.second += (int)rowsOut;
        if (g.bg >= 0) g.bg += (int)rowsOut;
        A.grids.push_back(std::move(g));
      }
      const int w = (type == L_TERMINAL && C.nSpatialSites) ? (int)(C.rules.size() / C.nSpatialSites) : 0;
      for (size_t k = 0; k < C.rules.size(); ++k) {
        A.rules.push_back(C.rules[k] >= 0 ? C.rules[k] + (int)inBase[t] : C.rules[k]);
        if (w && (int)(k % w) == w - 1) A.rules.insert(A.rules.end(), width - w, -1);
      }
      for (int c : C.choices) A.choices.push_back(c >= 0 ? c + (int)(inBase[t] * C.nFeatures) : c);
      A.features.insert(A.features.end(), C.features.begin(), C.features.end());
      rowsOut += C.nSpatialSites;
      C = Iface();
    }
    A.nSpatialSites = (int)rowsOut;
  }
  return all;
}

} // namespace orc

using namespace orc;

// =================================================================== C interface (ctypes)
extern "C" {

int orc_ipow(int b, int e) { return ipow(b, e); }
int orc_triangleSize(int s, int d) { return triangleSize(s, d); }
int orc_intRound(int a, int d) { return intRound(a, d); }

struct OrcRules {
  std::vector<int> rules; std::vector<int64_t> outKeys; std::vector<int> outRows, outOff, outBg; int nOutSites = 0;
};

// kind: 0 square, 1 triangular, 2 terminal pooling (size/stride/minActive ignored).
// Same flat protocol as ref_grid_rules in ref_wrap.cpp.
void *orc_grid_rules(int kind, int dim, int nIn, int nOut, int size, int stride, int minActive, int batch,
                     const int64_t *inKeys, const int *inRows, const int *inOff, const int *inBg) {
  OrcRules *res = new OrcRules();
  res->outOff.push_back(0);
  std::vector<Grid> in(batch);
  size_t S = 1;
  for (int b = 0; b < batch; ++b) {
    in[b].bg = inBg[b];
    for (int i = inOff[b]; i < inOff[b + 1]; ++i) in[b].sites.emplace_back(inKeys[i], inRows[i]);
    std::sort(in[b].sites.begin(), in[b].sites.end());
    S = std::max(S, in[b].sites.size());
  }
  for (int b = 0; b < batch; ++b) {
    Grid out;
    if (kind == 2) terminalRules(in[b], out, (int)S, res->nOutSites, res->rules);
    else { Regions R(kind, dim, nIn, nOut, size, stride); gridRules(in[b], out, R, res->nOutSites, res->rules, minActive); }
    for (auto &s : out.sites) { res->outKeys.push_back(s.first); res->outRows.push_back(s.second); }
    res->outOff.push_back((int)res->outKeys.size());
    res->outBg.push_back(out.bg);
  }
  return res;
}
// Tick tables of `count` consecutive FractionalPoolingRegions<ticks> objects drawn from one RNG
// seeded with `seed` (one per sample, one ticks object per axis, in that order):
// out[(b*dim + axis) * (2*nOut + 2*nIn)] = inputL[nOut], inputR[nOut], outputL[nIn], outputR[nIn].
void orc_fmp_ticks(int kind, int dim, int nIn, int nOut, int poolSize, unsigned seed, int count, int *out) {
  FmpRng rng;
  rng.gen.seed(seed);
  const int stride = 2 * nOut + 2 * nIn;
  for (int b = 0; b < count; ++b)
    for (int a = 0; a < dim; ++a) {
      Ticks t = makeTicks(kind, nIn, nOut, poolSize, rng);
      int *o = out + ((size_t)b * dim + a) * stride;
      std::copy(t.inputL.begin(), t.inputL.end(), o);
      std::copy(t.inputR.begin(), t.inputR.end(), o + nOut);
      std::copy(t.outputL.begin(), t.outputL.end(), o + 2 * nOut);
      std::copy(t.outputR.begin(), t.outputR.end(), o + 2 * nOut + nIn);
    }
}
// Rules of one FMP layer from given tick tables (same flat protocol as orc_grid_rules).
void *orc_fmp_rules(int dim, int nIn, int nOut, int poolSize, int overlapping, int batch, const int *ticks,
                    const int64_t *inKeys, const int *inRows, const int *inOff, const int *inBg) {
  OrcRules *res = new OrcRules();
  res->outOff.push_back(0);
  const int stride = 2 * nOut + 2 * nIn;
  for (int b = 0; b < batch; ++b) {
    Grid in, out;
    in.bg = inBg[b];
    for (int i = inOff[b]; i < inOff[b + 1]; ++i) in.sites.emplace_back(inKeys[i], inRows[i]);
    std::sort(in.sites.begin(), in.sites.end());
    Ticks pb[4];
    for (int a = 0; a < dim; ++a) {
      const int *o = ticks + ((size_t)b * dim + a) * stride;
      pb[a].inputL.assign(o, o + nOut); pb[a].inputR.assign(o + nOut, o + 2 * nOut);
      pb[a].outputL.assign(o + 2 * nOut, o + 2 * nOut + nIn); pb[a].outputR.assign(o + 2 * nOut + nIn, o + stride);
    }
    gridRulesFmp(in, out, pb, dim, nIn, nOut, poolSize, overlapping != 0, res->nOutSites, res->rules);
    for (auto &s : out.sites) { res->outKeys.push_back(s.first); res->outRows.push_back(s.second); }
    res->outOff.push_back((int)res->outKeys.size());
    res->outBg.push_back(out.bg);
  }
  return res;
}
long long orc_result_n_rules(void *h) { return (long long)((OrcRules *)h)->rules.size(); }
long long orc_result_n_out(void *h) { return (long long)((OrcRules *)h)->outKeys.size(); }
int orc_result_n_sites(void *h) { return ((OrcRules *)h)->nOutSites; }
void orc_result_fetch(void *h, int *rules, int64_t *outKeys, int *outRows, int *outOff, int *outBg) {
  OrcRules *r = (OrcRules *)h;
  if (!r->rules.empty()) std::memcpy(rules, r->rules.data(), r->rules.size() * sizeof(int));
  if (!r->outKeys.empty()) {
    std::memcpy(outKeys, r->outKeys.data(), r->outKeys.size() * sizeof(int64_t));
    std::memcpy(outRows, r->outRows.data(), r->outRows.size() * sizeof(int));
  }
  std::memcpy(outOff, r->outOff.data(), r->outOff.size() * sizeof(int));
  if (!r->outBg.empty()) std::memcpy(outBg, r->outBg.data(), r->outBg.size() * sizeof(int));
}
void orc_result_free(void *h) { delete (OrcRules *)h; }

void orc_gather(const float *feat, const int *rules, long long count, int nIn, float *out) { gather(feat, rules, count, nIn, out); }
void orc_nin_forward(const float *X, long long rows, int K, const float *W, const float *B, const float *prelu,
                     int N, float p, int act, int accum64, float *out) {
  if (accum64) ninForward<double>(X, rows, K, W, B, prelu, N, p, act, out);
  else ninForward<float>(X, rows, K, W, B, prelu, N, p, act, out);
}
void orc_maxpool(const float *in, const int *rules, long long rowsOut, int sd, int C, float *out, int *choice) { maxPool(in, rules, rowsOut, sd, C, out, choice); }
void orc_terminal_pool(const float *in, const int *rules, int count, int S, int C, float *out) { terminalPool(in, rules, count, S, C, out); }
void orc_top_indices(const float *v, int n, int k, int *out) { topIndices(v, n, k, out); }

// ---- networks
void *orc_net_create(int dim, int nInputFeatures, int nClasses, int nTop) {
  Net *n = new Net(); n->dim = dim; n->nInputFeatures = nInputFeatures; n->nClasses = nClasses; n->nTop = nTop; n->nOutputFeatures = nInputFeatures; return n;
}
void orc_net_free(void *h) { delete (Net *)h; }
void orc_net_addLeNetLayerMP(void *h, int nFeatures, int fs, int fstride, int ps, int pstride, int act, float dropout, int minActive) { ((Net *)h)->addLeNetLayerMP(nFeatures, fs, fstride, ps, pstride, act, dropout, minActive); }
void orc_net_addTriangularLeNetLayerMP(void *h, int nFeatures, int fs, int fstride, int ps, int pstride, int act, float dropout, int minActive) { ((Net *)h)->addTriangularLeNetLayerMP(nFeatures, fs, fstride, ps, pstride, act, dropout, minActive); }
void orc_net_addLeNetLayerFMP(void *h, int kind, int nFeatures, int fs, int fstride, int ps, float shrink, int act, float dropout, int minActive) { ((Net *)h)->addLeNetLayerFMP(kind, nFeatures, fs, fstride, ps, shrink, act, dropout, minActive); }
void orc_net_set_fmp_seed(void *h, unsigned seed) { ((Net *)h)->fmpSeed = seed; }
// The output features learnt layer `layer` keeps in the training steps that follow (n ascending indices; n = 0: all).
int orc_net_set_dropout_features(void *h, int layer, const int *present, int n) {
  Net *net = (Net *)h;
  if (layer < 0 || layer >= (int)net->layers.size() || net->layers[layer].type != L_NIN || n < 0 || n > net->layers[layer].nOut) return 1;
  net->layers[layer].present.assign(present, present + n);
  return 0;
}
void orc_net_addTerminalPoolingLayer(void *h, int poolSize, int S) { ((Net *)h)->addTerminalPoolingLayer(poolSize, S); }
void orc_net_addSoftmaxLayer(void *h) { ((Net *)h)->addSoftmaxLayer(); }
// NetworkArchitectures.cpp:3-11.
void *orc_net_DeepCNet(int dim, int l, int k, int fn, int nInputFeatures, int nClasses, float p, int nTop) {
  Net *n = (Net *)orc_net_create(dim, nInputFeatures, nClasses, nTop);
  for (int i = 0; i <= l; i++) n->addLeNetLayerMP((i + 1) * k, (i == 0) ? 3 : 2, 1, (i < l) ? 3 : 1, (i < l) ? 2 : 1, fn, p * i * 1.0f / l, 1);
  n->addSoftmaxLayer();
  return n;
}
int orc_net_n_layers(void *h) { return (int)((Net *)h)->layers.size(); }
int orc_net_input_spatial_size(void *h) { return ((Net *)h)->inputSpatialSize; }
// info[0..9] = type,size,stride,minActive,nIn,nOut,fs,act,inSpatial,outSpatial; *dropout
void orc_net_layer_info(void *h, int i, int *info, float *dropout) {
  const Layer &L = ((Net *)h)->layers[i];
  int v[10] = {L.type, L.size, L.stride, L.minActive, L.nIn, L.nOut, L.fs, L.act, L.inSpatial, L.outSpatial};
  std::memcpy(info, v, sizeof(v)); *dropout = L.dropout;
}
void orc_net_set_weights(void *h, int i, const float *W, const float *B, const float *prelu) {
  Layer &L = ((Net *)h)->layers[i];
  std::memcpy(L.W.data(), W, L.W.size() * sizeof(float));
  std::memcpy(L.B.data(), B, L.B.size() * sizeof(float));
  if (prelu && !L.prelu.empty()) std::memcpy(L.prelu.data(), prelu, L.prelu.size() * sizeof(float));
}
// The .cnn layout (SparseConvNetCUDA.cu:406-424; NetworkInNetworkLayer.cu:290-307;
// NetworkInNetworkPReLULayer.cu:280-304) without momentum: per learnt layer W, B[, PReLU].
int orc_net_load_weights(void *h, const char *path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) return -1;
  for (Layer &L : ((Net *)h)->layers) {
    if (L.type != L_NIN) continue;
    f.read((char *)L.W.data(), sizeof(float) * L.W.size());
    f.read((char *)L.B.data(), sizeof(float) * L.B.size());
    if (!L.prelu.empty()) f.read((char *)L.prelu.data(), sizeof(float) * L.prelu.size());
  }
  return f ? 0 : -2;
}

// Fractional max-pooling: every sample's tick tables, drawn in batch order from each layer's generator, which is seeded
// anew (seed + layer index) for every batch.
static std::vector<std::vector<Ticks>> drawFmpTicks(const Net &net, int batch) {
  std::vector<std::vector<Ticks>> fmpTicks(net.layers.size());
  for (size_t l = 0; l < net.layers.size(); ++l) {
    const Layer &L = net.layers[l];
    if (L.type != L_FMP) continue;
    FmpRng rng;
    rng.gen.seed(net.fmpSeed + (unsigned)l);
    for (int b = 0; b < batch; ++b)
      for (int a = 0; a < net.dim; ++a) fmpTicks[l].push_back(makeTicks(L.fmpKind, L.inSpatial, L.outSpatial, L.size, rng));
  }
  return fmpTicks;
}

// Full forward.  probs [batch x nClasses], predictions [batch x nTop] (SoftmaxClassifier.cu:36-41).
// nThreads > 1 splits the batch into contiguous chunks (samples are independent); keep=1
// retains every interface for layer-by-layer comparison (chunks are joined into the whole
// batch's numbering: row ids, rule cells and pooling choices shifted by the rows in front).
// times[0] = rule construction seconds (summed over chunks / nThreads), times[1] = wall seconds.
void orc_net_forward(void *h, int batch, const int64_t *keys, const int *off, const float *features,
                     int nThreads, int accum64, int keep, float *probs, int *predictions, double *times) {
  Net *net = (Net *)h;
  auto t0 = std::chrono::steady_clock::now();
  if (nThreads < 1) nThreads = 1;
  nThreads = std::min(nThreads, std::max(1, batch));
  std::vector<double> tr(nThreads, 0.0);
  std::vector<std::vector<Iface>> ifs(nThreads);
  std::vector<std::vector<Ticks>> fmpTicks = drawFmpTicks(*net, batch);
  auto work = [&](int t) {
    int b0 = (int)((long long)batch * t / nThreads), b1 = (int)((long long)batch * (t + 1) / nThreads);
    if (b1 <= b0) return;
    forwardChunk(*net, b1 - b0, keys, off + b0, features, accum64 != 0, ifs[t], &tr[t], fmpTicks, b0);
    const Iface &top = ifs[t].back();
    for (int b = b0; b < b1; ++b) {
      const float *pr = top.features.data() + (size_t)(b - b0) * net->nClasses;
      std::memcpy(probs + (size_t)b * net->nClasses, pr, sizeof(float) * net->nClasses);
      if (predictions) topIndices(pr, net->nClasses, net->nTop, predictions + (size_t)b * net->nTop);
    }
  };
  if (nThreads == 1) work(0);
  else { std::vector<std::thread> th; for (int t = 0; t < nThreads; ++t) th.emplace_back(work, t); for (auto &x : th) x.join(); }
  if (keep && nThreads == 1) net->kept = std::move(ifs[0]);
  else if (keep) net->kept = joinChunks(*net, ifs);
  else net->kept.clear();
  if (times) {
    double s = 0; for (double v : tr) s += v;
    times[0] = s / nThreads;
    times[1] = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  }
}
// One training step on one batch (TRAINBATCH without dropout): forward (fp32 or fp64 accumulation), SoftmaxClassifier,
// then every layer's backwards() in reverse order with the SGD update of its weights.  Keeps every interface
// (features and dfeatures) for orc_net_iface_fetch / orc_net_iface_dfeatures.  stats = {negativeLogLikelihood, mistakes}.
// backpropErrors is false for the input and true from the first learnt layer's output on (NetworkInNetworkLayer.cu:155).
int orc_net_train_step(void *h, int batch, const int64_t *keys, const int *off, const float *features, const int *labels,
                       float learningRate, float momentum, int accum64, float *probs, double *stats) {
  Net *net = (Net *)h;
  // (a layer built with dropout must have been told its subset: the random draw itself is not restated)
  for (const Layer &L : net->layers) if (L.type == L_NIN && L.dropout > 0 && L.present.empty()) return 1;
  std::vector<std::vector<Ticks>> fmpTicks = drawFmpTicks(*net, batch);
  std::vector<Iface> ifs;
  forwardChunk(*net, batch, keys, off, features, accum64 != 0, ifs, nullptr, fmpTicks, 0, true);
  const int nL = (int)net->layers.size();
  Iface &top = ifs.back();
  const int C = net->nClasses;
  std::memcpy(probs, top.features.data(), sizeof(float) * (size_t)batch * C);
  double nll = 0; int mistakes = batch;
  for (int b = 0; b < batch; ++b) { // SoftmaxClassifier.cu:43-53
    nll -= std::log(std::max(probs[(size_t)b * C + labels[b]], 1.0e-15f));
    int best; topIndices(probs + (size_t)b * C, C, 1, &best);
    if (best == labels[b]) --mistakes;
  }
  if (stats) { stats[0] = nll; stats[1] = mistakes; }
  top.dfeatures.resize(top.features.size());
  softmaxNllBackward(top.features.data(), labels, batch, C, top.dfeatures.data());
  std::vector<char> backprop(nL + 1, 0);
  for (int l = 0; l < nL; ++l) backprop[l + 1] = net->layers[l].type == L_NIN ? 1 : backprop[l];
  for (int l = nL - 1; l >= 0; --l) {
    Layer &L = net->layers[l];
    Iface &in = ifs[l], &out = ifs[l + 1];
    const long long rowsOut = out.nSpatialSites, rowsIn = in.nSpatialSites;
    if (L.type == L_NIN) {
      // dropout: gradients of dropped features are zero on both sides, and the update leaves every weight that touches
      // one (and its momentum) as it is (dGradientDescentShrunkMatrix / ...Vector, NetworkInNetworkLayer.cu:43-81)
      const std::vector<char> outMask = keptMask(L);
      std::vector<char> inMask;
      for (int k = l - 1; k >= 0; --k)
        if (net->layers[k].type == L_NIN) { inMask = keptMask(net->layers[k]); break; }
      if (!outMask.empty())
        for (long long r = 0; r < rowsOut; ++r)
          for (int n = 0; n < L.nOut; ++n)
            if (!outMask[n]) out.dfeatures[(size_t)r * L.nOut + n] = 0.f;
      std::vector<float> dprelu(L.nOut, 0.f);
      if (accum64) activationBackward<double>(out.features.data(), out.dfeatures.data(), rowsOut, L.nOut, L.act, L.prelu.empty() ? nullptr : L.prelu.data(), dprelu.data());
      else activationBackward<float>(out.features.data(), out.dfeatures.data(), rowsOut, L.nOut, L.act, L.prelu.empty() ? nullptr : L.prelu.data(), dprelu.data());
      std::vector<float> dW((size_t)L.nIn * L.nOut), dB(L.nOut);
      if (backprop[l]) in.dfeatures.assign((size_t)rowsIn * L.nIn, 0.f);
      float *dX = backprop[l] ? in.dfeatures.data() : nullptr;
      if (accum64) ninBackward<double>(in.features.data(), out.dfeatures.data(), rowsOut, L.nIn, L.nOut, L.W.data(), dW.data(), dB.data(), dX);
      else ninBackward<float>(in.features.data(), out.dfeatures.data(), rowsOut, L.nIn, L.nOut, L.W.data(), dW.data(), dB.data(), dX);
      if (dX && !inMask.empty()) { // (the convolution in front repeats the features: the mask applies with its own period)
        const size_t period = inMask.size();
        for (size_t i = 0; i < (size_t)rowsIn * L.nIn; ++i)
          if (!inMask[i % period]) dX[i] = 0.f;
      }
      if (L.MW.empty()) { L.MW.assign(L.W.size(), 0.f); L.MB.assign(L.B.size(), 0.f); L.Mprelu.assign(L.prelu.size(), 0.f); }
      const std::vector<float> W0 = L.W, MW0 = L.MW, B0 = L.B, MB0 = L.MB, P0 = L.prelu, MP0 = L.Mprelu;
      sgdUpdate(L.W.data(), L.MW.data(), dW.data(), L.W.size(), learningRate, momentum);
      sgdUpdate(L.B.data(), L.MB.data(), dB.data(), L.B.size(), learningRate, momentum);
      if (L.act == PRELU) sgdUpdate(L.prelu.data(), L.Mprelu.data(), dprelu.data(), L.prelu.size(), learningRate, momentum, true);
      if (!outMask.empty() || !inMask.empty()) {
        for (int k = 0; k < L.nIn; ++k)
          for (int n = 0; n < L.nOut; ++n)
            if ((!inMask.empty() && !inMask[k % inMask.size()]) || (!outMask.empty() && !outMask[n])) {
              L.W[(size_t)k * L.nOut + n] = W0[(size_t)k * L.nOut + n];
              L.MW[(size_t)k * L.nOut + n] = MW0[(size_t)k * L.nOut + n];
            }
        for (int n = 0; n < L.nOut && !outMask.empty(); ++n)
          if (!outMask[n]) {
            L.B[n] = B0[n]; L.MB[n] = MB0[n];
            if (L.act == PRELU) { L.prelu[n] = P0[n]; L.Mprelu[n] = MP0[n]; } // (what NetworkInNetworkPReLULayer.cu:199-207 means to do)
          }
      }
    } else if (!backprop[l]) {
      continue;
    } else if (L.type == L_CONV || L.type == L_CONV_TRI) {
      in.dfeatures.resize((size_t)rowsIn * L.nIn);
      if (accum64) gatherBackward<double>(out.dfeatures.data(), out.rules.data(), rowsOut * L.fs, L.nIn, rowsIn, in.dfeatures.data());
      else gatherBackward<float>(out.dfeatures.data(), out.rules.data(), rowsOut * L.fs, L.nIn, rowsIn, in.dfeatures.data());
    } else if (L.type == L_MAXPOOL || L.type == L_MAXPOOL_TRI || L.type == L_FMP) {
      in.dfeatures.resize(in.features.size());
      if (accum64) maxPoolBackward<double>(out.dfeatures.data(), out.choices.data(), (long long)out.dfeatures.size(), (long long)in.features.size(), in.dfeatures.data());
      else maxPoolBackward<float>(out.dfeatures.data(), out.choices.data(), (long long)out.dfeatures.size(), (long long)in.features.size(), in.dfeatures.data());
    } else if (L.type == L_TERMINAL) {
      in.dfeatures.resize(in.features.size());
      terminalPoolBackward(out.dfeatures.data(), out.rules.data(), (int)rowsOut, (int)(out.rules.size() / batch), L.nOut, rowsIn, in.dfeatures.data());
    }
  }
  net->kept = std::move(ifs);
  return 0;
}
// dfeatures of kept interface i after orc_net_train_step: returns their count, copies them if d is not null.
long long orc_net_iface_dfeatures(void *h, int i, float *d) {
  const Iface &I = ((Net *)h)->kept[i];
  if (d && !I.dfeatures.empty()) std::memcpy(d, I.dfeatures.data(), I.dfeatures.size() * sizeof(float));
  return (long long)I.dfeatures.size();
}
void orc_net_get_weights(void *h, int i, float *W, float *B, float *prelu) {
  const Layer &L = ((Net *)h)->layers[i];
  std::memcpy(W, L.W.data(), L.W.size() * sizeof(float));
  std::memcpy(B, L.B.data(), L.B.size() * sizeof(float));
  if (prelu && !L.prelu.empty()) std::memcpy(prelu, L.prelu.data(), L.prelu.size() * sizeof(float));
}
// Single backward operations, for layer-level tests.
void orc_activation_backward(const float *b, float *d, long long rows, int N, int act, const float *prelu, float *dprelu) { activationBackward<double>(b, d, rows, N, act, prelu, dprelu); }
void orc_nin_backward(const float *X, const float *d, long long rows, int K, int N, const float *W, float *dW, float *dB, float *dX) { ninBackward<double>(X, d, rows, K, N, W, dW, dB, dX); }
void orc_gather_backward(const float *dConv, const int *rules, long long count, int nIn, long long rowsIn, float *dIn) { gatherBackward<double>(dConv, rules, count, nIn, rowsIn, dIn); }
void orc_maxpool_backward(const float *dOut, const int *choice, long long n, long long nIn, float *dIn) { maxPoolBackward<double>(dOut, choice, n, nIn, dIn); }
void orc_terminal_pool_backward(const float *dOut, const int *rules, int count, int S, int C, long long rowsIn, float *dIn) { terminalPoolBackward(dOut, rules, count, S, C, rowsIn, dIn); }
void orc_sgd_update(float *w, float *m, const float *d, long long n, float lr, float momentum, int keepPositive) { sgdUpdate(w, m, d, (size_t)n, lr, momentum, keepPositive != 0); }
// Kept interface i (0 = input): sizes[0..4] = nSpatialSites, nFeatures, spatialSize, rules.size(), choices.size()
void orc_net_iface_sizes(void *h, int i, long long *sizes) {
  const Iface &I = ((Net *)h)->kept[i];
  sizes[0] = I.nSpatialSites; sizes[1] = I.nFeatures; sizes[2] = I.spatialSize; sizes[3] = (long long)I.rules.size(); sizes[4] = (long long)I.choices.size();
}
// keys[row] = site key of each row (-1 for background rows), gridOff[batch+1] = first row per sample.
void orc_net_iface_fetch(void *h, int i, float *features, int *rules, int *choices, int64_t *rowKeys) {
  const Iface &I = ((Net *)h)->kept[i];
  if (features && !I.features.empty()) std::memcpy(features, I.features.data(), I.features.size() * sizeof(float));
  if (rules && !I.rules.empty()) std::memcpy(rules, I.rules.data(), I.rules.size() * sizeof(int));
  if (choices && !I.choices.empty()) std::memcpy(choices, I.choices.data(), I.choices.size() * sizeof(int));
  if (rowKeys) {
    for (int r = 0; r < I.nSpatialSites; ++r) rowKeys[r] = -2;
    for (const Grid &g : I.grids) {
      for (auto &s : g.sites) rowKeys[s.second] = s.first;
      if (g.bg >= 0) rowKeys[g.bg] = -1;
    }
  }
}
}
