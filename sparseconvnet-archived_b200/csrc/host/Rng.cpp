#include "Rng.h"
#include <algorithm>

namespace {
std::mutex seedMutex;
std::mt19937 seedGenerator; // default seed: the n-th RNG of a process always starts the same way
} // namespace

RNG::RNG() : stdNormal(0, 1), uniform01(0, 1) {
  std::lock_guard<std::mutex> lock(seedMutex);
  gen.seed(seedGenerator());
}
int RNG::randint(int n) { return n == 0 ? 0 : (int)(gen() % n); } // Rng.cpp:22-27
float RNG::uniform(float a, float b) { return a + (b - a) * uniform01(gen); }
float RNG::normal(float mean, float sd) { return mean + sd * stdNormal(gen); }
int RNG::bernoulli(float p) { return uniform01(gen) < p ? 1 : 0; }
std::vector<int> RNG::NchooseM(int n, int m) { // Rng.cpp:41-48
  std::vector<int> ret(m, 100);
  int ctr = m;
  for (int i = 0; i < n; i++)
    if (uniform01(gen) < ctr * 1.0 / (n - i)) ret[m - ctr--] = i;
  return ret;
}
std::vector<int> RNG::permutation(int n) {
  std::vector<int> ret(n);
  for (int i = 0; i < n; i++) ret[i] = i;
  std::shuffle(ret.begin(), ret.end(), gen);
  return ret;
}
