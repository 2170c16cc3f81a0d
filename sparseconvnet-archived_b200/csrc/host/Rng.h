// Random numbers with the reference's interface (Rng.h): a std::mt19937 behind a double-valued
// uniform distribution and std::shuffle.  The reference seeds every RNG from the clock; here
// each new RNG takes the next value of a process-wide, default-seeded generator, so runs
// repeat; `gen` is public (as in the reference) for callers that want their own seed.
#pragma once
#include <algorithm>
#include <mutex>
#include <random>
#include <vector>

class RNG {
  std::normal_distribution<> stdNormal;
  std::uniform_real_distribution<> uniform01;

public:
  std::mt19937 gen;
  RNG();
  int randint(int n);
  float uniform(float a = 0, float b = 1);
  float normal(float mean = 0, float sd = 1);
  int bernoulli(float p);
  template <typename T> int index(std::vector<T> &v) { return v.empty() ? 0 : (int)(gen() % v.size()); }
  std::vector<int> NchooseM(int n, int m);
  std::vector<int> permutation(int n);
  template <typename T> void vectorShuffle(std::vector<T> &v) { std::shuffle(v.begin(), v.end(), gen); }
};
