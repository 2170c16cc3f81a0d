#include "vectorCUDA.h"
#include <cmath>
#include <cstring>
#include <iostream>
#include <random>

namespace {
std::mt19937 &fillRng() { // deterministic fills (the reference seeds from the clock, Rng.cpp:11-15)
  static thread_local std::mt19937 g(20151117u);
  return g;
}
} // namespace

template <typename t> vectorCUDA<t>::vectorCUDA(bool onGPU, unsigned int dsize)
    : d_vec(nullptr), dsize(dsize), dAllocated(0), ownVec(nullptr), ownAllocated(0), borrowed(false), onGPU(onGPU) {
  if (onGPU && dsize > 0) { dAllocated = dsize; cudaSafeCall(cudaMalloc((void **)&d_vec, sizeof(t) * dAllocated)); }
  else if (!onGPU) vec.resize(dsize);
}
template <typename t> vectorCUDA<t>::~vectorCUDA() { giveBack(); if (dAllocated > 0) cudaFree(d_vec); }
template <typename t> void vectorCUDA<t>::giveBack() {
  if (!borrowed) return;
  d_vec = ownVec; dAllocated = ownAllocated; ownVec = nullptr; ownAllocated = 0; borrowed = false; dsize = 0;
}
template <typename t> void vectorCUDA<t>::borrowDevice(t *p, unsigned int n) {
  if (!onGPU) { vec.clear(); onGPU = true; }
  if (!borrowed) { ownVec = d_vec; ownAllocated = dAllocated; borrowed = true; }
  d_vec = p; dsize = n; dAllocated = 0; // (nothing here may be freed)
}
template <typename t> vectorCUDA<t>::vectorCUDA(vectorCUDA &&o) noexcept
    : d_vec(o.d_vec), dsize(o.dsize), dAllocated(o.dAllocated), vec(std::move(o.vec)), ownVec(o.ownVec), ownAllocated(o.ownAllocated),
      borrowed(o.borrowed), onGPU(o.onGPU) {
  o.d_vec = nullptr; o.dAllocated = 0; o.dsize = 0; o.ownVec = nullptr; o.ownAllocated = 0; o.borrowed = false;
}
template <typename t> void vectorCUDA<t>::reserveDevice(size_t n) {
  giveBack();
  if (n > dAllocated) {
    if (dAllocated > 0) cudaSafeCall(cudaFree(d_vec));
    d_vec = nullptr; dAllocated = 0;
    cudaSafeCall(cudaMalloc((void **)&d_vec, sizeof(t) * n));
    dAllocated = n;
  }
}
template <typename t> void vectorCUDA<t>::copyToCPU() {
  if (!onGPU) return;
  onGPU = false;
  vec.resize(dsize);
  if (dsize > 0) cudaSafeCall(cudaMemcpy(vec.data(), d_vec, sizeof(t) * dsize, cudaMemcpyDeviceToHost));
  giveBack(); // a later upload goes to this vector's own memory
}
template <typename t> void vectorCUDA<t>::copyToGPU() {
  if (onGPU) return;
  onGPU = true;
  dsize = (unsigned int)vec.size();
  reserveDevice(dsize);
  if (dsize > 0) {
    cudaSafeCall(cudaMemcpy(d_vec, vec.data(), sizeof(t) * dsize, cudaMemcpyHostToDevice));
    // a copy from pageable memory may return before its DMA has landed; kernels on other
    // (non-default) streams are not ordered behind it, so wait for it here
    cudaSafeCall(cudaStreamSynchronize(cudaStreamLegacy));
  }
  vec.clear();
}
template <typename t> void vectorCUDA<t>::copyToGPUAsync(cudaMemStream &ms) {
  if (onGPU) return;
  onGPU = true;
  dsize = (unsigned int)vec.size();
  reserveDevice(dsize);
  if (dsize > 0) {
    void *stage = ms.staging(sizeof(t) * dsize);
    std::memcpy(stage, vec.data(), sizeof(t) * dsize);
    cudaSafeCall(cudaMemcpyAsync(d_vec, stage, sizeof(t) * dsize, cudaMemcpyHostToDevice, ms.stream));
    cudaSafeCall(cudaStreamSynchronize(ms.stream)); // the staging buffer is reused by the next copy
  }
  vec.clear();
}
template <typename t> void vectorCUDA<t>::copyToCPUAsync(cudaMemStream &ms) {
  if (!onGPU) return;
  onGPU = false;
  vec.resize(dsize);
  if (dsize > 0) {
    void *stage = ms.staging(sizeof(t) * dsize);
    cudaSafeCall(cudaMemcpyAsync(stage, d_vec, sizeof(t) * dsize, cudaMemcpyDeviceToHost, ms.stream));
    cudaSafeCall(cudaStreamSynchronize(ms.stream));
    std::memcpy(vec.data(), stage, sizeof(t) * dsize);
  }
  giveBack();
}
template <typename t> t *&vectorCUDA<t>::dPtr() { copyToGPU(); return d_vec; }
template <typename t> std::vector<t> &vectorCUDA<t>::hVector() { copyToCPU(); return vec; }
template <typename t> unsigned int vectorCUDA<t>::size() { return onGPU ? dsize : (unsigned int)vec.size(); }
template <typename t> void vectorCUDA<t>::resize(int n) {
  if (onGPU) { reserveDevice(n); dsize = n; }
  else vec.resize(n);
}
template <typename t> float vectorCUDA<t>::meanAbs() {
  bool was = onGPU;
  std::vector<t> &v = hVector();
  double a = 0;
  for (auto x : v) a += std::fabs((double)x);
  float r = v.empty() ? 0.f : (float)(a / v.size());
  if (was) copyToGPU();
  return r;
}
template <typename t> void vectorCUDA<t>::multiplicativeRescale(float m) {
  bool was = onGPU;
  for (auto &x : hVector()) x = (t)(x * m);
  if (was) copyToGPU();
}
template <typename t> void vectorCUDA<t>::setZero() {
  if (onGPU) { if (dsize > 0) cudaSafeCall(cudaMemset(d_vec, 0, sizeof(t) * dsize)); }
  else std::fill(vec.begin(), vec.end(), (t)0);
}
template <typename t> void vectorCUDA<t>::setZero(cudaMemStream &ms) {
  if (onGPU) { if (dsize > 0) cudaSafeCall(cudaMemsetAsync(d_vec, 0, sizeof(t) * dsize, ms.stream)); }
  else std::fill(vec.begin(), vec.end(), (t)0);
}
template <typename t> void vectorCUDA<t>::setConstant(float a) { for (auto &x : hVector()) x = (t)a; }
template <typename t> void vectorCUDA<t>::setUniform(float a, float b) {
  std::uniform_real_distribution<double> u(0, 1);
  for (auto &x : hVector()) x = (t)(a + (b - a) * u(fillRng()));
}
template <typename t> void vectorCUDA<t>::setBernoulli(float p) {
  std::uniform_real_distribution<double> u(0, 1);
  for (auto &x : hVector()) x = (t)(u(fillRng()) < p ? 1 : 0);
}
template <typename t> void vectorCUDA<t>::setNormal(float mean, float sd) {
  std::normal_distribution<double> nd(0, 1);
  for (auto &x : hVector()) x = (t)(mean + sd * nd(fillRng()));
}
template <typename t> void vectorCUDA<t>::printSubset(const char *name, int nCol, int maxPrint) {
  bool was = onGPU;
  std::vector<t> &v = hVector();
  int nRow = nCol > 0 ? (int)v.size() / nCol : 0;
  std::cout << name << " " << nRow << " " << nCol << " ---------------------------------------\n";
  for (int r = 0; r < std::min(nRow, maxPrint); ++r) {
    for (int c = 0; c < std::min(nCol, maxPrint); ++c) std::cout << v[(size_t)r * nCol + c] << "\t";
    std::cout << "\n";
  }
  if (was) copyToGPU();
}
template <typename t> void vectorCUDA<t>::check(const char *file, int linenumber) {
  bool was = onGPU;
  for (auto x : hVector())
    if (std::isnan((double)x)) { std::cout << "NaN in vectorCUDA at " << (file ? file : "?") << ":" << linenumber << std::endl; break; }
  if (was) copyToGPU();
}
template <typename t> void vectorCUDA<t>::summary(const char *file, int linenumber) {
  std::cout << (file ? file : "") << ":" << linenumber << " onGPU " << onGPU << " size " << size() << " allocated " << dAllocated << std::endl;
}
template class vectorCUDA<float>;
template class vectorCUDA<int>;
