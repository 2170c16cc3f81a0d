// vectorCUDA<T>: a vector that lives either in a std::vector or in device memory and
// migrates when the other side is asked for (vectorCUDA.h:7-37).  dPtr() uploads,
// hVector() downloads, resize() on the device never shrinks the allocation and does not
// keep contents (vectorCUDA.cu:209-225).  Unlike the reference, migrations are silent.
#pragma once
#include <vector>
#include "utilities.h"

template <typename t> class vectorCUDA {
private:
  t *d_vec;
  unsigned int dsize; // size while on the device
  size_t dAllocated;  // elements allocated on the device (>= dsize)
  std::vector<t> vec;
  t *ownVec;          // while borrowing: this vector's own allocation, kept for later
  size_t ownAllocated;
  bool borrowed;
  void giveBack();

public:
  vectorCUDA(bool onGPU = true, unsigned int dsize = 0);
  ~vectorCUDA();
  vectorCUDA(const vectorCUDA &) = delete;
  vectorCUDA &operator=(const vectorCUDA &) = delete;
  vectorCUDA(vectorCUDA &&o) noexcept;
  bool onGPU;
  void copyToCPU();
  void copyToGPU();
  void copyToCPUAsync(cudaMemStream &memStream); // staged through pinned memory, then waits
  void copyToGPUAsync(cudaMemStream &memStream);
  t *&dPtr();
  std::vector<t> &hVector();
  unsigned int size();
  float meanAbs();
  void multiplicativeRescale(float multiplier);
  void setZero();
  void setZero(cudaMemStream &memStream);
  void setConstant(float a = 0);
  void setUniform(float a = 0, float b = 1);
  void setBernoulli(float p = 0.5);
  void setNormal(float mean = 0, float sd = 1);
  void resize(int n);
  void reserveDevice(size_t n); // grow the device allocation without changing size()
  // Stand for n elements of device memory that the caller owns (no copy; not in the reference).  The vector
  // reads them until its next resize(), host access or borrowDevice(); it never writes or frees them.
  void borrowDevice(t *p, unsigned int n);
  void dropBorrowed() { giveBack(); } // forget the caller's memory (size becomes 0); no-op otherwise
  void printSubset(const char *name, int nCol, int maxPrint = 10);
  void check(const char *file = 0, int linenumber = 0);
  void summary(const char *file = 0, int linenumber = 0);
};
