// The one exchange step of the path when a batch is sharded by sample over the GPUs of a node: every rank's block of
// class probabilities (what SoftmaxClassifier.cu:36-41 brings to the host) goes to every other rank.  The reference runs
// on a single device (SparseConvNetCUDA.cu:43-71) and has no counterpart.  A rank stores its block into a buffer of
// every peer and collects the peers' blocks of the step before with a kernel whose wait is bounded; both run on the
// network's stream in front of the copy that returns the step's results, so a step has no host-side collective.
#pragma once
#include <vector>
#include "utilities.h"

class ResultExchange {
public:
  static const int maxRanks = 16;
  const int world, rank, capRows, nClasses, capFloats;
  unsigned published = 0; // steps this rank has published (the steps count 1, 2, 3, ... on every rank alike)
  unsigned collected = 0; // last step collected
  ResultExchange(int world, int rank, int capRows, int nClasses);
  ~ResultExchange();
  ResultExchange(const ResultExchange &) = delete;
  ResultExchange &operator=(const ResultExchange &) = delete;
  void *localBuffer() { return local; }
  const unsigned char *handle() const { return ipcHandle; } // 64 bytes another process of this node passes to connect()
  void connect(const unsigned char *handles);               // world x 64 bytes, in rank order (the own entry is not opened)
  void connectLocal(void *const *buffers);                  // the peers' buffers as device pointers of this process
  bool connected() const { return isConnected; }
  // Enqueue ONE kernel that collects the last published step, if it has not been collected yet, and publishes dProbs
  // [rows x nClasses] as the next step (dProbs NULL: collect only).  The collected blocks go to dGathered
  // [world x capFloats] and dRowsStatus [world + 1] (row counts, then the status word), or, where those are NULL, to
  // this object's own device block (deviceGathered / deviceRows).
  void step(const float *dProbs, int rows, cudaStream_t stream, float *dGathered = nullptr, int *dRowsStatus = nullptr);
  // Device block of the last collect: gathered[world x capFloats] floats, then rows[world] and the status word as ints.
  float *deviceGathered() { return dOut; }
  int *deviceRows() { return (int *)(dOut + (size_t)world * capFloats); }
  size_t blockBytes() const { return sizeof(float) * (size_t)world * capFloats + sizeof(int) * (world + 1); }
  // Enqueue the copy of that block into page-locked host memory; after the stream has been waited for, deliver() hands
  // it out (gathered may be NULL) and throws if a rank's block did not arrive within the time limit.
  void copyBlockToHost(cudaStream_t stream);
  void deliver(float *gathered, int *rows);
  // The same step on a stream of this object's own, ordered behind what `main` holds now: the device-resident caller's
  // next forward does not queue behind the exchange kernel.  What the step collected is complete for work enqueued on
  // `main` after the NEXT call of stepBeside (or after this one, when dProbs is NULL: a collect-only call ends a run).
  void stepBeside(const float *dProbs, int rows, cudaStream_t main, float *dGathered, int *dRowsStatus);

private:
  void *local = nullptr;
  void *peers[maxRanks] = {};
  bool opened[maxRanks] = {};
  unsigned char ipcHandle[64] = {};
  bool isConnected = false;
  float *dOut = nullptr; // device block
  char *hOut = nullptr;  // page-locked copy
  cudaStream_t side = nullptr;
  cudaEvent_t mainReady = nullptr, sideDone = nullptr;
  bool sidePending = false;
};
