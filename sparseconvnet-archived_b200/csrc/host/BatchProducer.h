// Batch assembly (BatchProducer.h): worker threads turn pictures into host-side batches
// (grids + feature rows); nextBatch() hands the next one to the caller's thread, which
// uploads it and runs the rule chain on the device (SparseConvNetCUDA::preprocessBatchOnDevice).
// In the reference the workers also ran every layer's host preprocess (BatchProducer.cu:72-75);
// that work is now a few kernels on the consumer's stream.
#pragma once
#include <condition_variable>
#include <mutex>
#include <thread>
#include <vector>
#include "Rng.h"
#include "SparseConvNetCUDA.h"
#include "SpatiallySparseDataset.h"

class BatchProducer {
public:
  SparseConvNetCUDA &cnn;
  SpatiallySparseDataset &dataset;
  int spatialSize;
  int batchSize;
  int nBatches;
  std::vector<int> permutation; // picture order: shuffled for a TRAINBATCH dataset (BatchProducer.cu:23-27)
  BatchProducer(SparseConvNetCUDA &cnn, SpatiallySparseDataset &dataset, int spatialSize, int batchSize);
  ~BatchProducer();
  // Next batch, uploaded and preprocessed, or nullptr after the last one.
  SpatiallySparseBatch *nextBatch();
  void preprocessBatch(int c, int cc); // assemble batch c into pool slot cc (host part)

private:
  std::vector<std::thread> workers;
  std::mutex mu;
  std::condition_variable cv;
  std::vector<int> slotState; // per pool slot: batch number ready in it, or -1
  int nextToServe;
  int lastServedSlot;
  bool stop;
  void worker(int t);
};
