#include "BatchProducer.h"
#include <algorithm>

void SitesPicture::codifyInputData(SparseGrid &grid, std::vector<float> &out, int &nSpatialSites, int) {
  if (backgroundRow) {
    out.insert(out.end(), nFeatures, 0.0f);
    grid.backgroundCol = nSpatialSites++;
  }
  for (size_t i = 0; i < keys.size(); ++i) {
    if (grid.mp.emplace(keys[i], nSpatialSites).second) {
      out.insert(out.end(), features.begin() + i * nFeatures, features.begin() + (i + 1) * nFeatures);
      ++nSpatialSites;
    }
  }
}
BatchProducer::BatchProducer(SparseConvNetCUDA &cnn, SpatiallySparseDataset &dataset, int spatialSize, int batchSize)
    : cnn(cnn), dataset(dataset), spatialSize(spatialSize), batchSize(batchSize), nextToServe(0), lastServedSlot(-1), stop(false) {
  if (batchSize < 1) throw ScnException("BatchProducer: batchSize must be positive");
  nBatches = ((int)dataset.pictures.size() + batchSize - 1) / batchSize;
  permutation = range((int)dataset.pictures.size());
  if (dataset.type == TRAINBATCH) { // BatchProducer.cu:23-27
    RNG rng;
    rng.vectorShuffle(permutation);
  }
  slotState.assign(cnn.nBatchProducerThreads, -1);
  for (auto &b : cnn.batchPool) cnn.prepareBatch(b);
  for (int t = 0; t < cnn.nBatchProducerThreads; ++t) workers.emplace_back(&BatchProducer::worker, this, t);
}
BatchProducer::~BatchProducer() {
  { std::lock_guard<std::mutex> lk(mu); stop = true; }
  cv.notify_all();
  for (auto &w : workers) w.join();
}

// Host part of BatchProducer.cu:40-71: codify the pictures of batch c into pool slot cc.
void BatchProducer::preprocessBatch(int c, int cc) {
  SpatiallySparseBatch &b = cnn.batchPool[cc];
  b.reset();
  b.type = dataset.type;
  SpatiallySparseBatchInterface &in = b.interfaces[0];
  in.nFeatures = dataset.nFeatures;
  in.spatialSize = spatialSize;
  in.featuresPresent.hVector() = range(dataset.nFeatures);
  in.sub->features.copyToCPU();
  std::vector<float> &feat = in.sub->features.hVector();
  feat.clear();
  b.labels.copyToCPU();
  const int lo = c * batchSize, hi = std::min((c + 1) * batchSize, (int)dataset.pictures.size());
  for (int i = lo; i < hi; ++i) {
    Picture *pic = dataset.pictures[permutation[i]]->distort(0, dataset.type);
    b.sampleNumbers.push_back(permutation[i]);
    b.batchSize++;
    in.grids.push_back(SparseGrid());
    b.labels.hVector().push_back(pic->label);
    pic->codifyInputData(in.grids.back(), feat, in.nSpatialSites, spatialSize);
    if (pic != dataset.pictures[permutation[i]]) delete pic;
  }
  if ((int)feat.size() != in.nFeatures * in.nSpatialSites) throw ScnException("codifyInputData wrote a wrong number of features");
  if (!cnn.inputNormalizingConstants.empty())
    for (size_t i = 0; i < feat.size(); ++i) feat[i] *= cnn.inputNormalizingConstants[i % in.nFeatures];
}

// Worker t owns pool slot t and fills it with batches t, t+T, t+2T, ...
void BatchProducer::worker(int t) {
  const int T = cnn.nBatchProducerThreads;
  for (int c = t; c < nBatches; c += T) {
    {
      std::unique_lock<std::mutex> lk(mu);
      cv.wait(lk, [&] { return stop || slotState[t] == -1; });
      if (stop) return;
    }
    preprocessBatch(c, t);
    { std::lock_guard<std::mutex> lk(mu); slotState[t] = c; }
    cv.notify_all();
  }
}

// Consumer side of BatchProducer.cu:108-142: wait for the next batch, upload it, run the
// rule chain on the device.
SpatiallySparseBatch *BatchProducer::nextBatch() {
  const int T = cnn.nBatchProducerThreads;
  {
    std::lock_guard<std::mutex> lk(mu);
    if (lastServedSlot >= 0) { slotState[lastServedSlot] = -1; lastServedSlot = -1; }
  }
  cv.notify_all();
  if (nextToServe >= nBatches) return nullptr;
  const int slot = nextToServe % T;
  {
    std::unique_lock<std::mutex> lk(mu);
    cv.wait(lk, [&] { return slotState[slot] == nextToServe; });
  }
  SpatiallySparseBatch &b = cnn.batchPool[slot];
  b.interfaces[0].uploadGrids(cnn.memStream);
  b.interfaces[0].sub->features.copyToGPUAsync(cnn.memStream);
  cnn.preprocessBatchOnDevice(b);
  lastServedSlot = slot;
  ++nextToServe;
  return &b;
}
