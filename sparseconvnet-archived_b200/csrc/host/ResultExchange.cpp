#include "ResultExchange.h"
#include <cstring>
#include <string>

ResultExchange::ResultExchange(int world_, int rank_, int capRows_, int nClasses_)
    : world(world_), rank(rank_), capRows(capRows_), nClasses(nClasses_), capFloats(capRows_ * nClasses_) {
  if (world < 1 || world > maxRanks || rank < 0 || rank >= world || capRows < 1 || nClasses < 1)
    throw ScnException("ResultExchange: 1..16 ranks, a rank among them, at least one row and one class");
  scnSafeCall(scn_exchange_alloc(scn_exchange_buffer_bytes(world, capFloats), &local, ipcHandle));
  cudaSafeCall(cudaMalloc((void **)&dOut, blockBytes()));
  cudaSafeCall(cudaMemset(dOut, 0, blockBytes()));
  cudaSafeCall(cudaMallocHost((void **)&hOut, blockBytes()));
  std::memset(hOut, 0, blockBytes());
}

ResultExchange::~ResultExchange() {
  cudaDeviceSynchronize(); // no kernel of this rank may still store into a peer's buffer
  for (int r = 0; r < world; ++r)
    if (opened[r]) scn_exchange_close(peers[r]);
  if (sideDone) cudaEventDestroy(sideDone);
  if (mainReady) cudaEventDestroy(mainReady);
  if (side) cudaStreamDestroy(side);
  if (hOut) cudaFreeHost(hOut);
  if (dOut) cudaFree(dOut);
  scn_exchange_free(local);
}

void ResultExchange::connect(const unsigned char *handles) {
  if (isConnected) throw ScnException("ResultExchange: already connected");
  for (int r = 0; r < world; ++r) {
    if (r == rank) { peers[r] = local; continue; }
    scnSafeCall(scn_exchange_open(handles + 64 * (size_t)r, &peers[r]));
    opened[r] = true;
  }
  isConnected = true;
}

void ResultExchange::connectLocal(void *const *buffers) {
  if (isConnected) throw ScnException("ResultExchange: already connected");
  for (int r = 0; r < world; ++r) {
    if (!buffers[r]) throw ScnException("ResultExchange: a peer buffer is missing");
    peers[r] = (r == rank) ? local : buffers[r];
  }
  isConnected = true;
}

void ResultExchange::step(const float *dProbs, int rows, cudaStream_t stream, float *dGathered, int *dRowsStatus) {
  if (!isConnected) throw ScnException("ResultExchange: not connected");
  if (dProbs && (rows < 0 || rows > capRows)) throw ScnException("ResultExchange: more rows than the exchange was made for");
  const unsigned collectStep = collected == published ? 0 : published;
  const unsigned publishStep = dProbs ? published + 1 : 0;
  if (!collectStep && !publishStep) return;
  float *out = dGathered ? dGathered : dOut;
  int *meta = dRowsStatus ? dRowsStatus : deviceRows();
  scnSafeCall(scn_exchange_step(local, collectStep, out, meta, meta + world, dProbs, rows * nClasses, rows, peers, world, rank, capFloats, publishStep,
                                stream));
  collected = published;
  if (publishStep) ++published;
}

void ResultExchange::stepBeside(const float *dProbs, int rows, cudaStream_t main, float *dGathered, int *dRowsStatus) {
  if (!side) {
    cudaSafeCall(cudaStreamCreateWithFlags(&side, cudaStreamNonBlocking));
    cudaSafeCall(cudaEventCreateWithFlags(&mainReady, cudaEventDisableTiming));
    cudaSafeCall(cudaEventCreateWithFlags(&sideDone, cudaEventDisableTiming));
  }
  if (sidePending) cudaSafeCall(cudaStreamWaitEvent(main, sideDone, 0)); // the step before: over long ago, but now ordered
  cudaSafeCall(cudaEventRecord(mainReady, main));
  cudaSafeCall(cudaStreamWaitEvent(side, mainReady, 0));
  step(dProbs, rows, side, dGathered, dRowsStatus);
  cudaSafeCall(cudaEventRecord(sideDone, side));
  sidePending = true;
  if (!dProbs) {
    cudaSafeCall(cudaStreamWaitEvent(main, sideDone, 0));
    sidePending = false;
  }
}

void ResultExchange::copyBlockToHost(cudaStream_t stream) {
  cudaSafeCall(cudaMemcpyAsync(hOut, dOut, blockBytes(), cudaMemcpyDeviceToHost, stream));
}

void ResultExchange::deliver(float *gathered, int *rows) {
  const int *meta = (const int *)(hOut + sizeof(float) * (size_t)world * capFloats);
  const int status = meta[world];
  if (status) {
    cudaMemset(deviceRows() + world, 0, sizeof(int)); // the word is sticky on the device until it has been reported
    std::string who;
    for (int r = 0; r < world; ++r)
      if (status >> r & 1) who += (who.empty() ? "" : ", ") + std::to_string(r);
    throw ScnException("ResultExchange: no block from rank " + who + " within the time limit; the gathered results of that step are not complete");
  }
  if (gathered) std::memcpy(gathered, hOut, sizeof(float) * (size_t)world * capFloats);
  if (rows) std::memcpy(rows, meta, sizeof(int) * world);
}
