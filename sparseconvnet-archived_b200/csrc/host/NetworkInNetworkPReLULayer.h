// NetworkInNetworkLayer with a learnt per-channel negative slope
// (NetworkInNetworkPReLULayer.h; slopes start at 0.25, NetworkInNetworkPReLULayer.cu:6).
#pragma once
#include "NetworkInNetworkLayer.h"

class NetworkInNetworkPReLULayer : public NetworkInNetworkLayer {
public:
  vectorCUDA<float> PReLU;  // [nFeaturesOut]
  vectorCUDA<float> MPReLU; // momentum of the SGD update
  vectorCUDA<float> dprelu; // slope gradient of the last training step
  NetworkInNetworkPReLULayer(cudaMemStream &memStream, cublasHandle_t &cublasHandle, int nFeaturesIn, int nFeaturesOut,
                             float dropout = 0, float alpha = 1);
  void loadWeightsFromStream(std::ifstream &f, bool momentum);
  void putWeightsToStream(std::ofstream &f, bool momentum);

protected:
  float *slopes();
  float *slopeGradient();
  void updateSlopes(float learningRate, float momentum, const float *presentMask);
};
