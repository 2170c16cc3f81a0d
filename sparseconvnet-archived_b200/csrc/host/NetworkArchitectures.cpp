#include "NetworkArchitectures.h"

// Pooling is 3/2 between levels and absent after the last one; dropout grows linearly to p
// (NetworkArchitectures.cpp:3-70).
namespace {
inline float ramp(float p, int i, int l) { return p * i * 1.0f / l; }
} // namespace

DeepCNet::DeepCNet(int dimension, int l, int k, ActivationFunction fn, int nInputFeatures, int nClasses, float p, int cudaDevice, int nTop)
    : SparseConvNet(dimension, nInputFeatures, nClasses, cudaDevice, nTop) {
  for (int i = 0; i <= l; ++i) {
    const bool last = (i == l);
    addLeNetLayerMP((i + 1) * k, i == 0 ? 3 : 2, 1, last ? 1 : 3, last ? 1 : 2, fn, ramp(p, i, l));
  }
  addSoftmaxLayer();
}
DeepC2::DeepC2(int dimension, int l, int k, ActivationFunction fn, int nInputFeatures, int nClasses, float p, int cudaDevice, int nTop)
    : SparseConvNet(dimension, nInputFeatures, nClasses, cudaDevice, nTop) {
  for (int i = 0; i <= l; ++i) {
    const bool last = (i == l);
    addLeNetLayerMP((i + 1) * k, 2, 1, last ? 1 : 3, last ? 1 : 2, fn, ramp(p, i, l));
  }
  addSoftmaxLayer();
}
DeepCNiN::DeepCNiN(int dimension, int l, int k, ActivationFunction fn, int nInputFeatures, int nClasses, float p, int cudaDevice, int nTop)
    : SparseConvNet(dimension, nInputFeatures, nClasses, cudaDevice, nTop) {
  for (int i = 0; i <= l; ++i) {
    const bool last = (i == l);
    addLeNetLayerMP((i + 1) * k, 2, 1, last ? 1 : 3, last ? 1 : 2, fn, ramp(p, i, l));
    addLeNetLayerMP((i + 1) * k, 1, 1, 1, 1, fn, ramp(p, i, l)); // the 1x1 "network in network" step
  }
  addSoftmaxLayer();
}
DeepC2C2::DeepC2C2(int dimension, int l, int k, ActivationFunction fn, int nInputFeatures, int nClasses, float p, int cudaDevice, int nTop)
    : SparseConvNet(dimension, nInputFeatures, nClasses, cudaDevice, nTop) {
  for (int i = 0; i < l; ++i) {
    addLeNetLayerMP((i + 1) * k, 2, 1, 1, 1, fn, ramp(p, i, l));
    addLeNetLayerMP((i + 1) * k, 2, 1, 3, 2, fn, ramp(p, i, l));
  }
  addLeNetLayerMP((l + 1) * k, 2, 1, 1, 1, fn, p);
  addLeNetLayerMP((l + 1) * k, 1, 1, 1, 1, fn, p);
  addSoftmaxLayer();
}
DeepC3C3Valid::DeepC3C3Valid(int dimension, int l, int k, ActivationFunction fn, int nInputFeatures, int nClasses, float p, int cudaDevice, int nTop)
    : SparseConvNet(dimension, nInputFeatures, nClasses, cudaDevice, nTop) {
  for (int i = 0; i < l; ++i) {
    addLeNetLayerMP((i + 1) * k, 3, 1, 1, 1, fn, ramp(p, i, l), -1);
    addLeNetLayerMP((i + 1) * k, 3, 1, 3, 2, fn, ramp(p, i, l), -1);
  }
  addLeNetLayerMP((l + 1) * k, 3, 1, 1, 1, fn, p, +1); // one ordinary convolution at the top
  addLeNetLayerMP((l + 1) * k, 1, 1, 1, 1, fn, p);
  addSoftmaxLayer();
}
DeepC3C3::DeepC3C3(int dimension, int l, int k, ActivationFunction fn, int nInputFeatures, int nClasses, float p, int cudaDevice, int nTop)
    : SparseConvNet(dimension, nInputFeatures, nClasses, cudaDevice, nTop) {
  for (int i = 0; i < l; ++i) {
    addLeNetLayerMP((i + 1) * k, 3, 1, 1, 1, fn, ramp(p, i, l));
    addLeNetLayerMP((i + 1) * k, 3, 1, 3, 2, fn, ramp(p, i, l));
  }
  addLeNetLayerMP((l + 1) * k, 3, 1, 1, 1, fn, p);
  addLeNetLayerMP((l + 1) * k, 1, 1, 1, 1, fn, p);
  addSoftmaxLayer();
}

// NetworkArchitectures.cpp:72-122.
#define SCN_FMP_NET(CLASS, ADD)                                                                                               \
  CLASS::CLASS(int dimension, int l, int k, float fmpShrink, ActivationFunction fn, int nInputFeatures, int nClasses, float p, \
               int cudaDevice, int nTop)                                                                                      \
      : SparseConvNet(dimension, nInputFeatures, nClasses, cudaDevice, nTop) {                                                \
    for (int i = 0; i < l; i++) ADD(k * (i + 1), 2, 1, 2, fmpShrink, fn, p * i / (l + 1));                                    \
    addLeNetLayerMP(k * (l + 1), 2, 1, 1, 1, fn, p * l / (l + 1));                                                            \
    addLeNetLayerMP(k * (l + 2), 1, 1, 1, 1, fn, p);                                                                          \
    addSoftmaxLayer();                                                                                                        \
  }
SCN_FMP_NET(POFMPSparseConvNet, addLeNetLayerPOFMP)
SCN_FMP_NET(ROFMPSparseConvNet, addLeNetLayerROFMP)
SCN_FMP_NET(PDFMPSparseConvNet, addLeNetLayerPDFMP)
SCN_FMP_NET(RDFMPSparseConvNet, addLeNetLayerRDFMP)
#undef SCN_FMP_NET
