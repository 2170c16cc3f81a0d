// Named architectures (NetworkArchitectures.h): DeepCNet and its relatives, expressed as
// sequences of addLeNetLayerMP calls.  l = number of pooling levels, k = width step,
// p = dropout of the last level (earlier levels scale linearly).
#pragma once
#include "SparseConvNet.h"

class DeepCNet : public SparseConvNet {
public:
  DeepCNet(int dimension, int l, int k, ActivationFunction fn, int nInputFeatures, int nClasses, float p = 0.0f, int cudaDevice = -1, int nTop = 1);
};
class DeepC2 : public SparseConvNet {
public:
  DeepC2(int dimension, int l, int k, ActivationFunction fn, int nInputFeatures, int nClasses, float p = 0.0f, int cudaDevice = -1, int nTop = 1);
};
class DeepCNiN : public SparseConvNet {
public:
  DeepCNiN(int dimension, int l, int k, ActivationFunction fn, int nInputFeatures, int nClasses, float p = 0.0f, int cudaDevice = -1, int nTop = 1);
};
class DeepC2C2 : public SparseConvNet {
public:
  DeepC2C2(int dimension, int l, int k, ActivationFunction fn, int nInputFeatures, int nClasses, float p = 0.0f, int cudaDevice = -1, int nTop = 1);
};
class DeepC3C3Valid : public SparseConvNet {
public:
  DeepC3C3Valid(int dimension, int l, int k, ActivationFunction fn, int nInputFeatures, int nClasses, float p = 0.0f, int cudaDevice = -1, int nTop = 1);
};
class DeepC3C3 : public SparseConvNet {
public:
  DeepC3C3(int dimension, int l, int k, ActivationFunction fn, int nInputFeatures, int nClasses, float p = 0.0f, int cudaDevice = -1, int nTop = 1);
};

// The four fractional max-pooling networks (NetworkArchitectures.h:43-69): l blocks of a 2^d
// convolution and an FMP layer of pool size 2, then a 2^d and a 1^d convolution block.
class POFMPSparseConvNet : public SparseConvNet {
public:
  POFMPSparseConvNet(int dimension, int l, int k, float fmpShrink, ActivationFunction fn, int nInputFeatures, int nClasses, float p = 0.0f,
                     int cudaDevice = -1, int nTop = 1);
};
class ROFMPSparseConvNet : public SparseConvNet {
public:
  ROFMPSparseConvNet(int dimension, int l, int k, float fmpShrink, ActivationFunction fn, int nInputFeatures, int nClasses, float p = 0.0f,
                     int cudaDevice = -1, int nTop = 1);
};
class PDFMPSparseConvNet : public SparseConvNet {
public:
  PDFMPSparseConvNet(int dimension, int l, int k, float fmpShrink, ActivationFunction fn, int nInputFeatures, int nClasses, float p = 0.0f,
                     int cudaDevice = -1, int nTop = 1);
};
class RDFMPSparseConvNet : public SparseConvNet {
public:
  RDFMPSparseConvNet(int dimension, int l, int k, float fmpShrink, ActivationFunction fn, int nInputFeatures, int nClasses, float p = 0.0f,
                     int cudaDevice = -1, int nTop = 1);
};
