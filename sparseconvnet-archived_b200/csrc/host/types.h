// Enumerations shared by the host classes; numeric values match the reference
// (types.h:4, 20-29) so integer-coded configuration carries over unchanged.
#pragma once
#include <cstdint>

enum batchType { TRAINBATCH, TESTBATCH, UNLABELEDBATCH, RESCALEBATCH };
extern const char *batchTypeNames[];

enum ActivationFunction { NOSIGMOID, RELU, VLEAKYRELU, LEAKYRELU, TANH, SOFTMAX, PRELU, SIGMOID };
extern const char *sigmoidNames[];

// Multiply-accumulate operations of the NetworkInNetwork layers run so far: rows x inputs x
// outputs per forward, background rows included (types.h:46-52;
// NetworkInNetworkLayer.cu:197-199).  Twice this number is the algorithmic FLOP count.
extern __int128_t multiplyAddCount;
