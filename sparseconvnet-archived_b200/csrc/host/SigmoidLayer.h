// applySigmoid (SigmoidLayer.h:4-6): the stand-alone activation pass.  The layers fuse the
// activation into their kernel; this entry point exists for callers that apply one themselves.
#pragma once
#include "SpatiallySparseBatchInterface.h"
#include "types.h"
void applySigmoid(SpatiallySparseBatchInterface &input, SpatiallySparseBatchInterface &output, ActivationFunction fn,
                  cudaMemStream &memStream);
