// Reads the class probabilities back and scores them (SoftmaxClassifier.h:10-12).
#pragma once
#include "SpatiallySparseBatch.h"
#include "SpatiallySparseBatchInterface.h"
void SoftmaxClassifier(SpatiallySparseBatchInterface &input, SpatiallySparseBatch &batch, int nTop, cudaMemStream &memStream);
