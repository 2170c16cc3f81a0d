// Reads the class probabilities back and scores them (SoftmaxClassifier.h:10-12).
#pragma once
#include "SpatiallySparseBatch.h"
#include "SpatiallySparseBatchInterface.h"
void SoftmaxClassifier(SpatiallySparseBatchInterface &input, SpatiallySparseBatch &batch, int nTop, cudaMemStream &memStream);
// The device half alone: one kernel, one copy, one wait.  Returns a block in memStream's page-locked staging memory laid out as
// float probabilities[n x nFeatures]; int top[n x nTop]; valid until the stream's staging memory is used again.
const char *fetchClassifierResult(SpatiallySparseBatchInterface &input, int n, int nTop, cudaMemStream &memStream);
