// Interface of the tcgen05/TMEM fused conv/NiN kernel (conv_nin_tc.cu).
#pragma once
#include "scn_common.cuh"

namespace scn {
// Can the tensor-core kernel take this layer shape at this precision?
bool tc_shape_ok(int fs, int nIn, int N, int precision);
// Bytes of the packed copy of W[K x N] the kernel reads (0 if unsupported).
size_t tc_packed_bytes(int K, int N, int precision);
int tc_pack(const float *d_W, int K, int N, int precision, void *d_packed, cudaStream_t s);
// Scratch for splitting K over several CTAs when a layer has few output tiles (0: not useful).
size_t tc_workspace_bytes(int rows, int fs, int nIn, int N, int precision);
// Pooling applied by the kernel that finishes a K split (see tc_launch): pooled row w takes the maximum over the
// layer-output rows poolRules[w * cells + c].
struct FinishPool { const int *poolRules; int cells, rowsPool; int *choices; };
// A second, small learnt layer (N2 <= 16 outputs, fp32, softmax allowed) applied by the kernel that finishes a K split.
struct FinishNin { const float *W2, *B2, *prelu2; int N2; float p2; int act2; float *out2; };
int tc_launch(const float *d_in, const int *d_rules, int rows, int fs, int nIn, const void *d_packed,
              const float *d_B, const float *d_prelu, int N, float p, int act, int precision, float *d_out,
              void *d_ws, size_t wsBytes, cudaStream_t s, const int *d_rows = nullptr, const int *d_pool_rules = nullptr,
              int pool_cells = 0, int *d_choices = nullptr, int rows_unpooled = 0, const FinishPool *finish_pool = nullptr,
              const FinishNin *finish_nin = nullptr);
// d_pool_rules: a non-overlapping max-pooling layer behind this layer is applied in the epilogue: `rows` then
// counts pooled rows, d_out / d_choices receive the pooled values and choices ([rows x N]), the layer's own
// output is never written.  3xTF32 without K split; pool_cells a power of two in 2..32.  rows_unpooled > 0 (rows
// of the layer's own output): the launch is refused where fusing would cost an extra wave of tiles.
// d_rows: when not null the kernel takes its row count from there (clamped to `rows`, which then is an
// upper bound); 3xTF32 without K split only.
// Error code a bounded wait of the kernel recorded since the last call (0 = none); waits for
// the device and clears it.  1 gather/empty, 2 epilogue/accumulator, 3 weight copy/empty, 4 MMA/full.
int tc_take_error();
// Device address of that error word on the current device (nullptr if it cannot be resolved): kernels that
// hand results to the host read and clear it there, so that the host sees it in a copy it makes anyway.
int *tc_error_word();
} // namespace scn
