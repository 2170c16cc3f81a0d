// tcgen05/TMEM fused conv/NiN kernel -- placeholder until the kernel lands.
#include "conv_nin_tc.cuh"
namespace scn {
bool tc_shape_ok(int, int, int, int) { return false; }
size_t tc_packed_bytes(int, int, int) { return 0; }
int tc_pack(const float *, int, int, int, void *, cudaStream_t) { return fail(SCN_ERR_UNSUPPORTED, "tensor-core path not built"); }
int tc_launch(const float *, const int *, int, int, int, const void *, const float *, const float *, int, float, int, int,
              float *, cudaStream_t) { return fail(SCN_ERR_UNSUPPORTED, "tensor-core path not built"); }
} // namespace scn
