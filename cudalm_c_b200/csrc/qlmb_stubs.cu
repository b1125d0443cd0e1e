// Temporary: entry points whose kernels are not built yet.
#include "qlmb_common.cuh"
#define STUB(name) { qlmb::set_error(name ": not built yet"); return QLMB_E_UNSUPPORTED; }
extern "C" {
int qlmb_linear_fwd(void *, const void *, const int8_t *, const float *, int, int, int, int, const void *, int, void *) STUB("qlmb_linear_fwd")
int qlmb_linear_dgrad(void *, const void *, const int8_t *, const float *, int, int, int, int, float, int, void *) STUB("qlmb_linear_dgrad")
int qlmb_linear_wgrad(float *, const void *, const void *, int, int, int, int, float, int, void *) STUB("qlmb_linear_wgrad")
int qlmb_gemv_decode(void *, const void *, const int8_t *, const float *, int, int, int, int, int, void *) STUB("qlmb_gemv_decode")
size_t qlmb_moe_arena_bytes(int, int, int, int, int) { return 0; }
void *qlmb_moe_arena_member(void *, int, int, int, int, int, const char *) { return nullptr; }
int qlmb_moe_forward(const qlmb_moe_layer *, void *, void *, const void *, const void *, void *) STUB("qlmb_moe_forward")
int qlmb_moe_backward(const qlmb_moe_layer *, void *, void *, const void *, const void *, float *, float *, float *, float *, float, void *) STUB("qlmb_moe_backward")
}
