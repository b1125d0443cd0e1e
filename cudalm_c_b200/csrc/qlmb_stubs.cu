// Temporary: entry points whose kernels are not built yet.
#include "qlmb_common.cuh"
#define STUB(name) { qlmb::set_error(name ": not built yet"); return QLMB_E_UNSUPPORTED; }
extern "C" {
int qlmb_gemv_decode(void *, const void *, const int8_t *, const float *, int, int, int, int, int, void *) STUB("qlmb_gemv_decode")
}
