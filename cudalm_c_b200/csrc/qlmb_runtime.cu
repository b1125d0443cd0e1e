// Status plumbing of libqlm_b200: thread-local error text, the per-device error
// word that kernels with bounded waits report into, and device queries.
#include "qlmb_common.cuh"
#include <string.h>

namespace qlmb {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char *what)
{
    set_error("CUDA error %d (%s) at %s", (int)e, cudaGetErrorString(e), what);
    return QLMB_E_CUDA;
}

static int *g_errword[64];
static int g_sms[64];

int *device_error_word(void)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!g_errword[dev]) {
        int *p = nullptr;
        if (cudaMalloc(&p, 16 * sizeof(int)) != cudaSuccess) return nullptr;
        if (cudaMemset(p, 0, 16 * sizeof(int)) != cudaSuccess) return nullptr;
        g_errword[dev] = p;
    }
    return g_errword[dev];
}

int sm_count(void)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!g_sms[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        g_sms[dev] = n;
    }
    return g_sms[dev];
}

}  // namespace qlmb

extern "C" const char *qlmb_last_error(void) { return qlmb::g_err; }
extern "C" int qlmb_version(void) { return 1; }

extern "C" int qlmb_check_device(void *stream)
{
    int *w = qlmb::device_error_word();
    if (!w) return qlmb::cuda_fail(cudaGetLastError(), "device_error_word");
    int h[4] = {0, 0, 0, 0};
    QLMB_CUDA(cudaMemcpyAsync(h, w, sizeof h, cudaMemcpyDeviceToHost, qlmb::as_stream(stream)));
    QLMB_CUDA(cudaStreamSynchronize(qlmb::as_stream(stream)));
    if (h[0] != 0) {
        qlmb::set_error("device reported error code %d (site %d, block %d, detail %d)", h[0], h[1], h[2], h[3]);
        QLMB_CUDA(cudaMemsetAsync(w, 0, sizeof h, qlmb::as_stream(stream)));
        return QLMB_E_DEVICE;
    }
    return QLMB_OK;
}
