// Exact 4-bit export of a parameter vector ("q4n") and its reader, on the device, plus the quantised container
// file.  Follows quantize_params / dequantize_params with qtype 3 (cudalm.cu:639-656, 688-695) and the TLQ1 / TLQ2
// container of the reference's quantize command and loader (cudalm.cu:9788-9793, 438-450).
//
// Stream layout per group of `group` values: a fp32 scale followed by ceil(g/2) bytes of two's-complement nibble
// pairs (even element in the low nibble); a group that lies on no 4-bit grid stores a NaN scale followed by its g
// raw fp32 values.  The scale is found by the reference's search: for k = 7..1 the candidates amax/k, its two
// neighbours below and above in that order {s0, -1 ulp, +1 ulp, -2 ulp, +2 ulp}; the first one for which every value
// satisfies |rint(P/s)| <= 7 and rint(P/s) * s == P wins.  Built with --fmad=false: every operation rounds once.
#include "qlmb_common.cuh"
#include <string.h>
#include <stdlib.h>
#include <unistd.h>
#include <math.h>

namespace qlmb {
namespace {

__device__ __forceinline__ int group_len(unsigned long long n, int group, long long gi)
{
    const unsigned long long i0 = (unsigned long long)gi * group;
    return i0 + group <= n ? group : (int)(n - i0);
}

// one warp per group: scale[gi] (NaN = raw), bytes[gi] = stream bytes of the group
__global__ void __launch_bounds__(256) k_q4n_search(float *scale, unsigned *bytes, const float *P, unsigned long long n, int group,
                                                    long long ng)
{
    const long long gi = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (gi >= ng) return;
    const int g = group_len(n, group, gi);
    const float *p = P + (unsigned long long)gi * group;
    float amax = 0.0f;
    for (int j = lane; j < g; j += 32) { const float a = fabsf(p[j]); if (a > amax) amax = a; }
    for (int o = 16; o; o >>= 1) { const float b = __shfl_xor_sync(~0u, amax, o); if (b > amax) amax = b; }
    int ok = amax == 0.0f;
    float s = 0.0f;
    for (int k = 7; k >= 1 && !ok; k--) {
        const float s0 = __fdiv_rn(amax, (float)k);
        float c[5];
        c[0] = s0; c[1] = nextafterf(s0, 0.0f); c[2] = nextafterf(s0, INFINITY);
        c[3] = nextafterf(c[1], 0.0f); c[4] = nextafterf(c[2], INFINITY);
        for (int t = 0; t < 5 && !ok; t++) {
            s = c[t];
            int good = 1;
            for (int j = lane; j < g; j += 32) {
                const float v = p[j], d = rintf(__fdiv_rn(v, s));
                if (fabsf(d) > 7.0f || __fmul_rn(d, s) != v) good = 0;
            }
            ok = __all_sync(~0u, good);
        }
    }
    if (lane == 0) {
        scale[gi] = ok ? s : __int_as_float(0x7fc00000);
        bytes[gi] = 4u + (ok ? (unsigned)((g + 1) / 2) : 4u * (unsigned)g);
    }
}

// exclusive prefix sums of bytes[ng] into off[ng + 1] by one block; totals[0] = stream length, totals[1] = raw groups
__global__ void __launch_bounds__(1024) k_q4n_scan(unsigned long long *off, unsigned long long *totals, const unsigned *bytes,
                                                   const float *scale, long long ng)
{
    __shared__ unsigned long long part[1024], rawp[1024];
    const int t = threadIdx.x;
    const long long chunk = (ng + 1023) / 1024, lo = t * chunk, hi = lo + chunk < ng ? lo + chunk : ng;
    unsigned long long sum = 0, raw = 0;
    for (long long i = lo; i < hi; i++) { sum += bytes[i]; const float s = scale[i]; raw += s != s; }
    part[t] = sum; rawp[t] = raw;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {
        const unsigned long long a = t >= o ? part[t - o] : 0, b = t >= o ? rawp[t - o] : 0;
        __syncthreads();
        part[t] += a; rawp[t] += b;
        __syncthreads();
    }
    unsigned long long run = part[t] - sum;
    for (long long i = lo; i < hi; i++) { off[i] = run; run += bytes[i]; }
    if (t == 1023) { off[ng] = part[t]; totals[0] = part[t]; totals[1] = rawp[t]; }
}

__global__ void __launch_bounds__(256) k_q4n_pack(unsigned char *out, unsigned long long cap, const unsigned long long *off,
                                                  const float *scale, const float *P, unsigned long long n, int group, long long ng)
{
    const long long gi = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (gi >= ng || off[ng] > cap) return;
    const int g = group_len(n, group, gi);
    const float *p = P + (unsigned long long)gi * group;
    unsigned char *o = out + off[gi];
    const float s = scale[gi];
    if (lane == 0) *(float *)o = s;
    o += 4;
    if (s != s) {
        for (int j = lane; j < g; j += 32) ((float *)o)[j] = p[j];
        return;
    }
    for (int b = lane; b < (g + 1) / 2; b += 32) {
        const int j = 2 * b;
        const int lo = s != 0.0f ? (int)rintf(__fdiv_rn(p[j], s)) : 0;
        const int hi = (j + 1 < g && s != 0.0f) ? (int)rintf(__fdiv_rn(p[j + 1], s)) : 0;
        o[b] = (unsigned char)((lo & 15) | ((hi & 15) << 4));
    }
}

__global__ void __launch_bounds__(256) k_q4n_decode(float *P, const unsigned char *in, const unsigned long long *off,
                                                    unsigned long long n, int group, long long ng)
{
    const long long gi = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (gi >= ng) return;
    const int g = group_len(n, group, gi);
    float *p = P + (unsigned long long)gi * group;
    const unsigned char *o = in + off[gi];
    const float s = *(const float *)o;
    o += 4;
    if (s != s) {
        for (int j = lane; j < g; j += 32) p[j] = ((const float *)o)[j];
        return;
    }
    for (int j = lane; j < g; j += 32) {
        const int b = o[j >> 1], nib = (j & 1) ? (b >> 4) : (b & 15);
        p[j] = __fmul_rn((float)((nib ^ 8) - 8), s);
    }
}

bool wr(FILE *f, const void *p, size_t sz, unsigned long long cnt) { return cnt == 0 || fwrite(p, sz, (size_t)cnt, f) == (size_t)cnt; }

} // namespace
} // namespace qlmb

using namespace qlmb;

static inline long long q4n_groups(unsigned long long n, int group) { return (long long)((n + (unsigned long long)group - 1) / (unsigned long long)group); }

extern "C" unsigned long long qlmb_q4n_work_bytes(unsigned long long n, int group)
{
    if (group <= 0) return 0;
    const unsigned long long ng = (unsigned long long)q4n_groups(n, group);
    return (ng + 1) * 8 + ng * 4 + ng * 4 + 64;
}
extern "C" unsigned long long qlmb_q4n_max_bytes(unsigned long long n, int group)
{
    return group > 0 ? (unsigned long long)q4n_groups(n, group) * 4 + n * 4 : 0;
}

extern "C" int qlmb_q4n_export(unsigned char *out, unsigned long long cap, unsigned long long *totals, const float *P,
                               unsigned long long n, int group, void *work, void *stream)
{
    QLMB_REQUIRE(out && totals && P && work, "qlmb_q4n_export: NULL argument");
    QLMB_REQUIRE(n > 0 && group >= 8 && group % 8 == 0 && group <= 4096, "qlmb_q4n_export: n %llu group %d (a multiple of 8 up to 4096)", n, group);
    QLMB_REQUIRE(((uintptr_t)out & 3) == 0 && ((uintptr_t)work & 7) == 0, "qlmb_q4n_export: out needs 4-byte, work 8-byte alignment");
    const long long ng = q4n_groups(n, group);
    unsigned long long *off = (unsigned long long *)work;
    float *scale = (float *)(off + ng + 1);
    unsigned *bytes = (unsigned *)(scale + ng);
    cudaStream_t st = as_stream(stream);
    const unsigned blocks = (unsigned)((ng + 7) / 8);
    k_q4n_search<<<blocks, 256, 0, st>>>(scale, bytes, P, n, group, ng);
    QLMB_LAUNCH_CHECK("k_q4n_search");
    k_q4n_scan<<<1, 1024, 0, st>>>(off, totals, bytes, scale, ng);
    QLMB_LAUNCH_CHECK("k_q4n_scan");
    k_q4n_pack<<<blocks, 256, 0, st>>>(out, cap, off, scale, P, n, group, ng);
    QLMB_LAUNCH_CHECK("k_q4n_pack");
    return QLMB_OK;
}

extern "C" int qlmb_q4n_index(const unsigned char *host_stream, unsigned long long len, unsigned long long n, int group,
                              unsigned long long *off)
{
    QLMB_REQUIRE(host_stream && off && group > 0, "qlmb_q4n_index: bad argument");
    const long long ng = q4n_groups(n, group);
    unsigned long long o = 0;
    for (long long gi = 0; gi < ng; gi++) {
        const unsigned long long i0 = (unsigned long long)gi * group;
        const unsigned long long g = i0 + group <= n ? (unsigned long long)group : n - i0;
        off[gi] = o;
        if (o + 4 > len) { set_error("qlmb_q4n_index: stream ends inside group %lld", gi); return QLMB_E_ARG; }
        float s;
        memcpy(&s, host_stream + o, 4);
        o += 4 + (s != s ? 4 * g : (g + 1) / 2);
        if (o > len) { set_error("qlmb_q4n_index: stream ends inside group %lld", gi); return QLMB_E_ARG; }
    }
    off[ng] = o;
    return QLMB_OK;
}

extern "C" int qlmb_q4n_decode(float *P, const unsigned char *in, const unsigned long long *off, unsigned long long n, int group,
                               void *stream)
{
    QLMB_REQUIRE(P && in && off, "qlmb_q4n_decode: NULL argument");
    QLMB_REQUIRE(n > 0 && group >= 8 && group % 8 == 0, "qlmb_q4n_decode: n %llu group %d", n, group);
    QLMB_REQUIRE(((uintptr_t)in & 3) == 0, "qlmb_q4n_decode: the stream needs 4-byte alignment");
    const long long ng = q4n_groups(n, group);
    k_q4n_decode<<<(unsigned)((ng + 7) / 8), 256, 0, as_stream(stream)>>>(P, in, off, n, group, ng);
    QLMB_LAUNCH_CHECK("k_q4n_decode");
    return QLMB_OK;
}

// ---- the quantised container: "TLQ1" + 11 header ints ("TLQ2" + 13 when the window is set), qtype, group, the body,
// the tokenizer blob's length and bytes (cudalm.cu:9783-9793); written through a temporary file and a rename
extern "C" int qlmb_qfile_write(const char *path, const int *hdr13, int qtype, int group, const void *body, unsigned long long body_len,
                                const void *tok_blob, int tok_bytes)
{
    QLMB_REQUIRE(path && hdr13 && body && group > 0 && qtype >= 0 && qtype <= 3, "qlmb_qfile_write: bad argument");
    QLMB_REQUIRE(tok_bytes >= 0 && (tok_bytes == 0 || tok_blob), "qlmb_qfile_write: tokenizer blob missing");
    QLMB_REQUIRE(strlen(path) < 1300, "qlmb_qfile_write: path too long");
    char tmp[1400];
    snprintf(tmp, sizeof tmp, "%s.tmp", path);
    FILE *f = fopen(tmp, "wb");
    if (!f) { set_error("qlmb_qfile_write: cannot create %s", tmp); return QLMB_E_ARG; }
    const bool win = hdr13[11] > 0;
    bool ok = wr(f, win ? "TLQ2" : "TLQ1", 1, 4) && wr(f, hdr13, 4, win ? 13 : 11) && wr(f, &qtype, 4, 1) && wr(f, &group, 4, 1)
           && wr(f, body, 1, body_len) && wr(f, &tok_bytes, 4, 1) && (tok_bytes == 0 || wr(f, tok_blob, 1, (unsigned long long)tok_bytes));
    ok = ok && fflush(f) == 0 && fsync(fileno(f)) == 0;
    if (fclose(f) != 0) ok = false;
    if (!ok) { remove(tmp); set_error("qlmb_qfile_write: write to %s failed (the previous file is kept)", tmp); return QLMB_E_ARG; }
    if (rename(tmp, path) != 0) { remove(tmp); set_error("qlmb_qfile_write: cannot replace %s", path); return QLMB_E_ARG; }
    return QLMB_OK;
}

// Header of a TLQ1 / TLQ2 file; *rest = bytes after qtype and group (body + tokenizer trailer)
extern "C" int qlmb_qfile_read_header(const char *path, int *hdr13, int *qtype, int *group, unsigned long long *rest)
{
    QLMB_REQUIRE(path && hdr13 && qtype && group && rest, "qlmb_qfile_read_header: NULL argument");
    FILE *f = fopen(path, "rb");
    if (!f) { set_error("qlmb_qfile_read_header: cannot open %s", path); return QLMB_E_ARG; }
    char m[4];
    int nh = 0;
    if (fread(m, 1, 4, f) == 4) nh = !memcmp(m, "TLQ1", 4) ? 11 : !memcmp(m, "TLQ2", 4) ? 13 : 0;
    if (!nh) { fclose(f); set_error("qlmb_qfile_read_header: %s is not a TLQ1 / TLQ2 file", path); return QLMB_E_UNSUPPORTED; }
    memset(hdr13, 0, 13 * sizeof(int));
    bool ok = fread(hdr13, 4, (size_t)nh, f) == (size_t)nh && fread(qtype, 4, 1, f) == 1 && fread(group, 4, 1, f) == 1;
    fseek(f, 0, SEEK_END);
    const long long len = ftell(f);
    fclose(f);
    if (!ok || *group <= 0) { set_error("qlmb_qfile_read_header: %s: bad header", path); return QLMB_E_ARG; }
    *rest = (unsigned long long)(len - 4 - 4LL * nh - 8);
    return QLMB_OK;
}

// Reads the `rest` bytes after the header into buf (host).  For a q4n body of n parameters the caller indexes buf with
// qlmb_q4n_index; off[groups] is the body's length, followed by the tokenizer blob's length (int) and bytes.
extern "C" int qlmb_qfile_read(const char *path, void *buf, unsigned long long rest)
{
    QLMB_REQUIRE(path && buf, "qlmb_qfile_read: NULL argument");
    FILE *f = fopen(path, "rb");
    if (!f) { set_error("qlmb_qfile_read: cannot open %s", path); return QLMB_E_ARG; }
    char m[4];
    int nh = 0;
    if (fread(m, 1, 4, f) == 4) nh = !memcmp(m, "TLQ1", 4) ? 11 : !memcmp(m, "TLQ2", 4) ? 13 : 0;
    bool ok = nh && fseek(f, 4 + 4L * nh + 8, SEEK_SET) == 0 && fread(buf, 1, (size_t)rest, f) == (size_t)rest;
    fclose(f);
    if (!ok) { set_error("qlmb_qfile_read: %s: short read", path); return QLMB_E_ARG; }
    return QLMB_OK;
}
