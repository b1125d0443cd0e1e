// QLMH optimizer-state file: the reference's durable checkpoint of the integer state
// (qlm_save / qlm_load, qlm.cuh:703-788), read and written on caller-owned HOST arrays so that
// a run of this library resumes a reference run and the other way round.  Layout (little endian):
//   "QLMH", int32 hdr[6] = {dmax, group, adam, nspan, packed, iter}, uint64 nq, ngrp, nfloat,
//   bf16 Mc[nfloat], bf16 Vc[nfloat], int8 d[qd_bytes], int8 r[nq], int8 m8[nq], (uint8 v8[nq]),
//   float s[ngrp], float m8s[ngrp], (float v8s[ngrp]),
//   "SREF", int32 nspan, float sref[nspan],  "PGN1", float prev_gn
// The parenthesised arrays exist when adam != 0; files written before the two trailers existed
// end after the scale arrays.  Writing follows the reference's discipline: temporary file,
// flush to disk, atomic rename.
#include <stdio.h>
#include <string.h>
#include <math.h>
#include <unistd.h>
#include "qlmb_common.cuh"

namespace qlmb {
static unsigned long long digit_bytes(unsigned long long nq, int packed) { return packed ? (nq + 1) / 2 : nq; }
static bool wr(FILE *f, const void *p, size_t sz, unsigned long long n) { return n == 0 || fwrite(p, sz, (size_t)n, f) == (size_t)n; }
static bool rd(FILE *f, void *p, size_t sz, unsigned long long n) { return n == 0 || fread(p, sz, (size_t)n, f) == (size_t)n; }
}  // namespace qlmb
using namespace qlmb;

extern "C" int qlmb_statefile_write(const char *path, const qlmb_statefile *v)
{
    QLMB_REQUIRE(path && v, "qlmb_statefile_write: NULL argument");
    QLMB_REQUIRE(v->nspan >= 0 && (v->nq == 0 || (v->d && v->r && v->m8)) && (v->ngrp == 0 || (v->s && v->m8s)),
                 "qlmb_statefile_write: missing array");
    QLMB_REQUIRE(!v->adam || ((v->nq == 0 || v->v8) && (v->ngrp == 0 || v->v8s)), "qlmb_statefile_write: adam state without v8 / v8s");
    QLMB_REQUIRE(v->nfloat == 0 || (v->Mc && v->Vc), "qlmb_statefile_write: float-span moments missing");
    QLMB_REQUIRE(v->nspan == 0 || v->sref, "qlmb_statefile_write: sref missing");
    char tmp[1400];
    QLMB_REQUIRE(strlen(path) < 1300, "qlmb_statefile_write: path too long");
    snprintf(tmp, sizeof tmp, "%s.tmp", path);
    FILE *f = fopen(tmp, "wb");
    if (!f) { set_error("qlmb_statefile_write: cannot create %s", tmp); return QLMB_E_ARG; }
    const int hdr[6] = {v->dmax, v->group, v->adam, v->nspan, v->packed, v->iter};
    const unsigned long long nq = v->nq, ng = v->ngrp, nf = v->nfloat, nd = digit_bytes(nq, v->packed);
    bool ok = wr(f, "QLMH", 1, 4) && wr(f, hdr, 4, 6) && wr(f, &nq, 8, 1) && wr(f, &ng, 8, 1) && wr(f, &nf, 8, 1)
           && wr(f, v->Mc, 2, nf) && wr(f, v->Vc, 2, nf) && wr(f, v->d, 1, nd) && wr(f, v->r, 1, nq) && wr(f, v->m8, 1, nq)
           && (!v->adam || wr(f, v->v8, 1, nq)) && wr(f, v->s, 4, ng) && wr(f, v->m8s, 4, ng) && (!v->adam || wr(f, v->v8s, 4, ng));
    const int ns = v->nspan;
    ok = ok && wr(f, "SREF", 1, 4) && wr(f, &ns, 4, 1) && wr(f, v->sref, 4, (unsigned long long)ns);
    ok = ok && wr(f, "PGN1", 1, 4) && wr(f, &v->prev_gn, 4, 1);
    ok = ok && fflush(f) == 0 && fsync(fileno(f)) == 0;
    if (fclose(f) != 0) ok = false;
    if (!ok) { remove(tmp); set_error("qlmb_statefile_write: write to %s failed (the previous file is kept)", tmp); return QLMB_E_ARG; }
    if (rename(tmp, path) != 0) { remove(tmp); set_error("qlmb_statefile_write: cannot replace %s", path); return QLMB_E_ARG; }
    return QLMB_OK;
}

extern "C" int qlmb_statefile_read_header(const char *path, qlmb_statefile *v)
{
    QLMB_REQUIRE(path && v, "qlmb_statefile_read_header: NULL argument");
    FILE *f = fopen(path, "rb");
    if (!f) { set_error("qlmb_statefile_read_header: cannot open %s", path); return QLMB_E_ARG; }
    char mg[4]; int hdr[6]; unsigned long long n[3];
    bool ok = fread(mg, 1, 4, f) == 4 && !memcmp(mg, "QLMH", 4) && fread(hdr, 4, 6, f) == 6 && fread(n, 8, 3, f) == 3;
    fclose(f);
    if (!ok) { set_error("qlmb_statefile_read_header: %s is not a QLMH file", path); return QLMB_E_ARG; }
    v->dmax = hdr[0]; v->group = hdr[1]; v->adam = hdr[2]; v->nspan = hdr[3]; v->packed = hdr[4]; v->iter = hdr[5];
    v->nq = n[0]; v->ngrp = n[1]; v->nfloat = n[2];
    return QLMB_OK;
}

// The scalar fields of *v describe the state the caller holds (its arrays are sized for them).  As in
// the reference, a file of another shape is refused: dmax, group, adam, packed, nq and ngrp must match
// and the file may hold fewer float-span moments than the caller (the rest keep their values), not more.
// On success iter, nfloat (= the count read), have_sref / sref[] (only when the file's span count
// matches) and have_prev_gn / prev_gn (only a positive finite value, and only after SREF) are filled.
extern "C" int qlmb_statefile_read(const char *path, qlmb_statefile *v)
{
    QLMB_REQUIRE(path && v, "qlmb_statefile_read: NULL argument");
    FILE *f = fopen(path, "rb");
    if (!f) { set_error("qlmb_statefile_read: cannot open %s", path); return QLMB_E_ARG; }
    char mg[4]; int hdr[6]; unsigned long long nq, ng, nf;
    bool ok = fread(mg, 1, 4, f) == 4 && !memcmp(mg, "QLMH", 4) && fread(hdr, 4, 6, f) == 6 && fread(&nq, 8, 1, f) == 1 &&
              fread(&ng, 8, 1, f) == 1 && fread(&nf, 8, 1, f) == 1;
    if (!ok) { fclose(f); set_error("qlmb_statefile_read: %s is not a QLMH file", path); return QLMB_E_ARG; }
    if (hdr[0] != v->dmax || hdr[1] != v->group || hdr[2] != v->adam || hdr[4] != v->packed || nq != v->nq || ng != v->ngrp || nf > v->nfloat) {
        fclose(f);
        set_error("qlmb_statefile_read: %s has a different shape (bits/group/optimizer/sizes)", path);
        return QLMB_E_UNSUPPORTED;
    }
    const unsigned long long nd = digit_bytes(nq, v->packed);
    ok = rd(f, v->Mc, 2, nf) && rd(f, v->Vc, 2, nf) && rd(f, v->d, 1, nd) && rd(f, v->r, 1, nq) && rd(f, v->m8, 1, nq)
      && (!v->adam || rd(f, v->v8, 1, nq)) && rd(f, v->s, 4, ng) && rd(f, v->m8s, 4, ng) && (!v->adam || rd(f, v->v8s, 4, ng));
    if (!ok) { fclose(f); set_error("qlmb_statefile_read: %s is truncated", path); return QLMB_E_ARG; }
    v->iter = hdr[5];
    v->nfloat = nf;
    v->have_sref = 0; v->have_prev_gn = 0;
    char tm[4]; int ns = 0;
    if (fread(tm, 1, 4, f) == 4 && !memcmp(tm, "SREF", 4) && fread(&ns, 4, 1, f) == 1 && ns == v->nspan && (ns == 0 || v->sref))
        v->have_sref = rd(f, v->sref, 4, (unsigned long long)ns) ? 1 : 0;
    float pg = 0.0f;
    if (v->have_sref && fread(tm, 1, 4, f) == 4 && !memcmp(tm, "PGN1", 4) && fread(&pg, 4, 1, f) == 1 && pg > 0.0f && isfinite(pg)) {
        v->prev_gn = pg; v->have_prev_gn = 1;
    }
    fclose(f);
    return QLMB_OK;
}

// ------------------------------------------------------------------ model file (TLM4 / TLM5)
// model_save_bundle / model_load_full (cudalm.cu:554-565, 431-466): magic, 11 (TLM4) or 13 (TLM5, window > 0)
// header ints {V, D, L, H, KV, F, T, eot, tmpl, n_mtp, n_exp[, win, full_every]}, the fp32 parameter vector, the
// tokenizer blob's length and bytes.  A model whose quantised weights exist only as digits writes their rendered
// values (digit * scale), which the reference re-encodes to the same digits.
extern "C" int qlmb_modelfile_write(const char *path, const int *hdr13, const float *P, unsigned long long n,
                                    const void *tok_blob, int tok_bytes)
{
    QLMB_REQUIRE(path && hdr13 && (P || n == 0), "qlmb_modelfile_write: NULL argument");
    QLMB_REQUIRE(tok_bytes >= 0 && (tok_bytes == 0 || tok_blob), "qlmb_modelfile_write: tokenizer blob missing");
    char tmp[1400];
    QLMB_REQUIRE(strlen(path) < 1300, "qlmb_modelfile_write: path too long");
    snprintf(tmp, sizeof tmp, "%s.tmp", path);
    FILE *f = fopen(tmp, "wb");
    if (!f) { set_error("qlmb_modelfile_write: cannot create %s", tmp); return QLMB_E_ARG; }
    const bool win = hdr13[11] > 0;
    bool ok = wr(f, win ? "TLM5" : "TLM4", 1, 4) && wr(f, hdr13, 4, win ? 13 : 11) && wr(f, P, 4, n) && wr(f, &tok_bytes, 4, 1)
           && (tok_bytes == 0 || wr(f, tok_blob, 1, (unsigned long long)tok_bytes));
    ok = ok && fflush(f) == 0 && fsync(fileno(f)) == 0;
    if (fclose(f) != 0) ok = false;
    if (!ok) { remove(tmp); set_error("qlmb_modelfile_write: write to %s failed (the previous file is kept)", tmp); return QLMB_E_ARG; }
    if (rename(tmp, path) != 0) { remove(tmp); set_error("qlmb_modelfile_write: cannot replace %s", path); return QLMB_E_ARG; }
    return QLMB_OK;
}

// Header of a TLM1..TLM5 file into hdr13 (ints a version lacks are 0); *n_params = fp32 values that follow, derived
// from the file length and the tokenizer trailer (the caller checks it against its own layout); *tok_bytes likewise.
extern "C" int qlmb_modelfile_read_header(const char *path, int *hdr13, unsigned long long *n_params, int *tok_bytes)
{
    QLMB_REQUIRE(path && hdr13 && n_params, "qlmb_modelfile_read_header: NULL argument");
    FILE *f = fopen(path, "rb");
    if (!f) { set_error("qlmb_modelfile_read_header: cannot open %s", path); return QLMB_E_ARG; }
    char m[4];
    int nh = 0;
    bool ok = fread(m, 1, 4, f) == 4;
    if (ok) {
        if (!memcmp(m, "TLM5", 4)) nh = 13; else if (!memcmp(m, "TLM4", 4)) nh = 11; else if (!memcmp(m, "TLM3", 4)) nh = 10;
        else if (!memcmp(m, "TLM2", 4)) nh = 9; else if (!memcmp(m, "TLM1", 4)) nh = 8;
    }
    if (!ok || !nh) { fclose(f); set_error("qlmb_modelfile_read_header: %s is not a TLM1..TLM5 model file", path); return QLMB_E_UNSUPPORTED; }
    memset(hdr13, 0, 13 * sizeof(int));
    ok = fread(hdr13, 4, (size_t)nh, f) == (size_t)nh;
    fseek(f, 0, SEEK_END);
    const long long len = ftell(f);
    fclose(f);
    if (!ok) { set_error("qlmb_modelfile_read_header: %s: truncated header", path); return QLMB_E_ARG; }
    const long long body = len - 4 - 4LL * nh;
    // with a tokenizer trailer the body is n*4 + 4 + tok_bytes; the caller's parameter count decides, so report the
    // largest n the file can hold and let qlmb_modelfile_read verify the trailer
    *n_params = body > 0 ? (unsigned long long)(body / 4) : 0;
    if (tok_bytes) *tok_bytes = -1;
    return QLMB_OK;
}

// Reads exactly n fp32 parameters after the header; *tok_bytes = length of the tokenizer blob that follows (0: none),
// copied into tok_blob when it is not NULL and tok_cap is large enough.
extern "C" int qlmb_modelfile_read(const char *path, float *P, unsigned long long n, void *tok_blob, int tok_cap, int *tok_bytes)
{
    QLMB_REQUIRE(path && (P || n == 0), "qlmb_modelfile_read: NULL argument");
    FILE *f = fopen(path, "rb");
    if (!f) { set_error("qlmb_modelfile_read: cannot open %s", path); return QLMB_E_ARG; }
    char m[4];
    int nh = 0;
    if (fread(m, 1, 4, f) == 4) {
        if (!memcmp(m, "TLM5", 4)) nh = 13; else if (!memcmp(m, "TLM4", 4)) nh = 11; else if (!memcmp(m, "TLM3", 4)) nh = 10;
        else if (!memcmp(m, "TLM2", 4)) nh = 9; else if (!memcmp(m, "TLM1", 4)) nh = 8;
    }
    if (!nh) { fclose(f); set_error("qlmb_modelfile_read: %s is not a TLM1..TLM5 model file", path); return QLMB_E_UNSUPPORTED; }
    bool ok = fseek(f, 4 + 4L * nh, SEEK_SET) == 0 && fread(P, 4, n, f) == n;
    if (!ok) { fclose(f); set_error("qlmb_modelfile_read: %s: model body truncated", path); return QLMB_E_ARG; }
    int tl = 0;
    if (fread(&tl, 4, 1, f) != 1) tl = 0;
    if (tl > 0 && tok_blob && tok_cap >= tl && fread(tok_blob, 1, (size_t)tl, f) != (size_t)tl) tl = 0;
    if (tok_bytes) *tok_bytes = tl > 0 ? tl : 0;
    fclose(f);
    return QLMB_OK;
}
