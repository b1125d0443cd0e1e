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
