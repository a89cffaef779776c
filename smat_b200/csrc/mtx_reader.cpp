// Matrix-Market reader of the engine (host side).
//
// Replaces mmio_allinone (src/cuda_hgemm/src/common/mmio_highlevel.h:619-786) and keeps its observable
// behaviour: coordinate files only; dimensions padded up to multiples of 16 (:609-616, :650);
// indices 1-based -> 0-based (:702-703); pattern entries get the value 1 (:695-699), complex entries
// keep the real part, integer entries are widened; values are rounded double -> fp16 once (:708);
// symmetric and hermitian files have every off-diagonal entry mirrored (:714-758); the CSR keeps
// FILE order inside each row (counting sort: per-row counts, exclusive scan, scatter, :705-767).
// Differences by design: the file is read in one piece and parsed with strtol/strtod instead of one
// fscanf per line, nothing is leaked, and errors are returned instead of printed.
#include <ctype.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <string>
#include <new>
#include <vector>

#include "smat_internal.h"

namespace smat {

// IEEE binary64 -> binary16 bit pattern, round-to-nearest-even, single rounding.
uint16_t half_bits_from_double(double d) {
    uint64_t u;
    memcpy(&u, &d, sizeof(u));
    const uint16_t sign = (uint16_t)((u >> 48) & 0x8000u);
    const int bexp = (int)((u >> 52) & 0x7FF);
    const uint64_t frac = u & ((1ull << 52) - 1);
    if (bexp == 0x7FF) return (uint16_t)(sign | 0x7C00u | (frac ? 0x0200u : 0u));
    if (bexp == 0) return sign;  // zero and binary64 subnormals vanish in fp16
    const int e = bexp - 1023;
    if (e > 15) return (uint16_t)(sign | 0x7C00u);
    if (e < -25) return sign;
    const uint64_t sig = frac | (1ull << 52);
    const int drop = (e >= -14) ? 42 : 42 + (-14 - e);
    uint64_t q = sig >> drop;
    const uint64_t rest = sig & ((1ull << drop) - 1), half = 1ull << (drop - 1);
    if (rest > half || (rest == half && (q & 1))) q++;
    uint32_t bits = (e >= -14) ? (uint32_t)(((uint64_t)(e + 14) << 10) + q) : (uint32_t)q;
    if (bits > 0x7C00u) bits = 0x7C00u;
    return (uint16_t)(sign | bits);
}

}  // namespace smat

using namespace smat;

extern "C" {

void smat_free_host(void* p) { free(p); }

int smat_read_mtx(const char* filename, size_t* M, size_t* K, size_t* nnz, int* is_symmetric, int** csr_rowptr,
                  int** csr_colidx, uint16_t** csr_vals) {
    clear_error();
    if (!filename || !M || !K || !nnz || !csr_rowptr || !csr_colidx || !csr_vals)
        return fail(SMAT_ERR_BAD_ARG, "NULL argument");
    FILE* f = fopen(filename, "rb");
    if (!f) return fail(SMAT_ERR_IO, "cannot open %s", filename);
    fseek(f, 0, SEEK_END);
    const long fsize = ftell(f);
    fseek(f, 0, SEEK_SET);
    if (fsize < 0) {
        fclose(f);
        return fail(SMAT_ERR_IO, "%s: cannot determine the file size", filename);
    }
    std::vector<char> text;
    try {
        text.resize((size_t)fsize + 1);
    } catch (const std::bad_alloc&) {
        fclose(f);
        return fail(SMAT_ERR_NOMEM, "%s: %ld bytes do not fit in host memory", filename, fsize);
    }
    const size_t got = fread(text.data(), 1, (size_t)fsize, f);
    fclose(f);
    if (got != (size_t)fsize) return fail(SMAT_ERR_IO, "%s: short read (%zu of %ld bytes)", filename, got, fsize);
    text[got] = 0;
    char* cur = text.data();
    char* const end = text.data() + got;

    // banner
    char* eol = (char*)memchr(cur, '\n', (size_t)(end - cur));
    if (!eol) return fail(SMAT_ERR_IO, "%s: no Matrix-Market banner", filename);
    std::string banner(cur, eol);
    for (char& ch : banner) ch = (char)tolower((unsigned char)ch);
    char w0[64], w1[64], w2[64], w3[64], w4[64];
    if (sscanf(banner.c_str(), "%63s %63s %63s %63s %63s", w0, w1, w2, w3, w4) != 5 || strcmp(w0, "%%matrixmarket") ||
        strcmp(w1, "matrix"))
        return fail(SMAT_ERR_IO, "%s: could not process the Matrix-Market banner", filename);
    if (strcmp(w2, "coordinate")) return fail(SMAT_ERR_IO, "%s: only coordinate files are supported", filename);
    enum { REAL, COMPLEX, INTEGER, PATTERN } field;
    if (!strcmp(w3, "real")) field = REAL;
    else if (!strcmp(w3, "complex")) field = COMPLEX;
    else if (!strcmp(w3, "integer")) field = INTEGER;
    else if (!strcmp(w3, "pattern")) field = PATTERN;
    else return fail(SMAT_ERR_IO, "%s: unknown field '%s'", filename, w3);
    const bool mirror = !strcmp(w4, "symmetric") || !strcmp(w4, "hermitian");
    cur = eol + 1;

    // comments, then "rows cols entries"
    long rows = 0, cols = 0, entries = 0;
    for (;;) {
        if (cur >= end) return fail(SMAT_ERR_IO, "%s: size line missing", filename);
        eol = (char*)memchr(cur, '\n', (size_t)(end - cur));
        if (!eol) eol = end;
        if (*cur != '%') {
            std::string line(cur, eol);
            cur = eol < end ? eol + 1 : end;
            if (sscanf(line.c_str(), "%ld %ld %ld", &rows, &cols, &entries) == 3) break;
            continue;
        }
        cur = eol + 1;
    }
    if (rows < 0 || cols < 0 || entries < 0) return fail(SMAT_ERR_IO, "%s: negative size", filename);
    // mirroring writes entry (a, b) again as (b, a): only a square matrix has room for it (the reference reads past its
    // arrays here, mmio_highlevel.h:714-758)
    if (mirror && rows != cols) return fail(SMAT_ERR_IO, "%s: a symmetric or hermitian matrix must be square (%ld x %ld)", filename, rows, cols);
    const long rows_p = (rows + 15) / 16 * 16, cols_p = (cols + 15) / 16 * 16;

    std::vector<int> er((size_t)entries), ec((size_t)entries);
    std::vector<uint16_t> ev((size_t)entries);
    std::vector<int> count((size_t)rows_p + 1, 0);
    for (long i = 0; i < entries; i++) {
        char* nx;
        const long a = strtol(cur, &nx, 10);
        if (nx == cur) return fail(SMAT_ERR_IO, "%s: entry %ld of %ld is missing", filename, i + 1, entries);
        cur = nx;
        const long b = strtol(cur, &nx, 10);
        cur = nx;
        double v = 1.0;
        if (field == REAL) { v = strtod(cur, &nx); cur = nx; }
        else if (field == COMPLEX) { v = strtod(cur, &nx); cur = nx; (void)strtod(cur, &nx); cur = nx; }
        else if (field == INTEGER) { v = (double)strtol(cur, &nx, 10); cur = nx; }
        if (a < 1 || a > rows || b < 1 || b > cols)
            return fail(SMAT_ERR_RANGE, "%s: entry %ld has index (%ld, %ld) outside %ld x %ld", filename, i + 1, a, b, rows,
                        cols);
        er[(size_t)i] = (int)(a - 1);
        ec[(size_t)i] = (int)(b - 1);
        ev[(size_t)i] = half_bits_from_double(v);
        count[(size_t)(a - 1)]++;
        if (mirror && a != b) count[(size_t)(b - 1)]++;
    }
    std::vector<char>().swap(text);

    int* rp = (int*)malloc(((size_t)rows_p + 1) * sizeof(int));
    if (!rp) return fail(SMAT_ERR_NOMEM, "out of host memory");
    long run = 0;
    for (long r = 0; r <= rows_p; r++) { rp[r] = (int)run; run += count[(size_t)r]; }
    const long total = rp[rows_p];
    int* ci = (int*)malloc(((size_t)total + 1) * sizeof(int));
    uint16_t* cv = (uint16_t*)malloc(((size_t)total + 1) * sizeof(uint16_t));
    if (!ci || !cv) { free(rp); free(ci); free(cv); return fail(SMAT_ERR_NOMEM, "out of host memory"); }
    std::fill(count.begin(), count.end(), 0);
    for (long i = 0; i < entries; i++) {
        const int r = er[(size_t)i], c = ec[(size_t)i];
        int at = rp[r] + count[(size_t)r]++;
        ci[at] = c;
        cv[at] = ev[(size_t)i];
        if (mirror && r != c) {
            at = rp[c] + count[(size_t)c]++;
            ci[at] = r;
            cv[at] = ev[(size_t)i];
        }
    }
    *M = (size_t)rows_p;
    *K = (size_t)cols_p;
    *nnz = (size_t)total;
    if (is_symmetric) *is_symmetric = mirror ? 1 : 0;
    *csr_rowptr = rp;
    *csr_colidx = ci;
    *csr_vals = cv;
    return SMAT_OK;
}

int smat_partition_block_rows(const int* rowptr, size_t Mb, int parts, size_t* bounds) {
    clear_error();
    if (!rowptr || !bounds || parts < 1) return fail(SMAT_ERR_BAD_ARG, "bad argument");
    const long long total = rowptr[Mb];
    bounds[0] = 0;
    size_t at = 0;
    for (int p = 1; p < parts; p++) {
        // first block-row boundary whose prefix count reaches p/parts of the blocks
        const long long want = (total * p + parts / 2) / parts;
        while (at < Mb && rowptr[at] < want) at++;
        // pick the nearer of the two candidate boundaries
        if (at > bounds[p - 1] && at <= Mb && (want - rowptr[at - 1]) < (rowptr[at] - want) && at - 1 >= bounds[p - 1]) at--;
        if (total == 0) at = Mb * (size_t)p / (size_t)parts;
        bounds[p] = at;
    }
    bounds[parts] = Mb;
    return SMAT_OK;
}

}  // extern "C"
