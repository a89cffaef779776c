// TEST INFRASTRUCTURE ONLY -- CPU oracle for the SMaT block-sparse SpMM hot path.
//
// This file is a plain, single-threaded-by-default CPU restatement of the reference's algorithms for
// the path  "read .mtx -> (optional) similarity row reorder -> 16x16 BCSR -> C = A_blocked x B".
// It is the checker for the CUDA product: only the test-suite, the smoke check and the benchmark's
// CPU-baseline leg may load it.  Nothing in the shipped package links or calls it.
//
// Pinning: the integer/structure functions below are checked (tests, "not gpu") against the real
// reference binaries built from the reference sources (oracle/_ref, see oracle/Makefile) and against
// the reference's own known-answer vectors (TEST_similarities fixed rows).  The reference has no test
// that pins the GPU SpMM values (its -enable_check branches are compiled out), so for the multiply
// the oracle follows the reference's CPU blocked multiply (VBR::multiply) arithmetic in fp32.
//
// Every function cites the reference file:line it follows (paths relative to the reference root).
//
// Written in C-style C++ (g++): two steps of the reference depend on libstdc++ behaviour
// (unstable std::sort in get_permutation, std::set iteration in IterativeBlockingKeeper) and are
// reproduced by calling the same library routines.

#include <algorithm>
#include <cctype>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <numeric>
#include <set>
#include <string>
#include <vector>

#include <atomic>
#include <thread>

extern "C" {

// ---------------------------------------------------------------------------------------------
// fp16 helpers (IEEE binary16, round-to-nearest-even).  The reference converts the parsed double
// straight to `half` (src/cuda_hgemm/src/common/mmio_highlevel.h:708), i.e. one rounding.
// ---------------------------------------------------------------------------------------------
uint16_t orc_double_to_half_bits(double d) {
    uint64_t u;
    memcpy(&u, &d, 8);
    uint16_t sign = (uint16_t)((u >> 48) & 0x8000u);
    int64_t exp = (int64_t)((u >> 52) & 0x7FF);
    uint64_t man = u & 0xFFFFFFFFFFFFFull;
    if (exp == 0x7FF) return (uint16_t)(sign | 0x7C00u | (man ? 0x200u : 0));
    if (exp == 0 && man == 0) return sign;
    int64_t e = exp - 1023;  // unbiased
    if (e > 15) return (uint16_t)(sign | 0x7C00u);
    // full significand with hidden bit (53 bits); subnormal doubles are far below half range
    uint64_t sig = (exp == 0) ? man : (man | (1ull << 52));
    int shift;  // number of low bits of `sig` to drop so that the result is the half significand
    if (e >= -14) {
        shift = 52 - 10;  // normal half: keep 11 bits (1 hidden + 10)
    } else {
        shift = 52 - 10 + (int)(-14 - e);  // subnormal half
        if (shift > 63) return sign;
    }
    uint64_t kept = sig >> shift;
    uint64_t rem = sig & ((1ull << shift) - 1);
    uint64_t half_ulp = 1ull << (shift - 1);
    if (rem > half_ulp || (rem == half_ulp && (kept & 1))) kept++;
    uint32_t out;
    if (e >= -14) {
        // kept has 11 bits (or 12 after carry); adding the exponent field absorbs the carry
        out = (uint32_t)(((uint64_t)(e + 15 - 1) << 10) + kept);
    } else {
        out = (uint32_t)kept;  // subnormal; a carry into bit 10 yields the smallest normal
    }
    if (out >= 0x7C00u) out = 0x7C00u;
    return (uint16_t)(sign | out);
}

float orc_half_bits_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1F;
    uint32_t man = h & 0x3FF;
    uint32_t out;
    if (exp == 0) {
        if (man == 0) {
            out = sign;
        } else {
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400));
            out = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FF) << 13);
        }
    } else if (exp == 0x1F) {
        out = sign | 0x7F800000u | (man << 13);
    } else {
        out = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &out, 4);
    return f;
}

void orc_free(void* p) { free(p); }

// ---------------------------------------------------------------------------------------------
// Matrix-Market reader.  Follows mmio_allinone
// (src/cuda_hgemm/src/common/mmio_highlevel.h:619-786):
//   * banner "%%MatrixMarket matrix coordinate <field> <symmetry>", '%' comment lines skipped,
//     then the "rows cols nnz" size line (mmio.h mm_read_banner / mm_read_mtx_crd_size);
//   * rows and cols padded UP to multiples of 16 (padSparseMatrix, :609-616, call at :650);
//   * entries converted from 1-based to 0-based (:702-703);
//   * pattern -> value 1.0 (:695-699); complex keeps the real part (:688-690); integer -> double;
//   * value double -> half in one rounding (:708);
//   * symmetric / hermitian: every off-diagonal entry is mirrored (:714-722, :738-758); skew is not
//     treated as symmetric (:658);
//   * CSR built by per-row counting + exclusive scan (:705,:724) + scatter in FILE order (:761-767),
//     so the columns inside a row keep file order (for a symmetric file an entry is followed
//     immediately by its mirror in the other row's sequence).
// Returns 0 on success; negative codes as the reference (-1 open, -2 banner, -4 size line).
// Output arrays are malloc'ed; free with orc_free.
// ---------------------------------------------------------------------------------------------
static char* read_whole_file(const char* path, size_t* len) {
    FILE* f = fopen(path, "rb");
    if (!f) return nullptr;
    fseek(f, 0, SEEK_END);
    long n = ftell(f);
    fseek(f, 0, SEEK_SET);
    char* buf = (char*)malloc((size_t)n + 1);
    if (!buf) { fclose(f); return nullptr; }
    size_t got = fread(buf, 1, (size_t)n, f);
    fclose(f);
    buf[got] = 0;
    *len = got;
    return buf;
}

int orc_read_mtx(const char* path, int64_t* M, int64_t* N, int64_t* nnz, int* is_symmetric,
                 int** rowptr_out, int** colidx_out, uint16_t** val_out) {
    size_t len = 0;
    char* buf = read_whole_file(path, &len);
    if (!buf) return -1;
    char* p = buf;
    char* end = buf + len;
    // banner line
    char* eol = (char*)memchr(p, '\n', (size_t)(end - p));
    if (!eol) { free(buf); return -2; }
    std::string banner(p, eol);
    for (auto& ch : banner) ch = (char)tolower((unsigned char)ch);
    char tag[64], obj[64], fmt[64], field[64], sym[64];
    if (sscanf(banner.c_str(), "%63s %63s %63s %63s %63s", tag, obj, fmt, field, sym) != 5 ||
        strcmp(tag, "%%matrixmarket") != 0 || strcmp(obj, "matrix") != 0) {
        free(buf);
        return -2;
    }
    int isPattern = !strcmp(field, "pattern"), isReal = !strcmp(field, "real"),
        isComplex = !strcmp(field, "complex"), isInteger = !strcmp(field, "integer");
    int symm = (!strcmp(sym, "symmetric") || !strcmp(sym, "hermitian")) ? 1 : 0;
    p = eol + 1;
    // comment lines, then the size line
    long m_tmp = 0, n_tmp = 0, nnz_rep = 0;
    for (;;) {
        if (p >= end) { free(buf); return -4; }
        eol = (char*)memchr(p, '\n', (size_t)(end - p));
        if (!eol) eol = end;
        if (*p == '%') { p = eol + 1; continue; }
        std::string line(p, eol);
        p = (eol < end) ? eol + 1 : end;
        if (sscanf(line.c_str(), "%ld %ld %ld", &m_tmp, &n_tmp, &nnz_rep) == 3) break;
    }
    // pad to multiples of 16
    if (m_tmp % 16) m_tmp += 16 - m_tmp % 16;
    if (n_tmp % 16) n_tmp += 16 - n_tmp % 16;

    std::vector<int> ri((size_t)nnz_rep), ci((size_t)nnz_rep);
    std::vector<uint16_t> vv((size_t)nnz_rep);
    std::vector<int> counter((size_t)m_tmp + 1, 0);
    for (long i = 0; i < nnz_rep; i++) {
        char* q;
        long a = strtol(p, &q, 10); p = q;
        long b = strtol(p, &q, 10); p = q;
        double fval = 1.0;
        if (isReal) { fval = strtod(p, &q); p = q; }
        else if (isComplex) { fval = strtod(p, &q); p = q; (void)strtod(p, &q); p = q; }
        else if (isInteger) { fval = (double)strtol(p, &q, 10); p = q; }
        else if (isPattern) { fval = 1.0; }
        a--; b--;
        counter[(size_t)a]++;
        ri[(size_t)i] = (int)a;
        ci[(size_t)i] = (int)b;
        vv[(size_t)i] = orc_double_to_half_bits(fval);
    }
    free(buf);
    if (symm)
        for (long i = 0; i < nnz_rep; i++)
            if (ri[(size_t)i] != ci[(size_t)i]) counter[(size_t)ci[(size_t)i]]++;
    // exclusive scan (mmio_highlevel.h:11-26)
    {
        int run = 0;
        for (long i = 0; i <= m_tmp; i++) { int c = counter[(size_t)i]; counter[(size_t)i] = run; run += c; }
    }
    int total = counter[(size_t)m_tmp];
    int* rowptr = (int*)malloc(((size_t)m_tmp + 1) * sizeof(int));
    int* colidx = (int*)malloc(((size_t)total + 1) * sizeof(int));
    uint16_t* val = (uint16_t*)malloc(((size_t)total + 1) * sizeof(uint16_t));
    memcpy(rowptr, counter.data(), ((size_t)m_tmp + 1) * sizeof(int));
    std::vector<int> fill((size_t)m_tmp + 1, 0);
    for (long i = 0; i < nnz_rep; i++) {
        int r = ri[(size_t)i], c = ci[(size_t)i];
        int off = rowptr[r] + fill[(size_t)r]++;
        colidx[off] = c; val[off] = vv[(size_t)i];
        if (symm && r != c) {
            off = rowptr[c] + fill[(size_t)c]++;
            colidx[off] = r; val[off] = vv[(size_t)i];
        }
    }
    *M = m_tmp; *N = n_tmp; *nnz = total; *is_symmetric = symm;
    *rowptr_out = rowptr; *colidx_out = colidx; *val_out = val;
    return 0;
}

// ---------------------------------------------------------------------------------------------
// CSR -> BCSR with 16x16 blocks.  Follows SparseMatrix::csrToBcsr
// (src/cuda_hgemm/src/common/matrix.h:376-502):
//   * a block is nonzero iff it holds at least one STORED entry, whatever its value (:388-404);
//   * blocks are numbered by a row-major scan over the (Mb x Kb) block grid (:425-431), which is
//     also the order in which bcsrRowPtr / bcsrColIdx are emitted (:441-463), so the block of
//     (blockRow, blockCol) sits at position rowptr[blockRow] + rank of blockCol in that row;
//   * bcsrColIdx holds the ELEMENT column of the block's left edge (col, a multiple of 16) (:455);
//   * values: zero-filled (:436), entry (row, col) lands at block*256 + (row%16)*16 + col%16 (:482);
//     duplicates: the last one in CSR order wins (:470-487).
// The reference materialises two dense Mb*Kb int maps; here one block-row of flags is kept at a
// time, which yields the same arrays.  Two-call protocol: pass vals_out == NULL to get nnzb and
// bcsr_rowptr only.
// ---------------------------------------------------------------------------------------------
int orc_csr_to_bcsr(int64_t M, int64_t K, const int* rowptr, const int* colidx, const uint16_t* vals,
                    int64_t* nnzb_out, int* bcsr_rowptr, int* bcsr_colidx, uint16_t* bcsr_vals) {
    const int64_t Mb = M / 16, Kb = (K + 15) / 16;
    std::vector<int> slot((size_t)Kb, -1);
    std::vector<int> touched;
    int64_t nb = 0;
    for (int64_t br = 0; br < Mb; br++) {
        bcsr_rowptr[br] = (int)nb;
        touched.clear();
        for (int64_t row = br * 16; row < br * 16 + 16; row++)
            for (int j = rowptr[row]; j < rowptr[row + 1]; j++) {
                int bc = colidx[j] / 16;
                if (slot[(size_t)bc] < 0) { slot[(size_t)bc] = 0; touched.push_back(bc); }
            }
        std::sort(touched.begin(), touched.end());
        for (size_t t = 0; t < touched.size(); t++) {
            slot[(size_t)touched[t]] = (int)(nb + (int64_t)t);
            if (bcsr_colidx) bcsr_colidx[nb + (int64_t)t] = touched[t] * 16;
        }
        if (bcsr_vals) {
            memset(bcsr_vals + nb * 256, 0, touched.size() * 256 * sizeof(uint16_t));
            for (int64_t row = br * 16; row < br * 16 + 16; row++)
                for (int j = rowptr[row]; j < rowptr[row + 1]; j++) {
                    int col = colidx[j];
                    int64_t b = slot[(size_t)(col / 16)];
                    bcsr_vals[b * 256 + (row % 16) * 16 + col % 16] = vals[j];
                }
        }
        nb += (int64_t)touched.size();
        for (int bc : touched) slot[(size_t)bc] = -1;
    }
    bcsr_rowptr[Mb] = (int)nb;
    *nnzb_out = nb;
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Blocked multiply  C = A_bcsr x B  on the CPU, fp32 arithmetic on fp16-rounded inputs.
// Arithmetic follows VBR::multiply (preprocess/src/general/vbr.cpp:323-372): for every nonzero
// block, in block-row order then stored order, C_blk[i][j] += A_blk[i][k] * B[k][j] with k
// innermost (:358-363), fp32 multiply-add into a zeroed fp32 C (DataT = DataT_C = float,
// preprocess/include/definitions.h:5-6).  Layouts follow the GPU boundary
// (src/cuda_hgemm/src/mma/mmaCBT.cu:49,52,78): A blocks row-major 16x16, B element (k,n) at
// B[n*K + k], C row-major M x N.  C is returned in fp32 (the caller rounds to fp16 to compare).
// Block-rows [brow_begin, brow_end) are computed; `threads` > 1 hands block-rows out to
// std::threads (the per-element summation order is unchanged).
// ---------------------------------------------------------------------------------------------
int orc_bcsr_spmm_f32(const uint16_t* bvals, const int* browptr, const int* bcolidx,
                      const uint16_t* B, float* C, int64_t M, int64_t N, int64_t K,
                      int64_t brow_begin, int64_t brow_end, int threads) {
    (void)M;
    if (threads < 1) threads = 1;
    std::atomic<int64_t> next(brow_begin);
    auto worker = [&]() {
      std::vector<float> bpanel((size_t)(16 * N));
      float ablk[256];
      for (;;) {
        const int64_t br = next.fetch_add(1);
        if (br >= brow_end) break;
        float* Crow = C + (br - brow_begin) * 16 * N;
        for (int64_t t = 0; t < 16 * N; t++) Crow[t] = 0.0f;
        for (int p = browptr[br]; p < browptr[br + 1]; p++) {
            const int c0 = bcolidx[p];
            for (int t = 0; t < 256; t++) ablk[t] = orc_half_bits_to_float(bvals[(int64_t)p * 256 + t]);
            for (int64_t n = 0; n < N; n++)
                for (int k = 0; k < 16; k++)
                    bpanel[(size_t)(n * 16 + k)] = orc_half_bits_to_float(B[n * K + c0 + k]);
            for (int i = 0; i < 16; i++)
                for (int64_t n = 0; n < N; n++) {
                    float acc = Crow[i * N + n];
                    for (int k = 0; k < 16; k++) acc += ablk[i * 16 + k] * bpanel[(size_t)(n * 16 + k)];
                    Crow[i * N + n] = acc;
                }
        }
      }
    };
    if (threads == 1) {
        worker();
    } else {
        std::vector<std::thread> pool;
        for (int t = 0; t < threads; t++) pool.emplace_back(worker);
        for (auto& th : pool) th.join();
    }
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Jaccard distance between a group pattern and a row, on column-block quotients.
// Follows JaccardDistanceGroup (preprocess/src/general/blocking.cpp:904-975): both inputs are
// ascending column lists; columns are quotiented by block_size; a block present only in A adds
// group_size_B to `count`, only in B adds group_size_A (count_zeros = 1, :911-918);
// result = 2*count / (nA*gA + nB*gB + count) evaluated in double and returned as float (:974);
// both empty -> 0, exactly one empty -> 1 (:907-908).
// ---------------------------------------------------------------------------------------------
float orc_jaccard_group(const int64_t* rowA, int64_t sizeA, int64_t gA, const int64_t* rowB,
                        int64_t sizeB, int64_t gB, int64_t bs) {
    if (sizeA == 0 && sizeB == 0) return 0;
    if (sizeA == 0 || sizeB == 0) return 1;
    int64_t i = 0, j = 0, count = 0, nA = 0, nB = 0;
    while (i < sizeA && j < sizeB) {
        int64_t pa = rowA[i] / bs, pb = rowB[j] / bs;
        if (pa < pb) { count += gB; nA++; while (i < sizeA && rowA[i] / bs == pa) i++; }
        else if (pa > pb) { count += gA; nB++; while (j < sizeB && rowB[j] / bs == pb) j++; }
        else {
            nA++; nB++;
            while (i < sizeA && rowA[i] / bs == pa) i++;
            while (j < sizeB && rowB[j] / bs == pb) j++;
        }
    }
    while (i < sizeA) { int64_t pa = rowA[i] / bs; count += gB; nA++; while (i < sizeA && rowA[i] / bs == pa) i++; }
    while (j < sizeB) { int64_t pb = rowB[j] / bs; count += gA; nB++; while (j < sizeB && rowB[j] / bs == pb) j++; }
    return (float)((2.0 * (double)count) / (double)(nA * gA + nB * gB + count));
}

// Hamming distance on column-block quotients, same calling convention
// (HammingDistanceGroup, preprocess/src/general/blocking.cpp:701-760): counts blocks present in
// exactly one of the two lists, weighted like the Jaccard count.
float orc_hamming_group(const int64_t* rowA, int64_t sizeA, int64_t gA, const int64_t* rowB,
                        int64_t sizeB, int64_t gB, int64_t bs) {
    int64_t i = 0, j = 0, count = 0;
    while (i < sizeA && j < sizeB) {
        int64_t pa = rowA[i] / bs, pb = rowB[j] / bs;
        if (pa < pb) { count += gB; while (i < sizeA && rowA[i] / bs == pa) i++; }
        else if (pa > pb) { count += gA; while (j < sizeB && rowB[j] / bs == pb) j++; }
        else {
            while (i < sizeA && rowA[i] / bs == pa) i++;
            while (j < sizeB && rowB[j] / bs == pb) j++;
        }
    }
    while (i < sizeA) { int64_t pa = rowA[i] / bs; count += gB; while (i < sizeA && rowA[i] / bs == pa) i++; }
    while (j < sizeB) { int64_t pb = rowB[j] / bs; count += gA; while (j < sizeB && rowB[j] / bs == pb) j++; }
    return (float)count;
}

// merge_rows (preprocess/src/general/utilities.cpp:145-173).  NOT a plain set union: the
// reference walks the row B, and for each of its values copies the pattern A up to that value's
// lower bound and then the value; when B is exhausted first, the rest of A (every pattern entry
// beyond the position reached for the last value of B) is DROPPED (:171 appends only the rest of
// B).  When A is exhausted first the rest of B is appended.  The clustering depends on this, so it
// is restated as it behaves.
static std::vector<int64_t> merge_rows_ref(const std::vector<int64_t>& A, const int64_t* B, int64_t sizeB) {
    std::vector<int64_t> out;
    out.reserve(A.size() + (size_t)sizeB);
    size_t i = 0;
    int64_t j = 0;
    while (j < sizeB) {
        const int64_t bval = B[j];
        size_t ni = (size_t)(std::lower_bound(A.begin() + (long)i, A.end(), bval) - A.begin());
        if (ni == A.size()) break;
        out.insert(out.end(), A.begin() + (long)i, A.begin() + (long)ni);
        out.push_back(bval);
        if (A[ni] == bval) ni++;
        i = ni;
        j++;
    }
    out.insert(out.end(), B + j, B + sizeB);
    return out;
}

// ---------------------------------------------------------------------------------------------
// Greedy similarity clustering, the algorithm SMaT runs as "-a 5".
// Follows IterativeBlockingKeeper (preprocess/src/general/blocking.cpp:431-547) statement by
// statement, including its quirks:
//   * `float distances[rows] = {-1}` : element 0 is -1, every other element 0 (:434);
//   * the pruning test compares stale distances of seed and candidate (:467-471);
//   * candidates beyond tau are kept in a std::set<pair<float,intT>>; when it grows past
//     k = max_row_block_size - merged_rows.size() the reference executes
//     `it = end(); advance(it, k); erase(it, end())` (:504-510).  Incrementing end() of a
//     libstdc++ red-black tree walks header -> leftmost-of-rightmost -> ... -> header cyclically,
//     so the call erases the last 0, 1 or 2 elements depending on k and on whether the rightmost
//     node has a left child.  That walk is reproduced here on the real std::set by reading the
//     node links, which are public members of libstdc++'s iterator;
//   * complete groups get id `seed`, incomplete ones `seed + rows` (:448, :525-531).
// Inputs: ragged CSR pattern as rowptr (int64, rows+1) + ascending column indices (int64).
// Output: grouping[rows].
// ---------------------------------------------------------------------------------------------
int orc_keeper_grouping(int64_t rows, const int64_t* rowptr, const int64_t* cols, float tau,
                        int64_t col_block_size, int64_t max_row_block_size, int use_pattern,
                        int64_t* grouping) {
    std::vector<float> distances((size_t)rows, 0.0f);
    if (rows > 0) distances[0] = -1.0f;
    for (int64_t i = 0; i < rows; i++) grouping[i] = -1;
    for (int64_t i = 0; i < rows; i++) {
        if (grouping[i] != -1) continue;
        std::set<std::pair<float, int64_t>> best;
        std::vector<int64_t> merged;
        int64_t group_number = i + rows;
        int64_t gsize = 1;
        grouping[i] = group_number;
        merged.push_back(i);
        std::vector<int64_t> pattern(cols + rowptr[i], cols + rowptr[i + 1]);
        for (int64_t j = i + 1; j < rows; j++) {
            if (gsize == max_row_block_size) break;
            if (distances[(size_t)i] != -1 && distances[(size_t)j] != -1 &&
                std::abs(distances[(size_t)i] - distances[(size_t)j]) > tau) {
                distances[(size_t)j] = -1;
                continue;
            }
            if (grouping[j] != -1) continue;
            float dist = orc_jaccard_group(pattern.data(), (int64_t)pattern.size(), gsize, cols + rowptr[j],
                                           rowptr[j + 1] - rowptr[j], 1, col_block_size);
            distances[(size_t)j] = dist;
            if (dist <= tau) {
                grouping[j] = group_number;
                merged.push_back(j);
                if (use_pattern) pattern = merge_rows_ref(pattern, cols + rowptr[j], rowptr[j + 1] - rowptr[j]);
                gsize++;
            } else {
                best.insert({dist, j});
                int64_t k = max_row_block_size - (int64_t)merged.size();
                if ((int64_t)best.size() > k) {
                    // emulate advance(end(), k) on libstdc++'s tree
                    auto hdr = best.end()._M_node;
                    auto rightmost = hdr->_M_right;
                    bool has_left = rightmost->_M_left != nullptr;
                    int64_t cyc = has_left ? 3 : 2;
                    int64_t pos = k % cyc;  // 0 = end(), 1 = first node after end(), ...
                    int64_t n_erase = 0;
                    if (pos != 0) n_erase = cyc - pos;  // distance from that node to end()
                    // same range-erase call as the reference, so the tree is rebalanced identically
                    if (n_erase > 0) best.erase(std::prev(best.end(), n_erase), best.end());
                }
            }
        }
        if (gsize < max_row_block_size) {
            for (auto it = best.begin(); it != best.end() && gsize != max_row_block_size; ++it) {
                grouping[it->second] = group_number;
                merged.push_back(it->second);
                gsize++;
            }
        }
        if (gsize == max_row_block_size)
            for (int64_t idx : merged) grouping[idx] -= rows;
    }
    return 0;
}

// get_permutation (preprocess/src/general/utilities.cpp:8-20): argsort of the grouping with
// libstdc++'s (unstable) std::sort and the reference's comparator, whose parameters are `int`.
int orc_get_permutation(int64_t n, const int64_t* grouping, int64_t* perm) {
    std::vector<int64_t> v((size_t)n);
    std::iota(v.begin(), v.end(), 0);
    auto comp = [&](int i, int j) { return grouping[i] < grouping[j]; };
    std::sort(v.begin(), v.end(), comp);
    memcpy(perm, v.data(), (size_t)n * sizeof(int64_t));
    return 0;
}

// get_fixed_size_grouping (preprocess/src/general/utilities.cpp:45-54), applied when -F 1
// (preprocess/src/general/blocking.cpp:651-654): result[perm[i]] = i / row_block_size.
int orc_fixed_size_grouping(int64_t n, const int64_t* grouping, int64_t row_block_size, int64_t* out) {
    std::vector<int64_t> perm((size_t)n);
    orc_get_permutation(n, grouping, perm.data());
    for (int64_t i = 0; i < n; i++) out[perm[(size_t)i]] = i / row_block_size;
    return 0;
}

// The whole reorder step as the Matrix_Blocking program performs it
// (preprocess/test/general/Matrix_Blocking.cpp:10-50 with -a 5 -F 1): Keeper grouping ->
// fixed-size grouping -> CSR::reorder (csr.cpp:97-105), whose permutation is the argsort of the
// FIXED-SIZE grouping; new row r is old row perm[r] (utilities.h:95-107).
int orc_reorder_rows(int64_t rows, const int64_t* rowptr, const int64_t* cols, float tau,
                     int64_t col_block_size, int64_t row_block_size, int64_t* grouping_fixed, int64_t* perm) {
    std::vector<int64_t> g((size_t)rows);
    orc_keeper_grouping(rows, rowptr, cols, tau, col_block_size, row_block_size, 1, g.data());
    orc_fixed_size_grouping(rows, g.data(), row_block_size, grouping_fixed);
    orc_get_permutation(rows, grouping_fixed, perm);
    return 0;
}

int orc_max_threads() {
    unsigned n = std::thread::hardware_concurrency();
    return n ? (int)n : 1;
}

}  // extern "C"
