// TEST INFRASTRUCTURE ONLY -- thin extern "C" doorway onto the UNMODIFIED reference CPU code.
//
// This file contains no algorithm of its own: it includes the reference's headers and is linked
// with the reference's own preprocess/src/general/*.cpp, compiled from where they lie (see
// oracle/Makefile, target `ref`).  The result, oracle/_ref/libsmat_ref.so, lets the test-suite call
// the real reference functions through ctypes to validate the restatement in smat_oracle.cpp, and
// lets the benchmark time the reference's CPU blocked multiply as the CPU baseline.
//
// Reference entry points used:
//   JaccardDistanceGroup / HammingDistanceGroup   preprocess/src/general/blocking.cpp:904-975, 701-760
//   BlockingEngine::GetGrouping (-a 5 -> Keeper)  preprocess/src/general/blocking.cpp:616-657, 431-547
//   get_permutation / get_fixed_size_grouping     preprocess/src/general/utilities.cpp:8-20, 45-54
//   CSR(ifstream) = read_from_edgelist            preprocess/src/general/csr.cpp:166-290
//   VBR::multiply                                 preprocess/src/general/vbr.cpp:323-372
//   VBR::fill_from_CSR_inplace (fixed-size blocks) preprocess/src/general/vbr.cpp:118-237

#include <cstdint>
#include <cstring>
#include <fstream>
#include <vector>

#include "blocking.h"
#include "definitions.h"
#include "matrices.h"
#include "utilities.h"

extern "C" {

float ref_jaccard_group(const long* rowA, long sizeA, long gA, long* rowB, long sizeB, long gB, long bs) {
    std::vector<intT> a(rowA, rowA + sizeA);
    return JaccardDistanceGroup(a, gA, rowB, sizeB, gB, bs);
}

float ref_hamming_group(const long* rowA, long sizeA, long gA, long* rowB, long sizeB, long gB, long bs) {
    std::vector<intT> a(rowA, rowA + sizeA);
    return HammingDistanceGroup(a, gA, rowB, sizeB, gB, bs);
}

// Reads an edge-list file with the reference reader, runs the reference grouping exactly as
// Matrix_Blocking does with "-a 5 -b cb -B rb -F force_fixed -t tau" and returns
// (rows, grouping, permutation-of-CSR::reorder).  Arrays must hold at least max_rows entries.
long ref_group_and_permute(const char* el_path, float tau, long cb, long rb, int force_fixed, long max_rows,
                           long* grouping_out, long* perm_out) {
    std::ifstream fin(el_path);
    if (!fin.good()) return -1;
    CSR cmat(fin, " ", true, el);
    BlockingEngine eng;
    eng.tau = tau;
    eng.col_block_size = cb;
    eng.row_block_size = rb;
    eng.use_groups = false;
    eng.use_pattern = true;
    eng.force_fixed_size = force_fixed != 0;
    eng.blocking_algo = iterative_max_size;
    eng.SetComparator(1);  // Jaccard, the CLI default (preprocess/include/input.h:29)
    std::vector<intT> g = eng.GetGrouping(cmat);
    long rows = (long)g.size();
    if (rows > max_rows) return -2;
    std::vector<intT> perm = get_permutation(g);
    for (long i = 0; i < rows; i++) { grouping_out[i] = g[i]; perm_out[i] = perm[i]; }
    return rows;
}

long ref_get_permutation(long n, const long* grouping, long* perm_out) {
    std::vector<intT> g(grouping, grouping + n);
    std::vector<intT> p = get_permutation(g);
    for (long i = 0; i < n; i++) perm_out[i] = p[i];
    return n;
}

long ref_fixed_size_grouping(long n, const long* grouping, long rb, long* out) {
    std::vector<intT> g(grouping, grouping + n);
    std::vector<intT> r = get_fixed_size_grouping(g, rb);
    for (long i = 0; i < n; i++) out[i] = r[i];
    return n;
}

// Runs VBR::multiply on caller-provided VBR arrays (fixed 16-row blocks): mab holds the blocks
// consecutively, COLUMN-major inside a block; jab holds block-column indices; B and C are
// column-major fp32 (B_rows = cols, C_rows = rows); C must be zeroed by the caller.
int ref_vbr_multiply(long rows, long cols, long block_rows, long block_col_size, const long* nzcount,
                     const long* jab, const float* mab, long nblocks, long row_block, float* B, int B_cols,
                     float* C) {
    VBR v;
    v.rows = rows;
    v.cols = cols;
    v.block_rows = block_rows;
    v.block_cols = (cols - 1) / block_col_size + 1;
    v.block_col_size = block_col_size;
    v.nzcount = new intT[block_rows];
    v.row_part = new intT[block_rows + 1];
    v.jab = new intT[nblocks > 0 ? nblocks : 1];
    v.nztot = nblocks * row_block * block_col_size;
    v.mab = new DataT[v.nztot > 0 ? v.nztot : 1];
    for (long i = 0; i < block_rows; i++) { v.nzcount[i] = nzcount[i]; v.row_part[i] = i * row_block; }
    v.row_part[block_rows] = rows;
    for (long i = 0; i < nblocks; i++) v.jab[i] = jab[i];
    memcpy(v.mab, mab, sizeof(DataT) * (size_t)v.nztot);
    v.multiply(B, B_cols, C);
    return 0;
}

// Blocks a CSR matrix (32-bit row pointers and columns, fp32 values, rows and cols as given) with the reference's
// VBR::fill_from_CSR_inplace(cmat, row_block, col_block, force_fixed_size = true) and copies out the structure
// (nzcount per block-row, block-column index per block) and the block values (column-major inside a block, rows of a
// block in the order of the reference's own get_permutation of the grouping i / row_block).  Returns the number of
// blocks, or -1 when max_blocks is too small.  The CSR object is laid out by hand: the reference's struct has no
// constructor from arrays, and its destructor must not run on memory it did not allocate.
long ref_vbr_from_csr(long rows, long cols, const int* rowptr, const int* colidx, const float* vals, long row_block,
                      long col_block, long max_blocks, long* nzcount_out, long* jab_out, float* mab_out) {
    CSR* c = static_cast<CSR*>(::operator new(sizeof(CSR)));
    c->rows = rows;
    c->cols = cols;
    c->pattern_only = false;
    c->nzcount = new intT[rows];
    c->ja = new intT*[rows];
    c->ma = new DataT*[rows];
    for (long r = 0; r < rows; r++) {
        const long n = rowptr[r + 1] - rowptr[r];
        c->nzcount[r] = n;
        c->ja[r] = new intT[n > 0 ? n : 1];
        c->ma[r] = new DataT[n > 0 ? n : 1];
        for (long j = 0; j < n; j++) {
            c->ja[r][j] = colidx[rowptr[r] + j];
            c->ma[r][j] = vals[rowptr[r] + j];
        }
    }
    VBR v;
    v.fill_from_CSR_inplace(*c, (intT)row_block, (intT)col_block, true);
    long nb = 0;
    for (long ib = 0; ib < v.block_rows; ib++) nb += v.nzcount[ib];
    long rc = nb;
    if (nb > max_blocks) {
        rc = -1;
    } else {
        for (long ib = 0; ib < v.block_rows; ib++) nzcount_out[ib] = v.nzcount[ib];
        for (long i = 0; i < nb; i++) jab_out[i] = v.jab[i];
        memcpy(mab_out, v.mab, sizeof(DataT) * (size_t)v.nztot);
    }
    for (long r = 0; r < rows; r++) { delete[] c->ja[r]; delete[] c->ma[r]; }
    delete[] c->nzcount;
    delete[] c->ja;
    delete[] c->ma;
    ::operator delete(c);
    return rc;
}

// VBR::fill_from_CSR_inplace(cmat, grouping, col_block) of the unmodified reference: the variable-height blocking
// (one block-row per group of the grouping, rows in the order of the reference's get_permutation).  Outputs: row_part
// (block_rows + 1 entries), nzcount, jab, mab (column-major blocks, floats).  Returns the number of blocks, -1 when a
// bound is too small; *block_rows_out and *nvals_out are set either way.
long ref_vbr_from_grouping(long rows, long cols, const int* rowptr, const int* colidx, const float* vals, const long* grouping,
                           long col_block, long max_block_rows, long max_blocks, long max_vals, long* block_rows_out,
                           long* row_part_out, long* nzcount_out, long* jab_out, long* nvals_out, float* mab_out) {
    CSR* c = static_cast<CSR*>(::operator new(sizeof(CSR)));
    c->rows = rows;
    c->cols = cols;
    c->pattern_only = false;
    c->nzcount = new intT[rows];
    c->ja = new intT*[rows];
    c->ma = new DataT*[rows];
    for (long r = 0; r < rows; r++) {
        const long n = rowptr[r + 1] - rowptr[r];
        c->nzcount[r] = n;
        c->ja[r] = new intT[n > 0 ? n : 1];
        c->ma[r] = new DataT[n > 0 ? n : 1];
        for (long j = 0; j < n; j++) {
            c->ja[r][j] = colidx[rowptr[r] + j];
            c->ma[r][j] = vals[rowptr[r] + j];
        }
    }
    std::vector<intT> g((size_t)rows);
    for (long r = 0; r < rows; r++) g[(size_t)r] = (intT)grouping[r];
    VBR v;
    v.fill_from_CSR_inplace(*c, g, (intT)col_block);
    long nb = 0;
    for (long ib = 0; ib < v.block_rows; ib++) nb += v.nzcount[ib];
    *block_rows_out = v.block_rows;
    *nvals_out = v.nztot;
    long rc = nb;
    if (v.block_rows > max_block_rows || nb > max_blocks || v.nztot > max_vals) {
        rc = -1;
    } else {
        for (long ib = 0; ib <= v.block_rows; ib++) row_part_out[ib] = v.row_part[ib];
        for (long ib = 0; ib < v.block_rows; ib++) nzcount_out[ib] = v.nzcount[ib];
        for (long i = 0; i < nb; i++) jab_out[i] = v.jab[i];
        memcpy(mab_out, v.mab, sizeof(DataT) * (size_t)v.nztot);
    }
    for (long r = 0; r < rows; r++) { delete[] c->ja[r]; delete[] c->ma[r]; }
    delete[] c->nzcount;
    delete[] c->ja;
    delete[] c->ma;
    ::operator delete(c);
    return rc;
}

}  // extern "C"
