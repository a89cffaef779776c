// Variable-height blocked format (VBR) of a CSR matrix from a row grouping, on the host.
//
// Replaces VBR::fill_from_CSR_inplace(cmat, grouping, col_block_size) (preprocess/src/general/vbr.cpp:135-237) with
// get_permutation / get_partition (preprocess/src/general/utilities.cpp:8-43): the rows are brought into the order of
// an argsort of their group numbers, every group becomes one block-row of as many rows as the group has, and a block
// (block-row x col_block columns) is stored iff one of its rows has a stored entry in those columns.  Same arrays as
// the reference: row_part (first row of each block-row in the permuted order, then the row count), nzcount (blocks per
// block-row), jab (block-column of each block, ascending inside a block-row), mab (the blocks one after the other,
// each column-major: entry (row r of the block-row, column c of the block) at c * height + r).  Values are fp16 bit
// patterns here (the reference holds floats).  The argsort is libstdc++'s unstable std::sort with the reference's
// comparator, so rows of one group come out in the reference's order.
//
// The SpMM kernels of this library work on 16-row block-rows (what the reference's pipeline produces with -F 1); this
// format is built for callers that want the reference's other blocking, and smat_vbr_to_csr turns it back.
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <numeric>
#include <vector>

#include "smat_internal.h"

#ifndef __GLIBCXX__
#error "the order of equal keys must be libstdc++'s std::sort order (the reference is built with it)"
#endif

using namespace smat;

extern "C" {

int smat_vbr_from_csr(const int* csr_rowptr, const int* csr_colidx, const uint16_t* csr_vals, size_t M, size_t K,
                      const int64_t* grouping, size_t col_block, size_t* block_rows_out, int64_t** row_part_out,
                      int64_t** row_perm_out, int64_t** nzcount_out, size_t* nblocks_out, int64_t** jab_out, size_t* nvals_out,
                      uint16_t** mab_out) {
    clear_error();
    if (!csr_rowptr || !grouping || !block_rows_out || !row_part_out || !row_perm_out || !nzcount_out || !nblocks_out || !jab_out ||
        !nvals_out || !mab_out)
        return fail(SMAT_ERR_BAD_ARG, "NULL argument");
    if (M == 0 || K == 0 || col_block == 0) return fail(SMAT_ERR_BAD_ARG, "empty matrix or zero block width");
    if (M >= ((size_t)1 << 31) || K >= ((size_t)1 << 31)) return fail(SMAT_ERR_RANGE, "size beyond 2^31");
    if (csr_rowptr[M] > 0 && (!csr_colidx || !csr_vals)) return fail(SMAT_ERR_BAD_ARG, "NULL argument");
    for (size_t r = 0; r < M; r++)
        if (csr_rowptr[r + 1] < csr_rowptr[r]) return fail(SMAT_ERR_BAD_ARG, "row pointers must not decrease (row %zu)", r);
    for (int j = 0; j < csr_rowptr[M]; j++)
        if (csr_colidx[j] < 0 || (size_t)csr_colidx[j] >= K) return fail(SMAT_ERR_RANGE, "column %d outside [0, %zu)", csr_colidx[j], K);

    // get_permutation: argsort of the group numbers (unstable sort, int comparator arguments as in the reference)
    std::vector<int64_t> perm(M);
    std::iota(perm.begin(), perm.end(), 0);
    auto comp = [&](int a, int b) { return grouping[(size_t)a] < grouping[(size_t)b]; };
    std::sort(perm.begin(), perm.end(), comp);
    // get_partition: a new block-row wherever the sorted group number changes.  Group numbers may be negative (the
    // clustering marks full groups that way); the reference starts its scan from "group -1", so a smallest group
    // numbered exactly -1 would not open a block-row there: rejected here.
    if (grouping[(size_t)perm[0]] == -1) return fail(SMAT_ERR_BAD_ARG, "the smallest group number must not be -1");
    std::vector<int64_t> part;
    int64_t current = -1;
    for (size_t i = 0; i < M; i++) {
        const int64_t g = grouping[(size_t)perm[i]];
        if (g != current) {
            current = g;
            part.push_back((int64_t)i);
        }
    }
    part.push_back((int64_t)M);
    const size_t block_rows = part.size() - 1, block_cols = (K - 1) / col_block + 1;

    std::vector<int64_t> nzcount(block_rows, 0), jab;
    std::vector<uint16_t> mab;
    std::vector<int64_t> slot(block_cols);  // position of a block-column among the block-row's blocks, or -1
    for (size_t ib = 0; ib < block_rows; ib++) {
        const size_t h = (size_t)(part[ib + 1] - part[ib]);
        std::fill(slot.begin(), slot.end(), -1);
        for (int64_t ir = part[ib]; ir < part[ib + 1]; ir++) {
            const size_t i = (size_t)perm[(size_t)ir];
            for (int j = csr_rowptr[i]; j < csr_rowptr[i + 1]; j++) slot[(size_t)csr_colidx[j] / col_block] = 0;
        }
        int64_t n = 0;
        for (size_t jb = 0; jb < block_cols; jb++)
            if (slot[jb] == 0) {
                slot[jb] = n++;
                jab.push_back((int64_t)jb);
            }
        nzcount[ib] = n;
        const size_t base = mab.size();
        if ((base + (size_t)n * h * col_block) / 2 >= ((size_t)1 << 40)) return fail(SMAT_ERR_RANGE, "blocked values beyond 2^41 bytes");
        mab.resize(base + (size_t)n * h * col_block, 0);
        for (int64_t ir = part[ib]; ir < part[ib + 1]; ir++) {
            const size_t i = (size_t)perm[(size_t)ir];
            for (int j = csr_rowptr[i]; j < csr_rowptr[i + 1]; j++) {
                const size_t c = (size_t)csr_colidx[j];
                // a later duplicate of (row, column) overwrites an earlier one, as in the reference
                mab[base + (size_t)slot[c / col_block] * h * col_block + h * (c % col_block) + (size_t)(ir - part[ib])] = csr_vals[j];
            }
        }
    }

    int64_t* rp = (int64_t*)malloc((block_rows + 1) * sizeof(int64_t));
    int64_t* pm = (int64_t*)malloc(M * sizeof(int64_t));
    int64_t* nz = (int64_t*)malloc((block_rows ? block_rows : 1) * sizeof(int64_t));
    int64_t* jb = (int64_t*)malloc((jab.empty() ? 1 : jab.size()) * sizeof(int64_t));
    uint16_t* mv = (uint16_t*)malloc((mab.empty() ? 1 : mab.size()) * sizeof(uint16_t));
    if (!rp || !pm || !nz || !jb || !mv) {
        free(rp);
        free(pm);
        free(nz);
        free(jb);
        free(mv);
        return fail(SMAT_ERR_NOMEM, "out of host memory");
    }
    memcpy(rp, part.data(), (block_rows + 1) * sizeof(int64_t));
    memcpy(pm, perm.data(), M * sizeof(int64_t));
    if (block_rows) memcpy(nz, nzcount.data(), block_rows * sizeof(int64_t));
    if (!jab.empty()) memcpy(jb, jab.data(), jab.size() * sizeof(int64_t));
    if (!mab.empty()) memcpy(mv, mab.data(), mab.size() * sizeof(uint16_t));
    *block_rows_out = block_rows;
    *row_part_out = rp;
    *row_perm_out = pm;
    *nzcount_out = nz;
    *nblocks_out = jab.size();
    *jab_out = jb;
    *nvals_out = mab.size();
    *mab_out = mv;
    return SMAT_OK;
}

int smat_vbr_to_csr(size_t M, size_t K, size_t col_block, size_t block_rows, const int64_t* row_part, const int64_t* row_perm,
                    const int64_t* nzcount, const int64_t* jab, const uint16_t* mab, size_t* nnz_out, int** csr_rowptr,
                    int** csr_colidx, uint16_t** csr_vals) {
    clear_error();
    if (!row_part || !row_perm || !nzcount || !nnz_out || !csr_rowptr || !csr_colidx || !csr_vals || col_block == 0)
        return fail(SMAT_ERR_BAD_ARG, "bad argument");
    // entries whose value is zero are padding of a block (a stored zero of the original matrix is not told apart)
    std::vector<int> count(M + 1, 0);
    size_t blk = 0, at = 0;
    for (size_t ib = 0; ib < block_rows; ib++) {
        const size_t h = (size_t)(row_part[ib + 1] - row_part[ib]);
        for (int64_t b = 0; b < nzcount[ib]; b++, blk++, at += h * col_block) {
            if (!jab || !mab) return fail(SMAT_ERR_BAD_ARG, "NULL argument");
            for (size_t c = 0; c < col_block; c++)
                for (size_t r = 0; r < h; r++)
                    if (mab[at + c * h + r] & 0x7fffu) {
                        const size_t col = (size_t)jab[blk] * col_block + c;
                        const int64_t row = row_perm[(size_t)row_part[ib] + r];
                        if (col >= K || row < 0 || (size_t)row >= M) return fail(SMAT_ERR_RANGE, "block %zu reaches outside the matrix", blk);
                        count[(size_t)row + 1]++;
                    }
        }
    }
    for (size_t r = 0; r < M; r++) count[r + 1] += count[r];
    const size_t nnz = (size_t)count[M];
    int* rp = (int*)malloc((M + 1) * sizeof(int));
    int* ci = (int*)malloc((nnz ? nnz : 1) * sizeof(int));
    uint16_t* v = (uint16_t*)malloc((nnz ? nnz : 1) * sizeof(uint16_t));
    if (!rp || !ci || !v) {
        free(rp);
        free(ci);
        free(v);
        return fail(SMAT_ERR_NOMEM, "out of host memory");
    }
    memcpy(rp, count.data(), (M + 1) * sizeof(int));
    std::vector<int> cur(count.begin(), count.end() - 1);
    blk = 0;
    at = 0;
    for (size_t ib = 0; ib < block_rows; ib++) {
        const size_t h = (size_t)(row_part[ib + 1] - row_part[ib]);
        for (int64_t b = 0; b < nzcount[ib]; b++, blk++, at += h * col_block)  // blocks of a block-row ascend: columns stay sorted
            for (size_t c = 0; c < col_block; c++)
                for (size_t r = 0; r < h; r++)
                    if (mab[at + c * h + r] & 0x7fffu) {
                        const size_t row = (size_t)row_perm[(size_t)row_part[ib] + r];
                        ci[cur[row]] = (int)((size_t)jab[blk] * col_block + c);
                        v[cur[row]++] = mab[at + c * h + r];
                    }
    }
    *nnz_out = nnz;
    *csr_rowptr = rp;
    *csr_colidx = ci;
    *csr_vals = v;
    return SMAT_OK;
}

}  // extern "C"
