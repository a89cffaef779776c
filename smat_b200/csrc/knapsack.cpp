// Gap-skipping 16x16 blocking of a CSR matrix on the host, block-rows in parallel.
//
// Replaces SparseMatrix::csrToBcsrKnapsacking (src/cuda_hgemm/src/common/matrix.h:504-671), the alternative to
// csrToBcsr that the reference keeps but does not call (matrix.h:174): inside a block-row of 16 rows the stored
// columns are visited in ascending order and a new 16-column block is opened at the first column the current block
// does not cover, so a block may start at any column and runs of empty columns between blocks cost nothing.  Where the
// columns still to come would leave a ragged last block, a block's start is moved left by up to the free room
// (matrix.h:551-570, 586-600).  Same results as the reference (row pointers, start columns, values); for duplicate
// (row, column) entries the reference's unstable sort decides which one survives, here it is the last in CSR order.
//
// The SpMM kernels of this library need block columns that are multiples of 16 (a TMA box starts on a 16-byte
// boundary), so they do not take this format; smat_knapsack_to_csr turns it back into CSR.  What the packing is for
// -- fewer nonzero blocks on scattered rows -- the column reorder achieves with aligned blocks.
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <thread>
#include <vector>

#include "smat_internal.h"

using namespace smat;

namespace {

struct Entry {
    int col, row;
    uint16_t val;
};

// Start column of a block opened at `col` when `add_left` columns are free to its left (matrix.h:551-570, 586-600).
inline long place_block(long col, long last, long add_left, long add_right) {
    const long span = last - col + 1;
    const long to_add = 16 - span % 16;
    if (span % 16 == 0 || add_right >= to_add) return col;
    if (add_left >= to_add) return col - to_add;
    return col - add_left;
}

// Blocks of one block-row: start columns appended to `starts`, values (row-major 16x16 fp16 bit patterns) to `vals`.
void pack_block_row(size_t K, const int* rowptr, const int* colidx, const uint16_t* csr_vals, size_t brow, std::vector<Entry>& tmp,
                    std::vector<int>& starts, std::vector<uint16_t>& vals) {
    tmp.clear();
    for (size_t r = brow * 16; r < brow * 16 + 16; r++)
        for (int j = rowptr[r]; j < rowptr[r + 1]; j++) tmp.push_back({colidx[j], (int)(r % 16), csr_vals[j]});
    if (tmp.empty()) return;
    std::stable_sort(tmp.begin(), tmp.end(), [](const Entry& a, const Entry& b) { return a.col < b.col; });
    const long first = tmp.front().col, last = tmp.back().col;
    const long add_right = (long)K - last - 1;
    long start = place_block(first, last, first, add_right);
    long end = start + 16;
    starts.push_back((int)start);
    vals.resize(vals.size() + 256, 0);
    for (const Entry& e : tmp) {
        if (e.col >= end) {
            start = place_block(e.col, last, e.col - end, add_right);
            end = start + 16;
            starts.push_back((int)start);
            vals.resize(vals.size() + 256, 0);
        }
        vals[vals.size() - 256 + (size_t)e.row * 16 + (size_t)(e.col - start)] = e.val;
    }
}

}  // namespace

extern "C" {

int smat_bcsr_knapsack(const int* csr_rowptr, const int* csr_colidx, const uint16_t* csr_vals, size_t M, size_t K, int threads,
                       size_t* nnzb_out, int** bcsr_rowptr, int** bcsr_colidx, uint16_t** bcsr_vals) {
    clear_error();
    if (M % 16) return fail(SMAT_ERR_BAD_ARG, "M (%zu) must be a multiple of 16", M);
    if (!csr_rowptr || !nnzb_out || !bcsr_rowptr || !bcsr_colidx || !bcsr_vals) return fail(SMAT_ERR_BAD_ARG, "NULL argument");
    const size_t Mb = M / 16;
    if (csr_rowptr[M] > 0 && (!csr_colidx || !csr_vals)) return fail(SMAT_ERR_BAD_ARG, "NULL argument");
    for (size_t r = 0; r < M; r++)
        if (csr_rowptr[r + 1] < csr_rowptr[r]) return fail(SMAT_ERR_BAD_ARG, "row pointers must not decrease (row %zu)", r);
    for (int j = 0; j < csr_rowptr[M]; j++)
        if (csr_colidx[j] < 0 || (size_t)csr_colidx[j] >= K) return fail(SMAT_ERR_RANGE, "column %d outside [0, %zu)", csr_colidx[j], K);
    if (threads <= 0) threads = (int)std::thread::hardware_concurrency();
    if (threads < 1) threads = 1;
    if ((size_t)threads > Mb) threads = Mb ? (int)Mb : 1;
    // contiguous ranges of block-rows per thread, each packed into its own vectors, then concatenated in order
    std::vector<std::vector<int>> t_starts((size_t)threads), t_counts((size_t)threads);
    std::vector<std::vector<uint16_t>> t_vals((size_t)threads);
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; t++) {
        pool.emplace_back([&, t]() {
            std::vector<Entry> tmp;
            const size_t b0 = Mb * (size_t)t / (size_t)threads, b1 = Mb * (size_t)(t + 1) / (size_t)threads;
            for (size_t b = b0; b < b1; b++) {
                const size_t before = t_starts[(size_t)t].size();
                pack_block_row(K, csr_rowptr, csr_colidx, csr_vals, b, tmp, t_starts[(size_t)t], t_vals[(size_t)t]);
                t_counts[(size_t)t].push_back((int)(t_starts[(size_t)t].size() - before));
            }
        });
    }
    for (auto& th : pool) th.join();
    size_t nnzb = 0;
    for (auto& v : t_starts) nnzb += v.size();
    if (nnzb >= ((size_t)1 << 31)) return fail(SMAT_ERR_RANGE, "more than 2^31 - 1 blocks");
    int* rp = (int*)malloc((Mb + 1) * sizeof(int));
    int* ci = (int*)malloc((nnzb ? nnzb : 1) * sizeof(int));
    uint16_t* bv = (uint16_t*)malloc((nnzb ? nnzb : 1) * 256 * sizeof(uint16_t));
    if (!rp || !ci || !bv) {
        free(rp);
        free(ci);
        free(bv);
        return fail(SMAT_ERR_NOMEM, "out of host memory");
    }
    size_t at = 0, brow = 0;
    for (int t = 0; t < threads; t++) {
        for (int c : t_counts[(size_t)t]) {
            rp[brow++] = (int)at;
            at += (size_t)c;
        }
    }
    rp[Mb] = (int)nnzb;
    at = 0;
    for (int t = 0; t < threads; t++) {
        const size_t n = t_starts[(size_t)t].size();
        if (n) {
            memcpy(ci + at, t_starts[(size_t)t].data(), n * sizeof(int));
            memcpy(bv + at * 256, t_vals[(size_t)t].data(), n * 256 * sizeof(uint16_t));
        }
        at += n;
    }
    *nnzb_out = nnzb;
    *bcsr_rowptr = rp;
    *bcsr_colidx = ci;
    *bcsr_vals = bv;
    return SMAT_OK;
}

int smat_knapsack_to_csr(const int* bcsr_rowptr, const int* bcsr_colidx, const uint16_t* bcsr_vals, size_t M, size_t K,
                         size_t* nnz_out, int** csr_rowptr, int** csr_colidx, uint16_t** csr_vals) {
    clear_error();
    if (M % 16 || !bcsr_rowptr || !nnz_out || !csr_rowptr || !csr_colidx || !csr_vals) return fail(SMAT_ERR_BAD_ARG, "bad argument");
    const size_t Mb = M / 16;
    const size_t nnzb = (size_t)bcsr_rowptr[Mb];
    // entries whose value is zero are padding of a block (a stored zero of the original matrix is not told apart)
    std::vector<int> count(M + 1, 0);
    for (size_t b = 0; b < Mb; b++)
        for (int p = bcsr_rowptr[b]; p < bcsr_rowptr[b + 1]; p++)
            for (int i = 0; i < 256; i++)
                if (bcsr_vals[(size_t)p * 256 + i] & 0x7fffu) {
                    const long c = (long)bcsr_colidx[p] + i % 16;
                    if (c < 0 || (size_t)c >= K) return fail(SMAT_ERR_RANGE, "block %d reaches column %ld outside [0, %zu)", p, c, K);
                    count[b * 16 + (size_t)(i / 16) + 1]++;
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
    for (size_t b = 0; b < Mb; b++)
        for (int p = bcsr_rowptr[b]; p < bcsr_rowptr[b + 1]; p++)  // blocks of a block-row ascend and do not overlap: columns stay sorted
            for (int i = 0; i < 256; i++)
                if (bcsr_vals[(size_t)p * 256 + i] & 0x7fffu) {
                    const size_t r = b * 16 + (size_t)(i / 16);
                    ci[cur[r]] = bcsr_colidx[p] + i % 16;
                    v[cur[r]++] = bcsr_vals[(size_t)p * 256 + i];
                }
    (void)nnzb;
    *nnz_out = nnz;
    *csr_rowptr = rp;
    *csr_colidx = ci;
    *csr_vals = v;
    return SMAT_OK;
}

}  // extern "C"
