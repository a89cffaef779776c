/* smat_b200 -- C ABI of the B200-native block-sparse SpMM engine.
 *
 * Drop-in boundary for the SpMM path of SMaT: every entry point below replaces one piece of the
 * reference's host/GPU code and keeps its argument meaning and memory layouts.  Plain pointers and
 * sizes only; `stream` is a cudaStream_t passed as void* (NULL = default stream).  All functions
 * return 0 on success or a negative smat_status code; none of them exits the process (the reference
 * calls exit() on error, src/cuda_hgemm/src/common/common.h:21-63).
 *
 * Layouts (identical to the reference kernels, src/cuda_hgemm/src/mma/mmaCBT.cu:13-88):
 *   vals     fp16, block p occupies [p*256, p*256+256), row-major 16x16
 *   rowptr   int32[M/16 + 1]
 *   colidx   int32[nnzb], ELEMENT column of the block's left edge (multiple of 16), ascending per row
 *   B        fp16, logical K x N, element (k, n) at B[n*K + k]   (K contiguous)
 *   C        fp16, row-major M x N, fully overwritten
 * M and K are multiples of 16, N a multiple of 8, device pointers 16-byte aligned.
 */
#ifndef SMAT_B200_H
#define SMAT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum smat_status {
    SMAT_OK = 0,
    SMAT_ERR_BAD_ARG = -1,      /* null pointer, misaligned pointer, size not a multiple of the tile */
    SMAT_ERR_CUDA = -2,         /* a CUDA runtime / driver call failed; see smat_last_error_string() */
    SMAT_ERR_DEVICE_WAIT = -3,  /* a bounded wait inside a kernel ran out (device status word set) */
    SMAT_ERR_IO = -4,           /* file could not be opened / parsed */
    SMAT_ERR_NOMEM = -5,
    SMAT_ERR_RANGE = -6         /* index out of range / size beyond a stated limit */
} smat_status;

/* C = A_bcsr x B on the current device, asynchronous on `stream`.
 * Replaces  void mmaCBTKernel(half*, int*, int*, half*, half*, size_t M, size_t N, size_t K,
 *                             size_t nonzeroBlocks, int* blockInfo, int* relativeBlockIndexMapping)
 * (src/cuda_hgemm/src/mma/mmaCBT.cu:83-88; declared through HGEMM_FUNC_SPARSE2,
 * src/cuda_hgemm/src/main.cu:7,19).  Same argument order; blockInfo and relativeBlockIndexMapping
 * are accepted for signature compatibility and ignored (may be NULL): the dense Mb*Kb maps are
 * redundant with rowptr/colidx. */
int smat_spmm_bcsr_f16(const void* bcsrValuesA, const int* bcsrRowPtrA, const int* bcsrColIdxA, const void* B, void* C,
                       size_t M, size_t N, size_t K, size_t nonzeroBlocks, const int* blockInfo,
                       const int* relativeBlockIndexMapping, void* stream);

/* Same product restricted to block-rows [brow_begin, brow_end): writes rows
 * [16*brow_begin, 16*brow_end) of C, where C points at the FIRST row of that range (the shard's own
 * C buffer).  This is the per-GPU unit of the block-row partitioning; the reference is single-GPU
 * (src/cuda_hgemm/src/main.cu:32,41 only selects a device), so there is no reference counterpart
 * beyond mmaCBTKernel itself.  rowptr/colidx/vals are the full matrix arrays or a shard of them:
 * only rowptr[brow_begin..brow_end] is read and its values index colidx/vals directly. */
int smat_spmm_bcsr_f16_rows(const void* bcsrValuesA, const int* bcsrRowPtrA, const int* bcsrColIdxA, const void* B,
                            void* C, size_t M, size_t N, size_t K, size_t nonzeroBlocks, size_t brow_begin,
                            size_t brow_end, void* stream);

/* Same product as smat_spmm_bcsr_f16 for callers that may not allocate device memory (fixed-budget
 * serving loops, callbacks that run while the allocator is locked, processes that gave their free
 * memory to a foreign pool): the per-call plan is built in a fixed array inside the library image
 * instead of freshly allocated scratch, so the call performs no allocation and no free.
 * No counterpart in the reference (its launcher needs no scratch, mmaCBT.cu:83-88).
 * Limits: nonzeroBlocks <= SMAT_STATIC_MAX_BLOCKS and M <= SMAT_STATIC_MAX_ROWS, else SMAT_ERR_RANGE;
 * the array (17.5 MB) stays resident on every GPU that loads the library.
 * All calls on a device share the array: calls that overlap on the GPU race; calls on one stream do
 * not.  The first call on a device also looks up the array's device address -- make it before
 * starting a stream capture.  Device-side errors (a bounded wait that ran out, row pointers that
 * disagree with nonzeroBlocks) are recorded in a word of the array that stays set until
 * smat_device_status reports and clears it. */
#define SMAT_STATIC_MAX_BLOCKS 32768
#define SMAT_STATIC_MAX_ROWS 1048576
int smat_spmm_bcsr_f16_static(const void* bcsrValuesA, const int* bcsrRowPtrA, const int* bcsrColIdxA, const void* B,
                              void* C, size_t M, size_t N, size_t K, size_t nonzeroBlocks, void* stream);


/* Multiplication plan: what the kernel needs beyond the BCSR arrays, computed on the device and
 * reusable for any number of multiplications:
 *   - the walk order (per group of up to 16 block-rows, its block-columns four at a time in ascending
 *     order with the blocks found there), and
 *   - a copy of the value blocks in that order, so that all blocks of a step arrive with one bulk
 *     copy (nonzeroBlocks * 512 bytes of device memory owned by the plan).
 * smat_spmm_bcsr_f16 builds all of this internally on every call (in stream-ordered scratch
 * memory); a caller that multiplies repeatedly, like the reference harness with its warm-up and
 * 10 timed launches (src/cuda_hgemm/src/common/tester.h:177-183, 344-347), creates it once instead.
 * The plan covers block-rows [brow_begin, brow_end) and keeps the rowptr pointer it was given (not
 * owned).  After the values of A changed (same structure) call smat_plan_set_values.
 * No counterpart in the reference (its kernel re-reads bcsrColIdx per tile, mmaCBT.cu:38-43). */
typedef struct smat_plan smat_plan;
/* N_hint: the number of columns of B the plan will mostly be used with (0 = unknown).  It only steers
 * how many block-rows form a work item (8 to 24) and which of the two kernels multiplies, so that small matrices or
 * shards still fill the SMs.
 * A plan also owns scratch for work items that a launch computes in segments (38.8 MB on a 148-SM device, twice
 * that for matrices whose work is very unevenly spread over the block-rows) and may be used by one stream at a
 * time. */
int smat_plan_create(smat_plan** plan, const void* bcsrValuesA, const int* bcsrRowPtrA, const int* bcsrColIdxA, size_t M,
                     size_t K, size_t nonzeroBlocks, size_t brow_begin, size_t brow_end, size_t N_hint, void* stream);
int smat_plan_set_values(smat_plan* plan, const void* bcsrValuesA, void* stream);
/* Rows [16*brow_begin, 16*brow_end) of C = A x B; C points at the first row of that range. */
int smat_plan_spmm(const smat_plan* plan, const void* B, void* C, size_t N, void* stream);

/* The same product with B and C in HOST memory (pinned memory for copies that overlap), pipelined on two
 * internal streams: B comes in by column chunks of one work-item width, each multiplied as soon as it has
 * arrived; the last chunk is multiplied range of block-rows by range, and the rows of C it completes are copied
 * out under the multiplication of the next range.  B_host is [N][K] (k contiguous), C_host row-major
 * [(brow_end - brow_begin) * 16][N].  Everything is ordered after earlier work on `stream`, and `stream` ends
 * after the last copy.  The staging buffers (all of B and C) and the streams belong to the plan and are created
 * by the first call, which therefore must not happen inside a stream capture.
 * No reference counterpart: the reference harness uploads B once and downloads C once
 * (src/cuda_hgemm/src/common/matrix.h:88-101). */
int smat_plan_spmm_host(smat_plan* plan, const void* B_host, void* C_host, size_t N, void* stream);
int smat_plan_destroy(smat_plan* plan);
/* What a plan turned out to be (informational, no reference counterpart): *rows_per_item = block-rows of a work item
 * (8..16: the kernel that reads both operands from shared memory; 16..24 with *tall = 1: the kernel that reads the
 * B panels from tensor memory), *steps = steps of the walk order.  Any pointer may be NULL. */
int smat_plan_info(const smat_plan* plan, int* tall, int* rows_per_item, size_t* steps);

/* Kernel variant used by every multiplication of this process: 0 = chosen per matrix (default),
 * 1 = both MMA operands from shared memory (two accumulator buffers, epilogue overlapped),
 * 2 = B panels copied to tensor memory and read from there (one accumulator buffer),
 * 3 = work items 256 columns of C wide: two MMAs per block, one accumulator buffer (default for N >= 256),
 * 4 = plans created from now on use work items of up to 24 block-rows and the kernel that reads the B panels
 *     from tensor memory (affects smat_plan_create, not plans that exist).
 * Meant for benchmarks and tests; no counterpart in the reference. */
int smat_spmm_set_variant(int variant);

/* Synchronises `stream` and reports whether any kernel launched by this library on the current
 * device recorded a device-side error: a bounded wait that ran out (SMAT_ERR_DEVICE_WAIT), or BCSR
 * arrays found inconsistent while a plan was built -- row pointers that are not monotone or exceed
 * nonzeroBlocks, a block column outside the matrix or out of order (SMAT_ERR_RANGE; such input gets
 * an empty or partial plan instead of an out-of-bounds write).  Clears the device status words (the
 * allocating entry points' and the static entry point's).
 * The reference never checks its launches (src/cuda_hgemm/src/mma/mmaCBT.cu:87). */
int smat_device_status(void* stream);

/* Self-test of the error path above: launches a one-thread kernel that waits, with the SpMM kernels' own bounded
 * wait and a limit of about 0.2 ms, on a barrier that nothing completes.  The kernel ends by itself with the device
 * status word set (site code 90); the next smat_device_status on the device returns SMAT_ERR_DEVICE_WAIT and clears
 * it.  Nothing faults and the context stays usable.  No counterpart in the reference. */
int smat_selftest_wait_timeout(void* stream);

/* Number of this library's kernels launched so far by the calling process (all devices). */
long long smat_launch_count(void);

/* Device-side BCSR builder: CSR (device arrays, int32 indices, fp16 values, M and K multiples of 16,
 * any column order inside a row; duplicate (row, col) entries allowed, the last one in CSR order
 * wins) -> 16x16 BCSR in the layout above.
 * Replaces SparseMatrix::csrToBcsr and the host-to-device uploads of its result
 * (src/cuda_hgemm/src/common/matrix.h:376-502, 185-199); the dense Mb*Kb maps blockInfo and
 * relativeBlockIndexMapping are never built.
 * Two-phase: smat_bcsr_count writes bcsr_rowptr (device, int32[M/16+1]) and returns nnzb to the
 * host (synchronises the stream); the caller allocates colidx (int32[nnzb]) and vals
 * (fp16[nnzb*256]) and calls smat_bcsr_fill, which is asynchronous on `stream`.
 * Limit: K <= 12,582,912 (one block-row's column-block bitmap is kept in shared memory). */
int smat_bcsr_count(const int* csr_rowptr, const int* csr_colidx, size_t M, size_t K, size_t nnz, int* bcsr_rowptr,
                    size_t* nnzb_out, void* stream);
int smat_bcsr_fill(const int* csr_rowptr, const int* csr_colidx, const void* csr_vals, size_t M, size_t K, size_t nnz,
                   const int* bcsr_rowptr, int* bcsr_colidx, void* bcsr_vals, size_t nnzb, void* stream);

/* Gap-skipping blocking (host, block-rows in parallel).  Replaces SparseMatrix::csrToBcsrKnapsacking
 * (src/cuda_hgemm/src/common/matrix.h:504-671), the alternative to csrToBcsr that the reference keeps without calling it
 * (matrix.h:174): blocks are 16 rows x 16 columns but may START AT ANY COLUMN, a new block being opened at the first
 * stored column the current one does not cover.  Input: host CSR (fp16 bit patterns), M a multiple of 16.  Output
 * arrays are malloc'ed (release with smat_free_host): bcsr_rowptr int32[M/16+1], bcsr_colidx int32[nnzb] = start
 * column of every block, bcsr_vals row-major 16x16 blocks.  threads <= 0 uses every hardware thread.
 * The SpMM entry points above take 16-aligned block columns only; smat_knapsack_to_csr converts back (entries that
 * are zero inside a block are dropped). */
int smat_bcsr_knapsack(const int* csr_rowptr, const int* csr_colidx, const uint16_t* csr_vals, size_t M, size_t K, int threads,
                       size_t* nnzb, int** bcsr_rowptr, int** bcsr_colidx, uint16_t** bcsr_vals);
int smat_knapsack_to_csr(const int* bcsr_rowptr, const int* bcsr_colidx, const uint16_t* bcsr_vals, size_t M, size_t K,
                         size_t* nnz, int** csr_rowptr, int** csr_colidx, uint16_t** csr_vals);

/* Variable-height blocking (host).  Replaces VBR::fill_from_CSR_inplace(cmat, grouping, col_block_size)
 * (preprocess/src/general/vbr.cpp:135-237, with get_permutation / get_partition, utilities.cpp:8-43), the blocked format
 * of the reference's preprocessing library when a grouping of unequal groups is kept as it is (its pipeline for the
 * kernels above passes -F 1 and gets 16-row groups): rows are taken in the order of an argsort of `grouping` (int64 per
 * row; negative numbers allowed, the smallest must not be -1), each group becomes a block-row of its own height, and
 * a block of that height x col_block columns is stored where any of its rows has a stored entry.  Output arrays are
 * malloc'ed (release with smat_free_host) and laid out as the reference's: row_part int64[block_rows + 1], row_perm
 * int64[M] (permuted position -> original row), nzcount int64[block_rows], jab int64[nblocks] (block-columns,
 * ascending inside a block-row), mab fp16 bit patterns, block after block, each column-major (height contiguous).
 * The SpMM entry points above take 16-row blocks only; smat_vbr_to_csr converts back (entries that are zero inside a
 * block are dropped). */
int smat_vbr_from_csr(const int* csr_rowptr, const int* csr_colidx, const uint16_t* csr_vals, size_t M, size_t K,
                      const int64_t* grouping, size_t col_block, size_t* block_rows, int64_t** row_part, int64_t** row_perm,
                      int64_t** nzcount, size_t* nblocks, int64_t** jab, size_t* nvals, uint16_t** mab);
int smat_vbr_to_csr(size_t M, size_t K, size_t col_block, size_t block_rows, const int64_t* row_part, const int64_t* row_perm,
                    const int64_t* nzcount, const int64_t* jab, const uint16_t* mab, size_t* nnz, int** csr_rowptr,
                    int** csr_colidx, uint16_t** csr_vals);

/* Matrix-Market reader (host).  Replaces mmio_allinone
 * (src/cuda_hgemm/src/common/mmio_highlevel.h:619-786): dimensions padded up to multiples of 16,
 * 0-based CSR in file order inside each row, symmetric/hermitian files mirrored, pattern files get
 * value 1, values rounded double -> fp16 once.  Output arrays are malloc'ed by the library and
 * released with smat_free_host.  `vals` receives fp16 bit patterns. */
int smat_read_mtx(const char* filename, size_t* M, size_t* K, size_t* nnz, int* is_symmetric, int** csr_rowptr,
                  int** csr_colidx, uint16_t** csr_vals);
void smat_free_host(void* p);

/* Similarity-based row reordering (host, multi-threaded).  Replaces the Matrix_Blocking program run
 * as `-a 5 -b col_block -B row_block -F 1 -t tau`
 * (preprocess/test/general/Matrix_Blocking.cpp:10-50 -> BlockingEngine::GetGrouping,
 * preprocess/src/general/blocking.cpp:616-657 -> IterativeBlockingKeeper :431-547 with
 * JaccardDistanceGroup :904-975, merge_rows preprocess/src/general/utilities.cpp:145-173,
 * get_fixed_size_grouping / get_permutation utilities.cpp:45-54, 8-20, CSR::reorder csr.cpp:97-105).
 * Input: CSR pattern with ASCENDING columns in every row (64-bit row pointers, 32-bit columns).
 * Output: grouping[rows] (the fixed-size grouping the program writes to its .g file) and
 * perm[rows] with "new row r = old row perm[r]".  Bit-identical to the reference program.
 * threads <= 0 uses every hardware thread. */
int smat_reorder_rows(size_t rows, const int64_t* rowptr, const int32_t* cols, float tau, int col_block,
                      int row_block, int threads, int64_t* grouping, int64_t* perm);
/* The same clustering without the fixed-size regrouping (the program run without -F 1): grouping[rows] as
 * BlockingEngine::GetGrouping returns it -- groups of at most max_group_rows rows, numbered by their seed row, full
 * groups lowered by the row count -- and, if perm is not NULL, get_permutation of it.  With smat_vbr_from_csr this is
 * the reference's variable-height blocking of a matrix. */
int smat_cluster_rows(size_t rows, const int64_t* rowptr, const int32_t* cols, float tau, int col_block, int max_group_rows,
                      int threads, int64_t* grouping, int64_t* perm);

/* Jaccard distance on column-block quotients between a group pattern and a row
 * (JaccardDistanceGroup, preprocess/src/general/blocking.cpp:904-975). */
float smat_jaccard_group(const int64_t* rowA, size_t sizeA, int64_t groupA, const int64_t* rowB, size_t sizeB,
                         int64_t groupB, int64_t block_size);

/* nnzb-balanced contiguous block-row ranges for `parts` GPUs: bounds[parts+1], bounds[0] = 0,
 * bounds[parts] = Mb; chosen on the prefix sums in bcsr_rowptr (host array) so that every part holds
 * about nnzb/parts blocks.  New work: the reference has no multi-GPU path. */
int smat_partition_block_rows(const int* bcsr_rowptr_host, size_t Mb, int parts, size_t* bounds);

/* Text of the most recent error on the calling thread ("" if none). */
const char* smat_last_error_string(void);

#ifdef __cplusplus
}
#endif
#endif /* SMAT_B200_H */
