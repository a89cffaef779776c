// Internal declarations shared by the translation units of libsmat_b200.so.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/smat_b200.h"

namespace smat {

// Argument checks shared by the SpMM entry points (capi.cu).
int check_spmm_args(const void* vals, const int* rowptr, const int* colidx, const void* B, const void* C, size_t M,
                    size_t N, size_t K, size_t nnzb);

// Error text of the calling thread; returns `code` so that callers can `return fail(...)`.
int fail(int code, const char* fmt, ...);
void clear_error();

#define SMAT_CUDA_TRY(expr)                                                                          \
    do {                                                                                             \
        cudaError_t e__ = (expr);                                                                    \
        if (e__ != cudaSuccess)                                                                      \
            return ::smat::fail(SMAT_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), \
                                __FILE__, __LINE__);                                                 \
    } while (0)

// Per-device state created lazily on first use (with that device current): SM count and a small
// device status word that kernels set when one of their bounded waits runs out.
struct DeviceCtx {
    int device = -1;
    int sm_count = 0;
    int* d_status = nullptr;
    cudaMemPool_t pool = nullptr;  // the library's own pool for stream-ordered scratch (null for the static entry point)
};
int get_device_ctx(DeviceCtx** out);

void count_launch();

// Status word of the allocation-free entry point's fixed array (spmm_static.cu); see there.
int static_status_take(int* out);

// Device status codes (the word kernels set): 1..99 a bounded wait ran out at that wait site; 100.. the input
// structure is inconsistent (101: row pointers disagree with the number of blocks, 102: a block column is out of range
// or the columns of a block-row are not ascending).
constexpr int kStatusBadRowptr = 101;
constexpr int kStatusBadColumns = 102;

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup (no link against libcuda).
int encode_tensor_map_2d_f16(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_pitch_bytes,
                             uint32_t box_inner, uint32_t box_outer, int swizzle_bytes, int l2_promo_bytes);

// Most block-rows per work item of the SpMM kernel (one accumulator each).  A plan is built for groups of
// `rg` <= kPlanRowsPerGroup block-rows: small matrices / shards use smaller groups to fill the SMs.
constexpr int kPlanRowsPerGroup = 16;
// Scheduling model shared by the plan builder (group height) and the launcher (item width).
// An item is not cut into segments shorter than this many steps (on average).
constexpr int kMinStepsPerCta = 16;
// ... nor into more than this many: measured, finer cuts cost more in partial tiles than they save.
constexpr size_t kMaxTailParts = 4;
// Segments per item of the last round: `items` work items of about `est_steps` steps over `sms` CTAs.
inline size_t tail_parts_for(size_t items, size_t sms, bool can_cut, size_t est_steps) {
    const size_t left = items % sms;
    if (!can_cut || left == 0) return 1;
    size_t P = sms / left;
    if (P > est_steps / kMinStepsPerCta) P = est_steps / kMinStepsPerCta;
    if (P > kMaxTailParts) P = kMaxTailParts;
    return P < 1 ? 1 : P;
}
// Rounds of items over the SMs.  When the items of the last round are cut into P segments it counts 1/P plus the
// measured cost of the cut (pipeline refill, partial tiles, their summation): about a third of an item for
// 128-column items, a twelfth for 256-column items.
inline double rounds_for(size_t items, size_t sms, bool can_cut, size_t est_steps, bool wide) {
    if (items % sms == 0) return (double)(items / sms);
    const size_t P = tail_parts_for(items, sms, can_cut, est_steps);
    return (double)(items / sms) + 1.0 / (double)P + (P > 1 ? (wide ? 0.08 : 0.35) : 0.0);
}
// Measured cost of a 256-column item relative to a 128-column item of the same group.
constexpr double kWideItemCost = 1.95;
// Group height for a range of `block_rows` block-rows when C is N columns wide (0 = unknown): the height in
// [8, 16] with the smallest estimated time, rounds x (height + per-item overhead), for the better item width.
size_t choose_rows_per_group(size_t block_rows, size_t N, int sm_count, bool can_cut, size_t nnzb, size_t K);
// Bytes of that scratch: one partial tile of 2 x 16 block-rows x 16 x 128 fp32 per SM.
inline size_t fix_scratch_bytes(int sm_count) { return (size_t)sm_count * (2 * 16 * 16 * 128) * sizeof(float); }
// A step of the plan covers four consecutive block-columns and carries at most this many blocks.
constexpr int kPlanBlocksPerStep = 24;
// ... or this many, for plans of densely filled quads (most steps would otherwise be pieces of a cut quad): fewer,
// fuller steps at the price of one pipeline stage.
constexpr int kPlanBlocksPerStepDense = 32;
// The tall kernel (spmm_tall_sm100.cu) works on groups of up to kTallRows block-rows: a B panel fetched once feeds
// half again as many rows, and the panels are read by the MMAs from tensor memory.  Its plans ("tall" plans) have
// steps of at most kTallBlocksPerStep blocks, an even number of steps per group, and per pair of steps the list of
// MMAs of each issuing warp (PlanView::winfo).
constexpr int kTallRows = 24;
constexpr int kTallBlocksPerStep = 24;
// MMA-issuing warps of the kernel; each owns kPlanRowsPerGroup / kPlanOwners consecutive accumulators.
#ifndef SMAT_OWNERS
#define SMAT_OWNERS 8
#endif
constexpr int kPlanOwners = SMAT_OWNERS;

// The precomputed walk order of a block-row range (plan.cu).  All pointers are device memory.
//   gsp[n_groups + 1]  first step of every group of kPlanRowsPerGroup block-rows
//   steps              uint4 {element column of the quad (multiple of 64), position of the step's first block in the
//                      packed stream in 256-byte units, mask bits 0..31, mask bits 32..63} per step; a step is a quad of four
//                      consecutive block-columns of a group (or a slice of one holding at most
//                      kPlanBlocksPerStep blocks), ascending inside a group; mask bit
//                      16 * sub-column + row marks a block
//   blk[nnzb]          block indices in (group, block-column, row) order; indexed with the ABSOLUTE
//                      block position, i.e. the entries of group g occupy
//                      [rowptr[first row of g], rowptr[first row of g + 1])
//   packed             the stream the kernel copies from: the value blocks (512 bytes each) in (group, quad,
//                      sub-column, row) order, i.e. step after step and inside a step in mask-bit order, each
//                      block in the 32-byte-swizzled form the MMA shared-memory descriptor reads (16-byte
//                      chunk index XOR bit 2 of the row).  A step preceded by b blocks starts at byte 512 * b.
struct PlanView {
    const int* rowptr = nullptr;  // bcsrRowPtr of the whole matrix
    const int* gsp = nullptr;
    const void* steps = nullptr;
    const int* blk = nullptr;
    const void* packed = nullptr;
    // nnzb: blocks of block-rows [brow_begin, brow_end) when known (plans), else of the whole arrays; steers heuristics only
    size_t K = 0, nnzb = 0, brow_begin = 0, brow_end = 0, n_groups = 0, rg = kPlanRowsPerGroup;
    size_t total_steps = 0;  // number of steps of the range when the host knows it, else 0
    size_t cap = kPlanBlocksPerStep;  // most blocks of a step: kPlanBlocksPerStep or kPlanBlocksPerStepDense
    // Tall plan: groups of rg <= kTallRows block-rows with an even number of steps, at most kTallBlocksPerStep blocks
    // per step.  A step record is {element column of the quad, position of the first block in the packed stream in
    // 256-byte units, number of blocks (0: a step that only pads its group), non-empty sub-columns (bit s)}; winfo
    // holds 16 x 16 bytes per PAIR of steps: entry m < 12 lists the MMAs of the warp that owns block-rows 2m, 2m + 1
    // (layout: tall_pair_kernel in plan.cu).
    bool tall = false;
    const void* winfo = nullptr;
    // The heaviest group has many times the average number of steps: deal out equal step ranges instead of items
    // (needs fix_scratch of 2 x fix_scratch_bytes).
    bool balanced = false;
    // Or, preferred when it balances well enough: a fixed assignment of whole groups to `sched_ctas` CTAs, heaviest
    // first to the least loaded (device arrays: CTA c works on groups sched_list[sched_off[c] .. sched_off[c + 1])).
    const int* sched_off = nullptr;
    const int* sched_list = nullptr;
    int sched_ctas = 0;
    // Scratch for work items that are computed in segments by several CTAs (null: items are never cut):
    // fix_scratch_bytes(SMs) bytes, used by one launch at a time.
    float* fix_scratch = nullptr;
};

// Work-list sizes for a block-row range and the asynchronous build on `stream` (plan.cu).
struct PlanSizes { size_t n_groups, gsp_bytes, steps_bytes, blk_bytes, packed_bytes; };  // for max_steps steps
// max_steps = 0 means "not known yet": the bound nnzb (a step holds at least one block) is used.
PlanSizes plan_sizes(size_t nnzb, size_t brow_begin, size_t brow_end, size_t rg, size_t max_steps = 0);
// `ctx` (here and below): per-device state to use; nullptr = the lazily created one of get_device_ctx.
// Phase 1 fills gsp (step counts, scanned); phase 2 fills steps and blk.
int plan_count_async(const int* rowptr, const int* colidx, size_t K, size_t nnzb, size_t brow_begin, size_t brow_end,
                     size_t rg, int* gsp, cudaStream_t stream, const DeviceCtx* ctx = nullptr, size_t cap = kPlanBlocksPerStep);
int plan_fill_async(const int* rowptr, const int* colidx, size_t K, size_t nnzb, size_t brow_begin, size_t brow_end,
                    size_t rg, const int* gsp, void* steps, int* blk, cudaStream_t stream, const DeviceCtx* ctx = nullptr,
                    size_t cap = kPlanBlocksPerStep);
// Copies the value blocks of block-rows [brow_begin, brow_end) into their places in the packed stream.
int pack_values_async(const int* rowptr, const void* vals, const int* gsp, const void* steps, const int* blk, void* packed,
                      size_t brow_begin, size_t brow_end, size_t rg, size_t nnzb, cudaStream_t stream,
                      const DeviceCtx* ctx = nullptr);

// The same three phases for a tall plan.
int plan_count_tall_async(const int* rowptr, const int* colidx, size_t K, size_t nnzb, size_t brow_begin, size_t brow_end,
                          size_t rg, int* gsp, cudaStream_t stream, const DeviceCtx* ctx = nullptr);
int plan_fill_tall_async(const int* rowptr, const int* colidx, size_t K, size_t nnzb, size_t brow_begin, size_t brow_end,
                         size_t rg, const int* gsp, void* steps, void* wstep, void* winfo, int* blk, cudaStream_t stream,
                         const DeviceCtx* ctx = nullptr);
int pack_values_tall_async(const int* rowptr, const void* vals, const int* gsp, const void* steps, const int* blk, void* packed,
                           size_t brow_begin, size_t brow_end, size_t rg, size_t nnzb, cudaStream_t stream,
                           const DeviceCtx* ctx = nullptr);

// Launch of the SpMM kernel (spmm_sm100.cu).  `ldc`: elements between rows of C (0 = N, i.e. C is exactly N wide).
// [group_begin, group_end): the groups of the plan to multiply (default: all); C points at the first row of
// group_begin.
int launch_spmm(const PlanView& plan, const void* B, void* C, size_t N, cudaStream_t stream,
                const DeviceCtx* ctx = nullptr, size_t ldc = 0, size_t group_begin = 0, size_t group_end = (size_t)-1);

// The view of groups [group_begin, group_end) of a plan (steps, blocks and row pointers are addressed absolutely, so
// a sub-range is the same plan with its first group, first block-row and group count moved).
PlanView plan_group_range(const PlanView& whole, size_t group_begin, size_t group_end);
// Launch of the tall kernel (spmm_tall_sm100.cu) for a tall plan; same arguments.
int launch_spmm_tall(const PlanView& plan, const void* B, void* C, size_t N, cudaStream_t stream,
                     const DeviceCtx* ctx = nullptr, size_t ldc = 0, size_t group_begin = 0, size_t group_end = (size_t)-1);
// Adds up the fp32 partial tiles of the `cut_items` work items that a launch computed in `parts` segments each (the
// items of its last round) and writes their part of C (spmm_sm100.cu); wide: items are 256 columns wide.
int launch_sum_cut_items(bool wide, int cut_items, const float* scratch, void* C, int brow_begin, int brow_end, int rg, int N,
                         int n_tiles, int n_full, int parts, size_t ldc, cudaStream_t stream);

// 0 = choose per call, 1 = shared-memory-operand kernel, 2 = tensor-memory-operand kernel, 3 = 256-column items,
// 4 = plans created from now on are tall plans (tall kernel).
extern int g_spmm_variant;

}  // namespace smat
