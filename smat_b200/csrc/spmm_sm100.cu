// Block-sparse SpMM  C = A_bcsr x B  for NVIDIA B200 (sm_100a): tcgen05.mma with fp32 accumulators
// in tensor memory, B panels fetched by TMA, A blocks by bulk copies, persistent warp-specialised CTAs.
//
// Replaces the reference's one-warp-per-tile mma.sync kernel and its launcher
// (mmaCBTKernelSparse / mmaCBTKernel, src/cuda_hgemm/src/mma/mmaCBT.cu:13-88) behind the same
// argument convention and memory layouts.
//
// Mapping onto the tensor core.  A nonzero block is a dense 16x16 contraction, far below the
// 128-row minimum of tcgen05.mma, so the product is computed transposed:
//     C^T[n0:n0+128, 16 rows of block-row r]  +=  B^T[n0:n0+128, 16 k of block-column c] * A_blk^T
//   * MMA "A" operand = a panel of B: 128 n x 16 k, K-major -- exactly how the boundary stores B
//     (element (k, n) at B[n*K + k]); a TMA box {64 k, 128 n} fetches four such panels side by side,
//     written with the 128-byte swizzle, and the MMA descriptor selects one by a 32-byte offset;
//   * MMA "B" operand = the 16x16 block of A, row-major = N(16 rows) x K(16) K-major -- exactly how
//     BCSR stores it.  The plan keeps a copy of the blocks in the order the kernel consumes them,
//     already in the 32-byte-swizzled form the descriptor expects, so that all blocks of a step
//     arrive with ONE bulk copy (measured: per-block 16-byte cp.async gathers sustain only ~6
//     bytes/clock/SM from HBM because few of them can be in flight);
//   * D = 128 lanes (columns of C) x 16 fp32 columns (rows of the block-row) in tensor memory.
//
// Work decomposition.  A work item is (group of rg <= 16 consecutive block-rows) x (128 or 256 columns
// of C).  The accumulators of an item live in tensor memory at once (narrow items: two buffers of 256
// columns, so the epilogue of one item overlaps the main loop of the next; wide items: one buffer of
// 512).  An item walks the group's block-columns in ascending order in units of FOUR block-columns
// (64 k): measured on B200, a gather of 32-byte rows (one block-column of B) is limited to one 32-byte
// L2 sector per clock per SM whatever the engine (TMA or cp.async), so the panel is fetched 128 bytes
// wide -- the same number of requests moves four block-columns -- and feeds every block of the group
// in those four columns.  The walk order is precomputed (plan.cu): one 16-byte step descriptor
// {element column of the quad, first block, 64-bit (sub-column, row) mask} per non-empty quad (quads
// with more than CAP blocks are split) and the blocks themselves copied into (group, column, row) order.
// Vertically adjacent blocks of one block-column (adjacent accumulators, adjacent in the stage) are
// multiplied by ONE MMA with N = 16 x run length.
//
// Measured on B200: one thread can issue a tcgen05.mma only every ~50 cycles (150-200 when the
// descriptors change from one MMA to the next) and a TMA / bulk copy only every ~160-250 cycles,
// whatever their size, while different warps issue concurrently.  So issue is spread over warps:
// 4 loader warps (each takes every 4th step: one TMA for the panel, one bulk copy for the step's A
// blocks), 8 MMA warps (each owns two accumulator rows, so that every accumulator is updated by a
// single thread, in order), 4 epilogue warps (tcgen05.ld -> zero the accumulator -> fp16 -> for narrow items a
// shared-memory tile per block-row stored with one TMA store, for wide items paired coalesced stores) and, for
// the tensor-memory-operand variant, 4 panel-copier warps.
//
// Scheduling.  Items go round-robin over the persistent CTAs while there is one for every CTA; the
// items left for the last round are cut into equal segments so that it keeps every SM busy (SegGen
// below), and a small second kernel adds the fp32 partial tiles of the cut items.
//
// Every wait is bounded: when a wait runs out the kernel records a status code, stops waiting
// anywhere in the CTA, and runs to completion (results are then invalid and the host reports
// SMAT_ERR_DEVICE_WAIT).
#include <cuda_fp16.h>
#include <limits.h>
#include <stdlib.h>

#include <cstdlib>

#include <type_traits>

#include "ptx_sm100.cuh"
#include "smat_internal.h"
#include "spmm_sched.cuh"

namespace smat {

using namespace ptx;

namespace {

constexpr int NL = 4;                  // loader warps
#ifndef SMAT_TMA_EPILOGUE
#define SMAT_TMA_EPILOGUE 1
#endif
// L2 prefetches of the panel and the blocks a few steps ahead of their copies (kernel argument `pf`) are off unless the
// environment variable SMAT_L2_PREFETCH=1 asks for them.  Measured on the final kernel they change nothing where the copies
// are not the limit (uniform, block-sparse layer and its shards, power-law) and cost a third of the time where they are
// (dense clusters: 0.335 -> 0.230 ms without), because a prefetch occupies the copy engine like a copy.
constexpr int NM = kPlanOwners;        // MMA-issuing warps; warp m owns accumulators [m * RG / NM, (m + 1) * RG / NM)
constexpr int NC = 4;                  // panel-copier warps (used by the tensor-memory-operand variant)
constexpr int kThreads = (NL + NC + NM + 4) * 32;
constexpr uint32_t TMEM_PANELS = 256;  // first tensor-memory column of the panel ring (TS variant): S x 32 columns
constexpr uint32_t ABLK_BYTES = 16 * 16 * 2;

// Shared-memory plan of a kernel whose work item is NH x 128 columns of C wide, for plans with at most CAP blocks
// per step.
template <int NH, int CAP>
struct Cfg {
    static constexpr uint32_t S = CAP <= 24 ? (NH == 1 ? 7 : 5) : (NH == 1 ? 6 : 4);              // steps in flight (pipeline stages)
    static constexpr uint32_t PANEL_BYTES = NH * 128 * 64 * 2;  // NH x (128 n x 64 k fp16)
    static constexpr uint32_t STAGE_BYTES = (PANEL_BYTES + CAP * ABLK_BYTES + 1023) / 1024 * 1024;
    static constexpr uint32_t OFF_STAGE = 0;
    static constexpr uint32_t OFF_META = OFF_STAGE + S * STAGE_BYTES;
    static constexpr uint32_t OFF_BAR = OFF_META + S * 8;
    static constexpr uint32_t N_BARS = 3 * S + 4;
    static constexpr uint32_t OFF_MISC = OFF_BAR + N_BARS * 8;
    // fp16 tiles of 16 rows x 128 columns that the epilogue hands to TMA stores (three per group of four epilogue
    // warps), 1024-byte aligned
    static constexpr uint32_t OFF_EPI = (OFF_MISC + 16 + 1023) / 1024 * 1024;
    static constexpr uint32_t EPI_TILE_BYTES = 16 * 128 * 2;
    // (narrow items only: wide items have no room left for them beside five stages, and their items are long enough
    // for the epilogue not to matter)
    static constexpr bool TMA_EPILOGUE = SMAT_TMA_EPILOGUE && NH == 1;
    static constexpr uint32_t SMEM_BYTES = (TMA_EPILOGUE ? OFF_EPI + 6 * EPI_TILE_BYTES : OFF_MISC + 16) + 1024;  // slack for the manual 1024-byte alignment
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
    static_assert(STAGE_BYTES % 1024 == 0 && CAP <= 32, "stage alignment");
};

static_assert(RG == 16, "row masks and accumulator ownership below assume 16 block-rows per group");
static_assert(RG * 2 * 16 <= 512 && TMEM_PANELS + Cfg<1, kPlanBlocksPerStep>::S * 32 <= 512, "tensor-memory budget");

// One loader-warp pipeline record: a step on its way from "descriptor requested" to "copies issued".
struct StepRec {
    int live;     // the record holds a step
    int tile;     // n-tile of the item
    uint32_t st;  // position of the step in this CTA's step sequence (selects the stage)
    uint4 d;      // {element column of the quad, first packed block, mask bits 0..31, mask bits 32..63}
};

// TS = false: both MMA operands from shared memory, two accumulator buffers (the epilogue of an item
//   overlaps the main loop of the next).
// TS = true: the panel is first copied shared -> tensor memory (tcgen05.cp, once per sub-column) and the
//   MMAs read it from there, so the 4 KB panel no longer crosses the shared-memory port once per block;
//   the panel ring takes the tensor-memory columns of the second accumulator buffer, so there is one
//   buffer and no epilogue overlap.
// NH = 1: a work item is 128 columns of C wide.  NH = 2: 256 columns -- every A block then feeds two
//   independent MMAs (one per 128-column half, own accumulator), which doubles the MMA work per stage
//   hand-over and halves the A traffic per MMA; the 32 accumulators fill tensor memory (one buffer).
template <bool TS, int NH, int SCHED, int CAP>
__global__ void __launch_bounds__(kThreads, 1)
spmm_bcsr_tc_kernel(const __grid_constant__ CUtensorMap mapB, const __grid_constant__ CUtensorMap mapC,
                    const uint8_t* __restrict__ packed,
                    const uint4* __restrict__ steps, const int* __restrict__ gsp,
                    const int* __restrict__ rowptr, __half* __restrict__ C, int brow_begin, int brow_end, int rg, int N,
                    int n_tiles, int n_items, int n_groups, int tail_parts, uint32_t panel_bytes,
                    float* __restrict__ fix_scratch, int* status, size_t ldc, const int* __restrict__ sched_off,
                    const int* __restrict__ sched_list, int nm, int pf) {
    static_assert(!(TS && NH == 2), "the panel ring and 32 accumulators do not fit tensor memory together");
    // The schedule is a template parameter: measured, the code generated for the MMA issue loop changed by up to 35 %
    // with the shape of the control flow around it, so each schedule gets a kernel with only its own loops.
    constexpr bool listed = SCHED == 1, balanced = SCHED == 2;
    // A loader waits on a stage's `empty` barrier by parity, which only tells phases apart while the waiter is
    // less than two uses ahead of the consumers; with steps consumed in order that holds iff NL <= S.
    static_assert(NL <= (int)Cfg<NH, CAP>::S, "more loader warps than stages would alias barrier phases");
    using G = Cfg<NH, CAP>;
    constexpr uint32_t S = G::S, PANEL_BYTES = G::PANEL_BYTES, STAGE_BYTES = G::STAGE_BYTES, OFF_STAGE = G::OFF_STAGE,
                       OFF_META = G::OFF_META, OFF_BAR = G::OFF_BAR, OFF_MISC = G::OFF_MISC;
    constexpr int NT = 128 * NH;  // columns of C per work item
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar0 = base + OFF_BAR;
    auto full = [&](uint32_t s) { return bar0 + 8 * s; };
    auto empty = [&](uint32_t s) { return bar0 + 8 * (S + s); };
    auto tfull = [&](uint32_t s) { return bar0 + 8 * (2 * S + s); };
    auto acc_full = [&](uint32_t b) { return bar0 + 8 * (3 * S + b); };
    auto acc_empty = [&](uint32_t b) { return bar0 + 8 * (3 * S + 2 + b); };
    constexpr uint32_t NBUF = (TS || NH == 2) ? 1 : 2;
    // Epilogue groups of four warps (one per tensor-memory lane quarter); group g takes block-rows g, g + EG, ...  The
    // panel-copier warps, idle unless the panels go through tensor memory, form the second group: measured on work items
    // of a dozen steps (dense clusters) the epilogue, not the main loop, bounds the kernel.
    constexpr int EG = TS ? 1 : 2;
    const uint32_t tmem_slot = base + OFF_MISC;
    const uint32_t abort_addr = base + OFF_MISC + 4;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // The CTA's share of the work (every role walks the same sequence of segments).
    const int n_full = n_items / (int)gridDim.x * (int)gridDim.x;  // items of the complete rounds
    Flat flat;
    flat.gsp = gsp; flat.n_tiles = n_tiles; flat.n_groups = n_groups;
    flat.total = balanced ? (long long)(__ldg(gsp + n_groups) - __ldg(gsp)) * n_tiles : 0;
    auto make_gen = [&]() {
        SegGen<SCHED> sg;
        sg.gsp = gsp; sg.n_tiles = n_tiles; sg.n_items = n_items; sg.n_ctas = (int)gridDim.x; sg.cta = (int)blockIdx.x;
        sg.item = (int)blockIdx.x; sg.n_full = n_full; sg.P = tail_parts; sg.tail_done = false;
        sg.flat = flat; sg.g = 0;
        sg.p = sg.p_begin = sg.p_end = 0;
        sg.list = sched_list; sg.li = sg.li_end = 0; sg.lt = 0;
        if (listed) { sg.li = __ldg(sched_off + blockIdx.x); sg.li_end = __ldg(sched_off + blockIdx.x + 1); }
        if (balanced) {
            sg.p = sg.p_begin = flat.range_begin((int)gridDim.x, (int)blockIdx.x);
            sg.p_end = flat.range_begin((int)gridDim.x, (int)blockIdx.x + 1);
            if (sg.p < sg.p_end) sg.g = flat.group_of(sg.p);
        }
        return sg;
    };

    if (threadIdx.x == 0) {
        // nm <= NM of the MMA warps take part (fewer warps own more rows each, so that runs of vertically adjacent
        // blocks -- one MMA each -- can be longer: plans of densely filled quads)
        for (uint32_t s = 0; s < S; s++) { mbar_init(full(s), 1); mbar_init(empty(s), (uint32_t)nm); mbar_init(tfull(s), 1); }
        for (uint32_t b = 0; b < 2; b++) { mbar_init(acc_full(b), (uint32_t)nm); mbar_init(acc_empty(b), 4 * EG); }
        st_shared_u32(abort_addr, 0);
        fence_barrier_init();
        fence_proxy_async();
        prefetch_tensormap(&mapB);
        prefetch_tensormap(&mapC);
    }
    if (warp == NL) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ld_shared_u32(tmem_slot);
    if (warp < 4) {
        // all accumulators start at zero (later the epilogue re-zeroes what it reads)
#pragma unroll 4
        for (uint32_t c = 0; c < 512; c += 16) tmem_zero_x16(tmem_base + ((uint32_t)(warp * 32) << 16) + c);
        tmem_st_wait();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    // ------------------------------ epilogue: tensor memory -> fp16 -> C ------------------------------
    auto epilogue = [&](const int grp) {
        const int quarter = warp & 3;  // a warp may only read tensor-memory lanes [32*(warp%4), +32)
        const bool odd = lane & 1;
        const int et = quarter * 32 + lane;  // index among the 128 epilogue threads = column within a 128-column half
        if (balanced && grp == 0) {
            // groups without any block have no steps, so no range reaches them: their rows of C are zeroed here
            for (int g = (int)blockIdx.x; g < n_groups; g += (int)gridDim.x) {
                if (__ldg(gsp + g + 1) != __ldg(gsp + g)) continue;
                const int r0 = brow_begin + g * rg;
                const int nrows = min(rg, brow_end - r0);
                for (int row = 0; row < nrows * 16; row++) {
                    uint4* dst = reinterpret_cast<uint4*>(C + ((size_t)(r0 - brow_begin) * 16 + row) * ldc);
                    for (int i = et; i < N / 8; i += 128) dst[i] = make_uint4(0, 0, 0, 0);
                }
            }
        }
        uint32_t it = 0, epi_n = 0;
        const uint32_t c_pitch = (uint32_t)(N < 128 ? N : 128) * 2u;  // bytes per row of a tile = the box of mapC
        SegGen<SCHED> sg = make_gen();
        Seg cs;
        for (; sg.next(cs); ++it) {
            const int g = cs.item / n_tiles, t = cs.item - g * n_tiles;
            const int r0 = brow_begin + g * rg;
            const int nrows = min(rg, brow_end - r0);
            const int lo = (lane < nrows) ? __ldg(rowptr + r0 + lane) : 0;
            const int hi = (lane < nrows) ? __ldg(rowptr + r0 + lane + 1) : 0;
            const uint32_t nonempty = __ballot_sync(0xffffffffu, hi > lo);
            const uint32_t buf = it % NBUF;
            const bool partial = cs.cut;
            float* part_dst = fix_scratch + (size_t)cs.slot * (size_t)kFixSlotFloats;  // scratch tile of this segment
            if (lane == 0) wait_bar(acc_full(buf), (it / NBUF) & 1, abort_addr, status, 6);
            __syncwarp();
            tc_fence_after();
            int last_r = -1;  // last block-row this group handles
            for (int r = grp; r < nrows; r += EG) last_r = r;
            if (last_r < 0 && lane == 0) mbar_arrive(acc_empty(buf));  // nothing to read: hand the accumulators back at once
            for (int r = grp; r < nrows; r += EG) {
#pragma unroll
                for (int h = 0; h < NH; h++) {
                    const int n = t * NT + h * 128 + et;
                    uint32_t v[16];
                    if ((nonempty >> r) & 1u) {
                        const uint32_t taddr =
                            tmem_base + ((uint32_t)(quarter * 32) << 16) + ((buf * NH + h) * RG + (uint32_t)r) * 16;
                        tmem_ld_x16(taddr, v);
                        tmem_ld_wait();
                        tmem_zero_x16(taddr);  // leave the accumulator zeroed for the next segment that uses this buffer
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; i++) v[i] = 0u;
                    }
                    if (r == last_r && h == NH - 1) {
                        // this warp has read and zeroed its share of the buffer: hand it back to the MMA warps
                        tmem_st_wait();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(acc_empty(buf));
                    }
                    if (partial) {
                        float* d = part_dst + ((size_t)(h * RG + r) * 16) * 128 + et;
#pragma unroll
                        for (int i = 0; i < 16; i++) d[(size_t)i * 128] = __uint_as_float(v[i]);
                        continue;
                    }
                    if constexpr (G::TMA_EPILOGUE) {
                        // fp16 tile of this block-row (16 rows x 128 columns, row-major, `c_pitch` bytes per row) in shared
                        // memory, handed to one TMA store; three tiles in rotation: the tile written now was last read by
                        // the store issued three tiles ago, whose completion the issuing thread awaited before the
                        // barrier of the previous tile.
                        const uint32_t tile = base + G::OFF_EPI + ((uint32_t)grp * 3u + epi_n % 3u) * G::EPI_TILE_BYTES;
                        if ((uint32_t)et * 2u < c_pitch) {  // C narrower than a tile: the rows of the box are N columns long
#pragma unroll
                            for (int i = 0; i < 16; i++)
                                st_shared_u16(tile + (uint32_t)i * c_pitch + (uint32_t)et * 2u,
                                              __half_as_ushort(__float2half_rn(__uint_as_float(v[i]))));
                        }
                        fence_proxy_async();
                        if (et == 0) bulk_wait_group_read<1>();
                        if (grp == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
                        else asm volatile("bar.sync 2, 128;" ::: "memory");
                        if (et == 0) {
                            tma_store_2d(&mapC, tile, t * NT + h * 128, (r0 - brow_begin + r) * 16);
                            bulk_commit_group();
                        }
                        epi_n++;
                        continue;
                    }
                    __half* crow = C + ((size_t)(r0 - brow_begin + r) * 16 + (odd ? 8 : 0)) * ldc + (size_t)(n & ~1);
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        // lane pairs exchange halves: even lanes keep rows 0..7, odd lanes rows 8..15,
                        // each for the two adjacent columns (n & ~1, n | 1) -> one 4-byte store per row
                        const float keep = __uint_as_float(odd ? v[i + 8] : v[i]);
                        const float send = __uint_as_float(odd ? v[i] : v[i + 8]);
                        const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
                        const __half2 hh = odd ? __floats2half2_rn(recv, keep) : __floats2half2_rn(keep, recv);
                        if (n < N) *reinterpret_cast<__half2*>(crow + (size_t)i * ldc) = hh;
                    }
                }
            }
        }
    };

    if (warp < NL) {
        // ------------------------------ loader warp j: every NL-th step ------------------------------
        const int j = warp;
        // Software pipeline over the warp's steps, unrolled U times so that every record lives in fixed
        // registers (a record whose descriptor load is still in flight is never copied): the descriptor
        // of position i + U is requested while position i is consumed.  One thread per warp works.
        if (lane == 0) {
            SegGen<SCHED> sg = make_gen();
            Seg cs;
            bool have = sg.next(cs);
            uint32_t h_st0 = 0, h_next = (uint32_t)j;  // sequence position of the segment's first step; next position of this warp
            constexpr int U = 8;
            StepRec rec[U];
            auto gen = [&](StepRec& r) {  // next step of this warp; requests its descriptor
                while (have && h_next >= h_st0 + (uint32_t)(cs.k1 - cs.k0)) {
                    h_st0 += (uint32_t)(cs.k1 - cs.k0);
                    have = sg.next(cs);
                }
                r.live = have;
                if (have) {
                    r.tile = cs.item % n_tiles;
                    r.st = h_next;
                    r.d = __ldg(steps + cs.gs + cs.k0 + (int)(h_next - h_st0));
                    h_next += NL;
                }
            };
            // When the launch asks for it (pf): the panel and the blocks of the step U/2 positions ahead (of this warp;
            // NL * U/2 steps ahead overall) are prefetched into L2.
            auto prefetch = [&](const StepRec& r) {
                if (pf && r.live) {
                    tma_prefetch_l2_2d(&mapB, (int)r.d.x, r.tile * NT);
                    bulk_prefetch_l2(packed + (size_t)r.d.y * 256, (uint32_t)(__popc(r.d.z) + __popc(r.d.w)) * ABLK_BYTES);
                }
            };
#pragma unroll
            for (int a = 0; a < U; a++) gen(rec[a]);
#pragma unroll
            for (int a = 0; a < U / 2; a++) prefetch(rec[a]);
            bool more = true;
            while (more) {
#pragma unroll
                for (int a = 0; a < U; a++) {
                    StepRec& r = rec[a];
                    if (!r.live) { more = false; break; }
                    prefetch(rec[(a + U / 2) % U]);
                    const uint32_t slot = r.st % S;
                    wait_bar(empty(slot), ((r.st / S) & 1) ^ 1, abort_addr, status, 1);
                    const uint32_t stage = base + OFF_STAGE + slot * STAGE_BYTES;
                    const uint32_t a_bytes = (uint32_t)(__popc(r.d.z) + __popc(r.d.w)) * ABLK_BYTES;
                    st_shared_u32(base + OFF_META + slot * 8, r.d.z);
                    st_shared_u32(base + OFF_META + slot * 8 + 4, r.d.w);
                    mbar_arrive_expect_tx(full(slot), panel_bytes + a_bytes);
                    tma_load_2d(stage, &mapB, (int)r.d.x, r.tile * NT, full(slot));
                    bulk_load(stage + PANEL_BYTES, packed + (size_t)r.d.y * 256, a_bytes, full(slot));
                    gen(r);  // this register set now follows the warp's step U positions ahead
                }
            }
        }
        __syncwarp();
    } else if (warp < NL + NC) {
        // ------------------------------ panel copier j (TS only): shared -> tensor memory, every NC-th step ------------------------------
        if constexpr (!TS) epilogue(1);
        if (TS && lane == 0) {
            const uint32_t j = (uint32_t)(warp - NL);
            uint32_t st = 0;
            SegGen<SCHED> sg = make_gen();
            Seg cs;
            while (sg.next(cs)) {
                for (int k = cs.k0; k < cs.k1; k++, st++) {
                    const uint32_t slot = st % S;
                    // Every copier observes every stage in order, although it copies only its own: a
                    // parity wait is only meaningful for a waiter that is less than one phase away, and
                    // a copier that skipped stages could meet a barrier one whole use behind.
                    wait_bar(full(slot), (st / S) & 1, abort_addr, status, 2);
                    if (st % NC != j) continue;
                    tc_fence_after();
                    const uint32_t mlo = ld_shared_u32(base + OFF_META + slot * 8);
                    const uint32_t mhi = ld_shared_u32(base + OFF_META + slot * 8 + 4);
                    const uint64_t pdesc = smem_desc_k_sw128(base + OFF_STAGE + slot * STAGE_BYTES);
                    const uint32_t tdst = tmem_base + TMEM_PANELS + slot * 32;
                    if (mlo & 0xffffu) tc_cp_128x256b(tdst, pdesc);
                    if (mlo >> 16) tc_cp_128x256b(tdst + 8, pdesc + 2);
                    if (mhi & 0xffffu) tc_cp_128x256b(tdst + 16, pdesc + 4);
                    if (mhi >> 16) tc_cp_128x256b(tdst + 24, pdesc + 6);
                    tc_commit(tfull(slot));
                }
            }
        }
        __syncwarp();
    } else if (warp < NL + NC + NM) {
        // ------------------------------ MMA warp m ------------------------------
        // The whole warp walks the step's (sub-column, row) mask in lock-step and one elected lane issues;
        // the mask words reach the loop as ballots, i.e. as values the compiler knows to be warp-uniform.
        // (Measured: a single lane walking a precomputed list of MMAs from shared memory was ~20 % slower.)
        if (warp - NL - NC < nm) {
            const uint32_t m = (uint32_t)__shfl_sync(0xffffffffu, warp - NL - NC, 0);
            const uint32_t P_HI = (uint32_t)(smem_desc_k_sw128(0) >> 32), B_HI = (uint32_t)(smem_desc_k_sw32(0) >> 32);
            constexpr uint32_t IDESC_N0 = idesc_f16_f32(128, 0);  // the N field is added per run: N = 16 * length
            const uint32_t rpo = (uint32_t)((rg + nm - 1) / nm);  // rows per owning warp (the last warps may own none)
            const uint32_t rows_m = ((1u << rpo) - 1u) << (m * rpo);
            const uint32_t own32 = (rows_m & 0xffffu) | (rows_m << 16);  // this warp's rows in both sub-columns of a mask word
            const bool leader = elect_one();  // the lane that issues; fixed, so that its commits cover its MMAs
            uint32_t st = 0, it = 0;
            // One segment = steps [k0, k1) of an item.  Kept as a plain counted loop called from two plain loops
            // (measured: driving it from the segment generator's control flow made the issue loop ~35 % slower).
            auto run_segment = [&](const int k0, const int k1) {
                const uint32_t buf = it % NBUF;
                // the accumulators were zeroed by the epilogue after it read them (or at kernel start), so
                // every MMA accumulates and runs may span rows with and without earlier blocks
                wait_bar(acc_empty(buf), ((it / NBUF) & 1) ^ 1, abort_addr, status, 3);
                tc_fence_after();
                const uint32_t acc0 = tmem_base + buf * RG * 16 * NH;
                for (int k = k0; k < k1; k++, st++) {
                    const uint32_t slot = st % S;
                    wait_bar(TS ? tfull(slot) : full(slot), (st / S) & 1, abort_addr, status, 4);
                    tc_fence_after();
                    const uint32_t stage = base + OFF_STAGE + slot * STAGE_BYTES;
                    const uint32_t p_lo = (uint32_t)smem_desc_k_sw128(stage);               // panel, sub-column 0
                    const uint32_t tpanel = tmem_base + TMEM_PANELS + slot * 32;            // its copy in tensor memory
                    const uint32_t b_lo = (uint32_t)smem_desc_k_sw32(stage + PANEL_BYTES);  // block slot 0
                    const uint32_t wlo = ld_shared_u32(base + OFF_META + slot * 8);
                    const uint32_t whi = ld_shared_u32(base + OFF_META + slot * 8 + 4);
                    const uint32_t mw0 = __ballot_sync(0xffffffffu, (wlo >> lane) & 1u);
                    const uint32_t mw1 = __ballot_sync(0xffffffffu, (whi >> lane) & 1u);
                    // one region of the elected lane per step: every separate `if (leader)` costs the warp a
                    // divergence and a reconvergence
                    if (leader) {
                    uint32_t qbase = 0;
#pragma unroll
                    for (int half = 0; half < 2; half++) {
                        const uint32_t mw = half ? mw1 : mw0;
                        uint32_t own = mw & own32;
                        while (own) {
                            const uint32_t b = (uint32_t)__ffs((int)own) - 1u;
                            // run of adjacent rows of this sub-column (a mask word holds two sub-columns of 16 rows)
                            const uint32_t len = min((uint32_t)__ffs((int)~(own >> b)) - 1u, 16u - (b & 15u));
                            const uint32_t q = qbase + (uint32_t)__popc(mw & ((1u << b) - 1u));   // blocks are stored in mask-bit order
                            const uint32_t r0 = b & 15u, sub = (uint32_t)half * 2u + (b >> 4);
                            const uint32_t idesc = IDESC_N0 + ((2u * len) << 17);
                            own &= ~(((1u << len) - 1u) << b);
                            if (TS) {
                                mma_f16_ts_lohi(acc0 + r0 * 16, tpanel + sub * 8u, b_lo + q * (ABLK_BYTES >> 4), B_HI, idesc, 1u);
                            } else {
#pragma unroll
                                for (int h = 0; h < NH; h++)  // one MMA per 128-column half, each into its own accumulators
                                    mma_f16_ss_lohi(acc0 + (h * RG + r0) * 16, p_lo + sub * 2u + h * (128 * 128 >> 4), P_HI,
                                                    b_lo + q * (ABLK_BYTES >> 4), B_HI, idesc, 1u);
                            }
                        }
                        qbase += (uint32_t)__popc(mw);
                    }
                    tc_commit(empty(slot));
                    }
                }
                if (leader) tc_commit(acc_full(buf));
                ++it;
            };
            if (listed) {  // this CTA's list of groups, every tile of each
                const int l1 = __ldg(sched_off + blockIdx.x + 1);
                for (int l = __ldg(sched_off + blockIdx.x); l < l1; l++) {
                    const int g = __ldg(sched_list + l);
                    const int ns = __ldg(gsp + g + 1) - __ldg(gsp + g);
                    for (int t = 0; t < n_tiles; t++) run_segment(0, ns);
                }
            } else if (balanced) {  // this CTA's range of the flattened (item, step) sequence
                long long pp = flat.range_begin((int)gridDim.x, (int)blockIdx.x);
                const long long pe = flat.range_begin((int)gridDim.x, (int)blockIdx.x + 1);
                int g = pp < pe ? flat.group_of(pp) : 0;
                while (pp < pe) {
                    while (flat.first_of_group(g + 1) <= pp) g++;
                    const int ns = __ldg(gsp + g + 1) - __ldg(gsp + g);
                    const long long off = pp - flat.first_of_group(g);
                    const int k0 = (int)(off % ns);
                    const int k1 = (pe - pp < (long long)(ns - k0)) ? k0 + (int)(pe - pp) : ns;
                    run_segment(k0, k1);
                    pp += k1 - k0;
                }
            }
            for (int item = blockIdx.x; SCHED == 0 && item < n_full; item += gridDim.x) {  // the complete rounds: whole items
                const int g = item / n_tiles;
                run_segment(0, __ldg(gsp + g + 1) - __ldg(gsp + g));
            }
            if (SCHED == 0 && (int)blockIdx.x < (n_items - n_full) * tail_parts) {  // the last round: one segment of an item
                const int i = (int)blockIdx.x / tail_parts, j = (int)blockIdx.x - i * tail_parts;
                const int g = (n_full + i) / n_tiles;
                const unsigned ns = (unsigned)(__ldg(gsp + g + 1) - __ldg(gsp + g));  // times j <= 4: fits 32 bits
                const int k0 = __shfl_sync(0xffffffffu, (int)(ns * (unsigned)j / (unsigned)tail_parts), 0);
                const int k1 = __shfl_sync(0xffffffffu, (int)(ns * (unsigned)(j + 1) / (unsigned)tail_parts), 0);
                run_segment(k0, k1);
            }
        }
        __syncwarp();
    } else {
        epilogue(0);
    }

    // the threads that issued the stores of C (one per epilogue group)
    if (G::TMA_EPILOGUE && (warp == NL + NC + NM || (!TS && warp == NL)) && lane == 0) bulk_wait_group_all();
    tc_fence_before();
    __syncthreads();
    if (ld_shared_u32(abort_addr)) {
        // a wait ran out somewhere: give copies still in flight time to land before the CTA retires
        for (int i = 0; i < 64; i++) __nanosleep(1000);
    }
    if (warp == NL) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

__global__ void zero_rows_kernel(uint4* dst, size_t n16) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n16; i += stride) dst[i] = make_uint4(0, 0, 0, 0);
}

// Adds up the partial tiles of the work items that the main kernel computed in `parts` segments (the items of its
// last round; segment j of the i-th of them is in scratch tile i * parts + j) and writes their part of C.
// One block of (128 columns x 4) threads per item.
template <int NH>
__global__ void __launch_bounds__(512) sum_cut_items_kernel(const float* __restrict__ scratch, __half* __restrict__ C, int brow_begin,
                                                           int brow_end, int rg, int N, int n_tiles, int n_full, int parts, size_t ldc) {
    const int item = n_full + (int)blockIdx.x;
    const int g = item / n_tiles, t = item - g * n_tiles;
    const int r0 = brow_begin + g * rg;
    const int nrows = min(rg, brow_end - r0);
    const float* tile0 = scratch + (size_t)blockIdx.x * parts * (size_t)kFixSlotFloats;
    for (int r = (int)threadIdx.y; r < nrows; r += (int)blockDim.y) {
#pragma unroll
        for (int h = 0; h < NH; h++) {
            const int n = t * (128 * NH) + h * 128 + (int)threadIdx.x;
            if (n >= N) continue;
            float acc[16];
#pragma unroll
            for (int i = 0; i < 16; i++) acc[i] = 0.0f;
            for (int j = 0; j < parts; j++) {
                const float* src = tile0 + (size_t)j * kFixSlotFloats + ((size_t)(h * RG + r) * 16) * 128 + threadIdx.x;
#pragma unroll
                for (int i = 0; i < 16; i++) acc[i] += __ldg(src + (size_t)i * 128);
            }
            __half* ccol = C + ((size_t)(r0 - brow_begin + r) * 16) * ldc + (size_t)n;
#pragma unroll
            for (int i = 0; i < 16; i++) ccol[(size_t)i * ldc] = __float2half_rn(acc[i]);
        }
    }
}

// The same for the balanced schedule.  Block c-1 looks at the boundary between the ranges of CTAs c-1 and c: if it
// falls strictly inside a work item and is the first boundary to do so, the block adds up that item's segments
// (tile 1 of the CTA in whose range the item begins, tile 0 of every later CTA up to the one holding its end).
template <int NH>
__global__ void __launch_bounds__(512) sum_split_items_kernel(const float* __restrict__ scratch, const int* __restrict__ gsp,
                                                             __half* __restrict__ C, int brow_begin, int brow_end, int rg, int N,
                                                             int n_tiles, int n_groups, int n_ctas, size_t ldc) {
    Flat flat;
    flat.gsp = gsp; flat.n_tiles = n_tiles; flat.n_groups = n_groups;
    flat.total = (long long)(__ldg(gsp + n_groups) - __ldg(gsp)) * n_tiles;
    const int c = (int)blockIdx.x + 1;
    const long long b = flat.range_begin(n_ctas, c);
    if (b <= 0 || b >= flat.total) return;
    int g = flat.group_of(b);
    while (flat.first_of_group(g + 1) <= b) g++;
    const int ns = __ldg(gsp + g + 1) - __ldg(gsp + g);
    const long long off = b - flat.first_of_group(g);
    const int t = (int)(off / ns);
    const long long item_p0 = flat.first_of_group(g) + (long long)t * ns;
    if (b == item_p0) return;                                       // the boundary is the start of an item
    if (c > 1 && flat.range_begin(n_ctas, c - 1) > item_p0) return;  // an earlier boundary cuts the same item
    const int c_first = c - 1, c_last = flat.range_owner(n_ctas, item_p0 + ns - 1);
    const int r0 = brow_begin + g * rg;
    const int nrows = min(rg, brow_end - r0);
    for (int r = (int)threadIdx.y; r < nrows; r += (int)blockDim.y) {
#pragma unroll
        for (int h = 0; h < NH; h++) {
            const int n = t * (128 * NH) + h * 128 + (int)threadIdx.x;
            if (n >= N) continue;
            float acc[16];
#pragma unroll
            for (int i = 0; i < 16; i++) acc[i] = 0.0f;
            for (int cc = c_first; cc <= c_last; cc++) {
                if (flat.range_begin(n_ctas, cc) == flat.range_begin(n_ctas, cc + 1)) continue;  // a CTA without work
                const int slot = cc * 2 + (flat.range_begin(n_ctas, cc) < item_p0 ? 1 : 0);
                const float* src = scratch + (size_t)slot * kFixSlotFloats + ((size_t)(h * RG + r) * 16) * 128 + threadIdx.x;
#pragma unroll
                for (int i = 0; i < 16; i++) acc[i] += __ldg(src + (size_t)i * 128);
            }
            __half* ccol = C + ((size_t)(r0 - brow_begin + r) * 16) * ldc + (size_t)n;
#pragma unroll
            for (int i = 0; i < 16; i++) ccol[(size_t)i * ldc] = __float2half_rn(acc[i]);
        }
    }
}

}  // namespace


int g_spmm_variant = 0;

PlanView plan_group_range(const PlanView& whole, size_t group_begin, size_t group_end) {
    PlanView plan = whole;
    if (group_begin > 0 || group_end < whole.n_groups) {
        plan.gsp = whole.gsp + group_begin;
        plan.n_groups = group_end - group_begin;
        plan.brow_begin = whole.brow_begin + group_begin * whole.rg;
        if (whole.brow_begin + group_end * whole.rg < whole.brow_end) plan.brow_end = whole.brow_begin + group_end * whole.rg;
        plan.nnzb = whole.nnzb * plan.n_groups / whole.n_groups;  // only steers the choice of the variant
        if (plan.nnzb == 0 && whole.nnzb) plan.nnzb = 1;
        plan.total_steps = whole.total_steps * plan.n_groups / whole.n_groups;
    }
    return plan;
}

int launch_sum_cut_items(bool wide, int cut_items, const float* scratch, void* C, int brow_begin, int brow_end, int rg, int N,
                         int n_tiles, int n_full, int parts, size_t ldc, cudaStream_t stream) {
    if (wide)
        sum_cut_items_kernel<2><<<cut_items, dim3(128, 4), 0, stream>>>(scratch, reinterpret_cast<__half*>(C), brow_begin, brow_end, rg, N,
                                                                       n_tiles, n_full, parts, ldc);
    else
        sum_cut_items_kernel<1><<<cut_items, dim3(128, 4), 0, stream>>>(scratch, reinterpret_cast<__half*>(C), brow_begin, brow_end, rg, N,
                                                                       n_tiles, n_full, parts, ldc);
    count_launch();
    SMAT_CUDA_TRY(cudaGetLastError());
    return SMAT_OK;
}

int launch_spmm(const PlanView& whole, const void* B, void* C, size_t N, cudaStream_t stream, const DeviceCtx* ctx_in,
                size_t ldc, size_t group_begin, size_t group_end) {
    const DeviceCtx* ctx = ctx_in;
    if (!ctx) {
        DeviceCtx* c = nullptr;
        if (int rc = get_device_ctx(&c)) return rc;
        ctx = c;
    }
    if (ldc == 0) ldc = N;
    // the view of the groups asked for: steps, blocks and row pointers are addressed absolutely, so a sub-range is
    // the same plan with its first group, first block-row and group count moved
    if (whole.tall) return launch_spmm_tall(whole, B, C, N, stream, ctx, ldc, group_begin, group_end);
    if (group_end > whole.n_groups) group_end = whole.n_groups;
    if (group_begin >= group_end) return SMAT_OK;
    const PlanView plan = plan_group_range(whole, group_begin, group_end);
    const size_t nb_rows = plan.brow_end - plan.brow_begin;
    if (nb_rows == 0 || N == 0) return SMAT_OK;
    if (plan.nnzb == 0) {
        if (ldc == N) {
            const size_t n16 = nb_rows * 16 * N * 2 / 16;
            zero_rows_kernel<<<ctx->sm_count * 4, 256, 0, stream>>>(reinterpret_cast<uint4*>(C), n16);
            count_launch();
            SMAT_CUDA_TRY(cudaGetLastError());
        } else {
            SMAT_CUDA_TRY(cudaMemset2DAsync(C, ldc * 2, 0, N * 2, nb_rows * 16, stream));
        }
        return SMAT_OK;
    }
    // Item width: 256 columns (every A block then feeds two MMAs; one accumulator buffer, so the epilogue is not
    // overlapped) or 128.  Wide items need C that wide and long items (many blocks, many steps: short items are
    // dominated by the epilogue, which only narrow items overlap); between the two the estimated time decides:
    // rounds of items over the SMs -- the last round counting 1/P when its items are cut into P segments -- times
    // the measured cost of an item (a wide one costs 1.95 narrow ones).
    const bool split = plan.fix_scratch != nullptr;
    const size_t sms = (size_t)ctx->sm_count;
    // steps per item: the average when the plan knows its step count, else a bound (one per block, one per 64 columns)
    size_t est_steps = plan.nnzb / plan.n_groups;
    if (plan.K / 64 < est_steps) est_steps = plan.K / 64;
    if (plan.total_steps) est_steps = plan.total_steps / plan.n_groups;
    auto tail_parts = [&](size_t items) { return tail_parts_for(items, sms, split, est_steps); };
    auto rounds = [&](size_t items, bool wide) { return rounds_for(items, sms, split, est_steps, wide); };
    // a plan's list of groups per CTA covers all its groups and was made for one CTA per SM
    const bool listed = plan.sched_list != nullptr && plan.sched_ctas == ctx->sm_count && plan.n_groups == whole.n_groups;
    const bool balanced = !listed && split && plan.balanced;
    int variant = g_spmm_variant;
    if (variant == 0 && (balanced || listed)) variant = (N >= 256 && plan.nnzb / plan.n_groups >= 256 && est_steps >= 64) ? 3 : 1;
    if (variant == 0) {
        variant = 1;
        if (N >= 256 && plan.nnzb / plan.n_groups >= 256 && est_steps >= 64 &&
            kWideItemCost * rounds(plan.n_groups * ((N + 255) / 256), true) < rounds(plan.n_groups * ((N + 127) / 128), false))
            variant = 3;
    }
    const size_t NTI = variant == 3 ? 256 : 128;
    const uint32_t panel_rows = (uint32_t)(N < NTI ? N : NTI);
    CUtensorMap mapB;
    if (int rc = encode_tensor_map_2d_f16(&mapB, B, plan.K, N, plan.K * 2, 64, panel_rows, 128, 0)) return rc;
    CUtensorMap mapC;  // C as the epilogue stores it: boxes of 16 rows x 128 columns (N columns when C is narrower)
    if (int rc = encode_tensor_map_2d_f16(&mapC, C, N, nb_rows * 16, ldc * 2, (uint32_t)(N < 128 ? N : 128), 16, 0, 0)) return rc;
    const int n_tiles = (int)((N + NTI - 1) / NTI);
    const size_t n_items = plan.n_groups * (size_t)n_tiles;
    if (n_items > (size_t)INT_MAX) return fail(SMAT_ERR_RANGE, "too many work items (%zu)", n_items);
    // one CTA per SM; fewer only when there are fewer items than SMs and they are not cut
    const int parts = (balanced || listed) ? 1 : (int)tail_parts(n_items);
    const int grid = (int)((balanced || listed || parts > 1 || n_items > sms) ? sms : n_items);
    const int n_full = (int)(n_items / (size_t)grid * (size_t)grid);
    // MMA-issuing warps: 8 own two accumulator rows each; plans whose steps are nearly full use fewer warps with more
    // rows each, so that a column of vertically adjacent blocks is multiplied by one MMA (N up to 256) instead of eight
    int nm = NM;
    if (plan.total_steps) {
        const size_t per_step = plan.nnzb / plan.total_steps;
        nm = per_step >= 40 ? 1 : per_step >= 20 ? 2 : NM;
    }
    if (const char* ev = std::getenv("SMAT_MMA_WARPS")) {  // tuning knob
        const int v = std::atoi(ev);
        if (v == 1 || v == 2 || v == 4 || v == 8) nm = v;
    }
    int pf = 0;  // L2 prefetch (see the top of the file)
    if (const char* ev = std::getenv("SMAT_L2_PREFETCH")) pf = std::atoi(ev) != 0;  // tuning knob
    auto launch = [&](auto kernel, uint32_t smem_bytes) -> int {
        SMAT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
        kernel<<<grid, kThreads, smem_bytes, stream>>>(
            mapB, mapC, reinterpret_cast<const uint8_t*>(plan.packed), reinterpret_cast<const uint4*>(plan.steps), plan.gsp,
            plan.rowptr, reinterpret_cast<__half*>(C), (int)plan.brow_begin, (int)plan.brow_end, (int)plan.rg, (int)N, n_tiles,
            (int)n_items, (int)plan.n_groups, parts, panel_rows * 128u, plan.fix_scratch, ctx->d_status, ldc,
            listed ? plan.sched_off : nullptr, listed ? plan.sched_list : nullptr, nm, pf);
        count_launch();
        SMAT_CUDA_TRY(cudaGetLastError());
        return SMAT_OK;
    };
    auto launch_sched = [&](auto sched, auto cap) -> int {
        constexpr int SCHED = decltype(sched)::value, CAP = decltype(cap)::value;
        if (variant == 3) return launch(spmm_bcsr_tc_kernel<false, 2, SCHED, CAP>, Cfg<2, CAP>::SMEM_BYTES);
        if (variant == 2) return launch(spmm_bcsr_tc_kernel<true, 1, SCHED, CAP>, Cfg<1, CAP>::SMEM_BYTES);
        return launch(spmm_bcsr_tc_kernel<false, 1, SCHED, CAP>, Cfg<1, CAP>::SMEM_BYTES);
    };
    auto launch_cap = [&](auto sched) -> int {
        if (plan.cap == (size_t)kPlanBlocksPerStepDense) return launch_sched(sched, std::integral_constant<int, kPlanBlocksPerStepDense>{});
        return launch_sched(sched, std::integral_constant<int, kPlanBlocksPerStep>{});
    };
    if (plan.cap != (size_t)kPlanBlocksPerStep && plan.cap != (size_t)kPlanBlocksPerStepDense)
        return fail(SMAT_ERR_BAD_ARG, "plan with %zu blocks per step: no kernel for it", plan.cap);
    int rc;
    if (listed) rc = launch_cap(std::integral_constant<int, 1>{});
    else if (balanced) rc = launch_cap(std::integral_constant<int, 2>{});
    else rc = launch_cap(std::integral_constant<int, 0>{});
    if (rc != SMAT_OK) return rc;
    if (balanced) {
        if (grid < 2) return SMAT_OK;
        if (variant == 3)
            sum_split_items_kernel<2><<<grid - 1, dim3(128, 4), 0, stream>>>(plan.fix_scratch, plan.gsp, reinterpret_cast<__half*>(C),
                                                                            (int)plan.brow_begin, (int)plan.brow_end, (int)plan.rg, (int)N,
                                                                            n_tiles, (int)plan.n_groups, grid, ldc);
        else
            sum_split_items_kernel<1><<<grid - 1, dim3(128, 4), 0, stream>>>(plan.fix_scratch, plan.gsp, reinterpret_cast<__half*>(C),
                                                                            (int)plan.brow_begin, (int)plan.brow_end, (int)plan.rg, (int)N,
                                                                            n_tiles, (int)plan.n_groups, grid, ldc);
        count_launch();
        SMAT_CUDA_TRY(cudaGetLastError());
        return SMAT_OK;
    }
    if (parts == 1) return rc;
    return launch_sum_cut_items(variant == 3, (int)n_items - n_full, plan.fix_scratch, C, (int)plan.brow_begin, (int)plan.brow_end,
                                (int)plan.rg, (int)N, n_tiles, n_full, parts, ldc, stream);
}

}  // namespace smat
