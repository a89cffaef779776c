// Block-sparse SpMM for NVIDIA B200 (sm_100a), "tall" variant: work items of up to 24 block-rows x 128 columns of C,
// B panels read by the MMAs from TENSOR memory.  Same boundary, layouts and transposed mapping as spmm_sm100.cu
// (replaces mmaCBTKernel, src/cuda_hgemm/src/mma/mmaCBT.cu:13-88); chosen by the plan for matrices whose groups hold
// several blocks per four block-columns without being dense (a block-sparse weight matrix, a reordered random matrix).
//
// Why a second kernel.  Measured on B200 (148 SMs, 1965 MHz):
//   * tcgen05.mma M128 x N16 x K16 with the "A" operand (the 128 n x 16 k panel slice of B) in SHARED memory takes
//     ~39 cycles per SM -- the 4 KB slice crosses the shared-memory operand port once per 16x16 block -- against ~9
//     cycles with the slice in TENSOR memory ([tmem] operand; N = 32: ~9, N = 64: 32).  A 16-row work item of the
//     shared-memory kernel is bound by exactly that port.
//   * Streaming the panels L2 -> shared memory sustains ~70 bytes/cycle/SM (19-20 TB/s over the chip).  The panel
//     traffic of a launch is (block-rows / rows per group) x K x N x 2 bytes, so taller groups cut it in proportion;
//     tensor memory (512 columns) holds 24 accumulators of 16 columns plus a ring of four panels.
//   * Issuing a tcgen05.mma costs a thread ~15 cycles when its operand registers are left alone, ~90 more when one
//     of them is written again right away, and each branch or register operation around it a few cycles more; with
//     12 warps issuing at once the tensor pipe (9 cycles per MMA) is what each of them waits for.  tcgen05.commit and
//     a barrier wait cost the issuing thread ~100-200 cycles each, the tensor pipe nothing.  So 12 warps issue, each
//     owning two accumulator rows (all MMAs into one accumulator come from one thread, in order: results do not
//     depend on warp timing), the steps are handed over two at a time, and the plan lists each warp's MMAs of a pair
//     of steps so that the warp works the list off in straight-line code.
//
// Pipeline per step (four block-columns of a group), all hand-overs by mbarriers, every wait bounded:
//   loader warps (4, one thread each, every 4th step): TMA box {64 k, 128 n} -> panel slot (6 slots), bulk copy of the
//     step's packed A blocks -> block slot (10 slots) and, with the first step of a pair, of the pair's MMA lists;
//   copier warps (4, one thread each, every 4th step): wait panel + blocks, tcgen05.cp the non-empty sub-columns
//     shared -> tensor memory ring, commit -> cp_done of the step's pair.  That frees the shared panel slot for the
//     loader and tells the MMA warps that panels AND blocks of the pair are in place;
//   MMA warps (one per two accumulator rows): per PAIR of steps wait cp_done once, read their list, issue, commit ->
//     step_done (a plain arrive when the warp had no block in the pair); step_done frees the block slots (loader)
//     and the tensor-memory panel slots (copier) of the pair;
//   epilogue warps (8 = two per tensor-memory lane quarter, alternating block-rows): tcgen05.ld -> zero the
//     accumulator -> fp16 -> 4-byte stores to C; cut items write fp32 partial tiles.
// Groups of at most 16 or 20 block-rows use fewer accumulators and a longer tensor-memory panel ring (8 or 6 slots
// instead of 4).  Scheduling is the round-robin-with-cut-last-round scheme of spmm_sm100.cu (SegGen<0>); the plan
// pads every group to an even number of steps and items are cut at even positions, so a pair never spans two items.
// What bounds the kernel on the block-sparse layer it was written for: every step moves 16 KB of panel and ~10 KB of
// blocks from L2 to the SM, and 148 SMs doing that every ~600 cycles is ~12 TB/s, two thirds of what L2 delivered
// to a pure streaming kernel (19-20 TB/s); the rest is latency of the chain copy -> MMAs -> slot release.
#include <cuda_fp16.h>
#include <limits.h>
#include <stdlib.h>

#include <cstdlib>

#include "ptx_sm100.cuh"
#include "smat_internal.h"
#include "spmm_sched.cuh"

namespace smat {

using namespace ptx;

namespace {

constexpr int NLW = 4;           // panel-loader warps, and as many block-loader warps
constexpr int LW = 2 * NLW;      // loader warps in all
constexpr int NCW = 4;           // copier warps
constexpr int NEW = 8;           // epilogue warps
constexpr uint32_t PS = 6;                                   // panel slots in shared memory (a slot is free once copied to tensor memory)
constexpr uint32_t BS = 10;                                  // block slots (held until the step's MMAs have completed)
constexpr uint32_t PANEL_BYTES = 128 * 64 * 2;               // 128 n x 64 k fp16
constexpr uint32_t BLK_SLOT_BYTES = kTallBlocksPerStep * 512;
constexpr uint32_t OFF_PANEL = 0;
constexpr uint32_t OFF_BLK = OFF_PANEL + PS * PANEL_BYTES;
constexpr uint32_t META_BYTES = 256;                          // per pair of steps: the MMA lists of the 12 issuing warps
constexpr uint32_t OFF_META = OFF_BLK + BS * BLK_SLOT_BYTES;
constexpr uint32_t OFF_SUBS = OFF_META + (BS / 2) * META_BYTES;  // per step: its non-empty sub-columns (written by the loader)
constexpr uint32_t OFF_BAR = OFF_SUBS + BS * 8;
// A thread that waits on an mbarrier by parity must see every phase of it.  Loader j and copier j handle the steps
// st = j (mod 4), so a "full" barrier ring is as long as lcm(slots, 4): barrier st % ring then always belongs to
// the same loader and the same copier.  The per-pair rings (8 barriers) are visited by a loader or copier at every
// other pair, i.e. each barrier of its parity class once per 8 pairs: once per phase.
constexpr uint32_t FP = 12;                                   // full_p ring: lcm(PS, 4)
constexpr uint32_t FB = 20;                                   // full_b ring: lcm(BS, 4)
constexpr uint32_t NPAIR = 8;                                 // cp_done / step_done rings (pairs of steps)
constexpr uint32_t N_BARS = FP + FB + NPAIR + NPAIR + 2;
constexpr uint32_t OFF_MISC = OFF_BAR + N_BARS * 8;
constexpr uint32_t SMEM_BYTES = OFF_MISC + 16 + 1024;        // slack for the manual 1024-byte alignment
constexpr uint32_t TMEM_ACC = 0;                             // accumulators: one per block-row, 16 columns each
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
static_assert(NLW == 4 && NCW == 4 && FP % PS == 0 && FP % 4 == 0 && FB % BS == 0 && FB % 4 == 0 && PS % 2 == 0 && BS % 2 == 0 &&
                  NPAIR % 2 == 0 && NPAIR > BS / 2,
              "the barrier phase arithmetic below assumes these");
static_assert(kTallRows * 16 * 128 <= kFixSlotFloats, "a partial tile must fit a scratch slot");

// Shape of a work item: TRG block-rows (accumulators), two of them per MMA-issuing warp.  What tensor memory the
// accumulators leave holds the panel ring (32 columns a slot, at most 8 slots).
template <int TRG>
struct Shape {
    static constexpr int NMW = TRG / 2;
    static constexpr int kThreads = (LW + NCW + NMW + NEW) * 32;
    static constexpr uint32_t TMEM_PANELS = TRG * 16;
    static constexpr uint32_t TS_ = (512 - TRG * 16) / 32 < 8 ? (512 - TRG * 16) / 32 : 8;
    static_assert(TRG % 2 == 0 && TRG <= kTallRows && kThreads <= 1024, "shape");
    static_assert(TS_ >= 4 && TS_ % 2 == 0 && TS_ / 2 < NPAIR && TMEM_PANELS + TS_ * 32 <= 512, "tensor-memory budget: whole pairs of panel slots");
};

struct TallStep {
    int live;
    int tile;
    int idx;      // index of the step in the plan
    uint32_t st;  // its position in this CTA's sequence
    uint4 a;      // {element column, packed position (256-byte units), blocks, non-empty sub-columns}
};

template <int TRG>
__global__ void __launch_bounds__((Shape<TRG>::kThreads), 1)
spmm_bcsr_tall_kernel(const __grid_constant__ CUtensorMap mapB, const uint8_t* __restrict__ packed,
                      const uint4* __restrict__ steps, const uint4* __restrict__ winfo, const int* __restrict__ gsp,
                      const int* __restrict__ rowptr,
                      __half* __restrict__ C, size_t ldc, int brow_begin, int brow_end, int rg, int N, int n_tiles, int n_items,
                      int tail_parts, uint32_t panel_bytes, float* __restrict__ fix_scratch, int* status, int pf) {
    constexpr int NMW = Shape<TRG>::NMW;
    constexpr uint32_t TS_ = Shape<TRG>::TS_, TMEM_PANELS = Shape<TRG>::TMEM_PANELS;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar0 = base + OFF_BAR;
    auto full_p = [&](uint32_t s) { return bar0 + 8 * s; };
    auto full_b = [&](uint32_t s) { return bar0 + 8 * (FP + s); };
    // The MMA warps are handed the steps two at a time (pair p = steps 2p, 2p + 1 of the CTA's sequence, whatever
    // work items they belong to): measured, a barrier wait or a commit costs the issuing thread about as much as an
    // MMA (~100 cycles), so one of each per step and warp would hold the whole pipeline back.
    auto cp_done = [&](uint32_t p) { return bar0 + 8 * (FP + FB + p); };            // both panels of pair p (mod NPAIR) copied
    auto step_done = [&](uint32_t p) { return bar0 + 8 * (FP + FB + NPAIR + p); };  // all MMAs of pair p (mod NPAIR) completed
    const uint32_t acc_full = bar0 + 8 * (FP + FB + 2 * NPAIR), acc_empty = acc_full + 8;
    const uint32_t tmem_slot = base + OFF_MISC;
    const uint32_t abort_addr = base + OFF_MISC + 4;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
#ifdef SMAT_PROFILE  // development aid: cycles this thread spends in each kind of wait (mbarrier.try_wait may itself suspend it)
    const long long t_kernel0 = clock64();
    unsigned int prof_c[16] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
    __shared__ unsigned int stamp_cp[8], stamp_mma[8];  // clock of the last commit of a pair's copies / MMAs
    if (threadIdx.x < 8) stamp_cp[threadIdx.x] = stamp_mma[threadIdx.x] = (unsigned int)clock();
    long long prof_t = 0;
#define PROF_MARK(code)                                          \
    do {                                                         \
        const long long t_ = clock64();                          \
        if (code) prof_c[code] += (unsigned int)(t_ - prof_t);   \
        prof_t = t_;                                             \
    } while (0)
#define TWAIT(bar, par, code)                                    \
    do {                                                         \
        const long long t_ = clock64();                          \
        wait_bar(bar, par, abort_addr, status, code);            \
        prof_c[code] += (unsigned int)(clock64() - t_);          \
    } while (0)
#else
#define TWAIT(bar, par, code) wait_bar(bar, par, abort_addr, status, code)
#define PROF_MARK(code)
#endif
    const int n_full = n_items / (int)gridDim.x * (int)gridDim.x;  // items of the complete rounds
    auto make_gen = [&]() {
        SegGen<0> sg;
        sg.gsp = gsp; sg.n_tiles = n_tiles; sg.n_items = n_items; sg.n_ctas = (int)gridDim.x; sg.cta = (int)blockIdx.x;
        sg.item = (int)blockIdx.x; sg.n_full = n_full; sg.P = tail_parts; sg.tail_done = false;
        sg.quantum = 2;  // groups hold an even number of steps (the plan pads them) and are cut at even positions
        sg.flat.gsp = gsp; sg.flat.n_tiles = n_tiles; sg.flat.n_groups = 0; sg.flat.total = 0; sg.g = 0;
        sg.p = sg.p_begin = sg.p_end = 0;
        sg.list = nullptr; sg.li = sg.li_end = 0; sg.lt = 0;
        return sg;
    };

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < FP; s++) mbar_init(full_p(s), 1);
        for (uint32_t s = 0; s < FB; s++) mbar_init(full_b(s), 1);
        for (uint32_t s = 0; s < NPAIR; s++) { mbar_init(cp_done(s), 4); mbar_init(step_done(s), NMW); }  // cp_done: per step a commit and an arrive
        mbar_init(acc_full, NMW);
        mbar_init(acc_empty, NEW);
        st_shared_u32(abort_addr, 0);
        fence_barrier_init();
        fence_proxy_async();
        prefetch_tensormap(&mapB);
    }
    if (warp == LW) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ld_shared_u32(tmem_slot);
    if (warp < 4) {  // all accumulators start at zero (later the epilogue re-zeroes what it reads)
#pragma unroll 4
        for (uint32_t c = 0; c < (uint32_t)TRG * 16; c += 16) tmem_zero_x16(tmem_base + ((uint32_t)(warp * 32) << 16) + TMEM_ACC + c);
        tmem_st_wait();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    if (warp < LW) {
        // ---------------- loader warps: panel loader j and block loader j take the steps j, j + NLW, ... ----------------
        // (two threads per step, so that neither waits for the other's slot and each has half the work per step)
        if (lane == 0) {
            const bool panels = warp < NLW;
            const int j = warp % NLW;
            SegGen<0> sg = make_gen();
            Seg cs;
            bool have = sg.next(cs);
            uint32_t h_st0 = 0, h_next = (uint32_t)j;
            constexpr int U = 4;  // step records in flight per loader (their descriptors are requested U positions ahead)
            constexpr int PF = 2;  // records ahead (of this loader) whose data is prefetched into L2 when the launch asks for it
            TallStep rec[U];
            auto gen = [&](TallStep& r) {
                while (have && h_next >= h_st0 + (uint32_t)(cs.k1 - cs.k0)) {
                    h_st0 += (uint32_t)(cs.k1 - cs.k0);
                    have = sg.next(cs);
                }
                r.live = have;
                if (have) {
                    r.tile = cs.item % n_tiles;
                    r.st = h_next;
                    r.idx = cs.gs + cs.k0 + (int)(h_next - h_st0);
                    r.a = __ldg(steps + r.idx);
                    h_next += NLW;
                }
            };
            auto prefetch = [&](const TallStep& r) {  // HBM latency is hidden in L2: fetched PF records ahead of the copies
                if (pf && r.live && r.a.z) {
                    if (panels) tma_prefetch_l2_2d(&mapB, (int)r.a.x, r.tile * 128);
                    else bulk_prefetch_l2(packed + (size_t)r.a.y * 256, r.a.z * 512u);
                }
            };
#pragma unroll
            for (int a = 0; a < U; a++) gen(rec[a]);
#pragma unroll
            for (int a = 0; a < PF; a++) prefetch(rec[a]);
            bool more = true;
            while (more) {
#pragma unroll
                for (int a = 0; a < U; a++) {
                    TallStep& r = rec[a];
                    if (!r.live) { more = false; break; }
                    const uint32_t ps = r.st % PS, bs = r.st % BS, pi = r.st >> 1;
                    const uint32_t a_bytes = r.a.z * 512u;  // 0: a step that only pads its group to an even count
                    if (panels) {
                        // the panel's slot is free once the copy of the step PS positions back (pair pi - PS / 2) has left it
                        if (r.st >= PS) TWAIT(cp_done((pi - PS / 2) % NPAIR), ((pi - PS / 2) / NPAIR) & 1, 1);
                        if (a_bytes) {
                            mbar_arrive_expect_tx(full_p(r.st % FP), panel_bytes);
                            tma_load_2d(base + OFF_PANEL + ps * PANEL_BYTES, &mapB, (int)r.a.x, r.tile * 128, full_p(r.st % FP));
                        } else {
                            mbar_arrive(full_p(r.st % FP));  // no panel: the phase completes at once
                        }
                    } else {
                        // the slot of the blocks is free once the MMAs of the step BS positions back (pair pi - BS / 2) have completed
                        if (r.st >= BS) TWAIT(step_done((pi - BS / 2) % NPAIR), ((pi - BS / 2) / NPAIR) & 1, 2);
                        st_shared_u32(base + OFF_SUBS + bs * 8, r.a.w);  // for the copier; ordered before its wait by the arrive below
                        const uint32_t m_bytes = (r.st & 1u) ? 0u : META_BYTES;  // the pair's lists travel with its first step
                        if (a_bytes + m_bytes) mbar_arrive_expect_tx(full_b(r.st % FB), a_bytes + m_bytes);
                        else mbar_arrive(full_b(r.st % FB));
                        if (m_bytes)
                            bulk_load(base + OFF_META + (bs >> 1) * META_BYTES, winfo + 16 * (size_t)(r.idx >> 1), META_BYTES, full_b(r.st % FB));
                        if (a_bytes) bulk_load(base + OFF_BLK + bs * BLK_SLOT_BYTES, packed + (size_t)r.a.y * 256, a_bytes, full_b(r.st % FB));
                    }
                    prefetch(rec[(a + PF) % U]);
                    gen(r);
                }
            }
        }
        __syncwarp();
    } else if (warp < LW + NCW) {
        // ------------------------------ copier j: steps j, j + NCW, ... ------------------------------
        // The whole warp runs the loop converged and one elected lane issues, like the MMA warps: operands a
        // tcgen05 instruction gets from warp-uniform values cost its thread far less than ones from a lone lane.
        {
            const uint32_t j = (uint32_t)__shfl_sync(0xffffffffu, warp - LW, 0);
            const bool leader = elect_one();
            uint32_t total = 0;  // steps of this CTA
            {
                SegGen<0> sg = make_gen();
                Seg cs;
                while (sg.next(cs)) total += (uint32_t)(cs.k1 - cs.k0);
            }
            total = (uint32_t)__shfl_sync(0xffffffffu, total, 0);
            for (uint32_t st = j; st < total; st += NCW) {
                const uint32_t ps = st % PS, bs = st % BS, pi = st >> 1;
                // what is usually there already first: blocks and panel wait in shared memory for a tensor-memory slot,
                // which is free once the MMAs of the step TS_ positions back (pair pi - TS_ / 2) have completed; only
                // the copies follow that
                TWAIT(full_b(st % FB), (st / FB) & 1, 4);
                const uint32_t subs_l = ld_shared_u32(base + OFF_SUBS + bs * 8);  // non-empty sub-columns
                const uint32_t subs = __ballot_sync(0xffffffffu, (subs_l >> lane) & 1u);
                const uint64_t pdesc = smem_desc_k_sw128(base + OFF_PANEL + ps * PANEL_BYTES);
                const uint32_t tdst = tmem_base + TMEM_PANELS + (st % TS_) * 32;
                TWAIT(full_p(st % FP), (st / FP) & 1, 3);
                if (pi >= TS_ / 2) TWAIT(step_done((pi - TS_ / 2) % NPAIR), ((pi - TS_ / 2) / NPAIR) & 1, 5);
#ifdef SMAT_PROFILE
                if (pi >= TS_ / 2) prof_c[13] += (unsigned int)clock() - *(volatile unsigned int*)&stamp_mma[(pi - TS_ / 2) % 8];
                const unsigned int t_cp0 = (unsigned int)clock();
#endif
                tc_fence_after();
                if (leader) {
#ifndef SMAT_TALL_NOCP
                    if (subs & 1u) tc_cp_128x256b(tdst, pdesc);
                    if (subs & 2u) tc_cp_128x256b(tdst + 8, pdesc + 2);
                    if (subs & 4u) tc_cp_128x256b(tdst + 16, pdesc + 4);
                    if (subs & 8u) tc_cp_128x256b(tdst + 24, pdesc + 6);
#endif
                    tc_commit(cp_done(pi % NPAIR));
                    // A plain arrive beside the commit's: it is ordered after this thread's wait for the blocks and
                    // lists of the step, so whoever passes cp_done may read them (the MMA warps wait for nothing else).
                    mbar_arrive(cp_done(pi % NPAIR));
                }
#ifdef SMAT_PROFILE
                if (leader) atomicMax(&stamp_cp[pi % 8], (unsigned int)clock());
                prof_c[14] += (unsigned int)clock() - t_cp0;
#endif
            }
        }
        __syncwarp();
    } else if (warp < LW + NCW + NMW) {
        // ------------------------------ MMA warp m: accumulator rows 2m, 2m + 1 ------------------------------
        // The whole warp runs the loop converged and one elected lane issues.  Every operand of a tcgen05.mma must
        // be a value the compiler knows to be warp-uniform (the instruction reads uniform registers): measured, the
        // same loop run by a single lane on values loaded from shared memory is 10 % slower over the whole kernel.
        // So the list words, read from shared memory, are turned into ballots before anything is derived from them.
        {
            const uint32_t m = (uint32_t)__shfl_sync(0xffffffffu, warp - LW - NCW, 0);
            const bool leader = elect_one();
            const uint32_t B_HI = (uint32_t)(smem_desc_k_sw32(0) >> 32);
            const uint32_t b_lo0 = (uint32_t)smem_desc_k_sw32(base + OFF_BLK);
            constexpr uint32_t IDESC16 = idesc_f16_f32(128, 16), IDESC32 = idesc_f16_f32(128, 32);
            const uint32_t acc_m = tmem_base + TMEM_ACC + 2u * m * 16u;  // this warp's two accumulators
            uint32_t st = 0, it = 0;
            SegGen<0> sg = make_gen();
            Seg cs;
            while (sg.next(cs)) {
                TWAIT(acc_empty, (it & 1) ^ 1, 6);
                tc_fence_after();
                // segments hold an even number of steps and start at an even position: a pair never spans two of them
                for (int k = cs.k0; k < cs.k1; k += 2, st += 2) {
                    const uint32_t pi = st >> 1, bs = st % BS;
                    PROF_MARK(0);
                    TWAIT(cp_done(pi % NPAIR), (pi / NPAIR) & 1, 7);
#ifdef SMAT_PROFILE
                    prof_c[12] += (unsigned int)clock() - *(volatile unsigned int*)&stamp_cp[pi % 8];
#endif
                    tc_fence_after();
                    // This warp's list for the pair: up to eight 16-bit entries, one per MMA (layout: tall_pair_kernel
                    // in plan.cu), their number in the top bits of the first word.  Measured: the branches and the
                    // register arithmetic around a tcgen05.mma cost the issuing thread far more than the instruction
                    // (~15 cycles), and writing an operand register of an MMA just issued stalls it ~90 cycles.  So
                    // the plan lists the MMAs, and the list is worked off in straight-line code entered at its length.
                    const uint4 l = ld_shared_v4(base + OFF_META + (bs >> 1) * META_BYTES + m * 16u);
                    uint32_t w[4];
                    w[0] = __ballot_sync(0xffffffffu, (l.x >> lane) & 1u);
                    w[1] = __ballot_sync(0xffffffffu, (l.y >> lane) & 1u);
                    w[2] = __ballot_sync(0xffffffffu, (l.z >> lane) & 1u);
                    w[3] = __ballot_sync(0xffffffffu, (l.w >> lane) & 1u);
                    const uint32_t tpanel = tmem_base + TMEM_PANELS + (st % TS_) * 32;
                    const uint32_t b_lo = b_lo0 + bs * (BLK_SLOT_BYTES >> 4);
                    const uint32_t count = w[0] >> 28;
                    PROF_MARK(9);
                    // operands of the first four entries (most lists are no longer) worked out here, where the warp is
                    // converged and the values stay in uniform registers; the elected lane's region below only issues
                    uint32_t od[4], oa[4], ob[4], oi[4];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const uint32_t e = (i & 1) ? (w[i >> 1] >> 16) : w[i >> 1];
                        od[i] = acc_m + ((e >> 5) & 16u);
                        oa[i] = tpanel + ((e >> 3) & 56u);
                        ob[i] = b_lo + (e & 63u) * 32u;
                        oi[i] = IDESC16 + ((e << 8) & (1u << 18));
                    }
#define SMAT_TALL_MMA(i)                                                                                               \
    {                                                                                                                  \
        if ((i) < 4) {                                                                                                 \
            mma_f16_ts_lohi(od[(i) & 3], oa[(i) & 3], ob[(i) & 3], B_HI, oi[(i) & 3], 1u);                             \
        } else {                                                                                                       \
            const uint32_t e = ((i) & 1) ? (w[(i) >> 1] >> 16) : w[(i) >> 1];                                          \
            mma_f16_ts_lohi(acc_m + ((e >> 5) & 16u), tpanel + ((e >> 3) & 56u), b_lo + (e & 63u) * 32u, B_HI,         \
                            IDESC16 + ((e << 8) & (1u << 18)), 1u);                                                    \
        }                                                                                                              \
    }
                    static_assert(IDESC32 == IDESC16 + (1u << 18), "the 32-column descriptor is the 16-column one plus bit 18");
                    // one region of the elected lane per pair (every separate `if (leader)` costs the warp a divergence
                    // and a reconvergence: one region instead of one per MMA was worth 7 % of the kernel's time)
                    if (leader) {
                        switch (count) {
                            case 8: SMAT_TALL_MMA(7) [[fallthrough]];
                            case 7: SMAT_TALL_MMA(6) [[fallthrough]];
                            case 6: SMAT_TALL_MMA(5) [[fallthrough]];
                            case 5: SMAT_TALL_MMA(4) [[fallthrough]];
                            case 4: SMAT_TALL_MMA(3) [[fallthrough]];
                            case 3: SMAT_TALL_MMA(2) [[fallthrough]];
                            case 2: SMAT_TALL_MMA(1) [[fallthrough]];
                            case 1: SMAT_TALL_MMA(0) tc_commit(step_done(pi % NPAIR)); break;
                            default: mbar_arrive(step_done(pi % NPAIR)); break;
                        }
#ifdef SMAT_PROFILE
                        atomicMax(&stamp_mma[pi % 8], (unsigned int)clock());
#endif
                    }
#undef SMAT_TALL_MMA
                    PROF_MARK(10);
                    PROF_MARK(11);
                }
                if (leader) tc_commit(acc_full);
                ++it;
            }
        }
        __syncwarp();
    } else {
        // ------------------------------ epilogue: tensor memory -> fp16 -> C ------------------------------
        const int e = warp - (LW + NCW + NMW);
        const int quarter = warp & 3;  // a warp may only read tensor-memory lanes [32 * (warp % 4), +32)
        const int grp = e >> 2;        // two groups of four warps; group g takes block-rows g, g + 2, ...
        const int et = quarter * 32 + lane;
        uint32_t it = 0;
        SegGen<0> sg = make_gen();
        Seg cs;
        for (; sg.next(cs); ++it) {
            const int g = cs.item / n_tiles, t = cs.item - g * n_tiles;
            const int r0 = brow_begin + g * rg;
            const int nrows = min(rg, brow_end - r0);
            const int lo = (lane < nrows) ? __ldg(rowptr + r0 + lane) : 0;
            const int hi = (lane < nrows) ? __ldg(rowptr + r0 + lane + 1) : 0;
            const uint32_t nonempty = __ballot_sync(0xffffffffu, hi > lo);
            const bool partial = cs.cut;
            float* part_dst = fix_scratch + (size_t)cs.slot * (size_t)kFixSlotFloats;
            if (lane == 0) TWAIT(acc_full, it & 1, 8);
            __syncwarp();
            tc_fence_after();
            int last_r = -1;  // last block-row this warp's group handles
            for (int r = grp; r < nrows; r += 2) last_r = r;
            if (last_r < 0) {  // nothing to read for this group: hand the accumulators back at once
                if (lane == 0) mbar_arrive(acc_empty);
            }
            for (int r = grp; r < nrows; r += 2) {
                uint32_t v[16];
                if ((nonempty >> r) & 1u) {
                    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + TMEM_ACC + (uint32_t)r * 16;
                    tmem_ld_x16(taddr, v);
                    tmem_ld_wait();
                    tmem_zero_x16(taddr);
                } else {
#pragma unroll
                    for (int i = 0; i < 16; i++) v[i] = 0u;
                }
                if (r == last_r) {
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty);
                }
                if (partial) {
                    float* dd = part_dst + ((size_t)r * 16) * 128 + et;
#pragma unroll
                    for (int i = 0; i < 16; i++) dd[(size_t)i * 128] = __uint_as_float(v[i]);
                    continue;
                }
                // lane pairs exchange halves: even lanes keep rows 0..7, odd lanes rows 8..15, each for the two adjacent
                // columns (n & ~1, n | 1) -> one 4-byte store per row, 128 contiguous bytes per warp
                const int n = t * 128 + et;
                const bool odd = lane & 1;
                __half* crow = C + ((size_t)(r0 - brow_begin + r) * 16 + (odd ? 8 : 0)) * ldc + (size_t)(n & ~1);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float keep = __uint_as_float(odd ? v[i + 8] : v[i]);
                    const float send = __uint_as_float(odd ? v[i] : v[i + 8]);
                    const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
                    const __half2 hh = odd ? __floats2half2_rn(recv, keep) : __floats2half2_rn(keep, recv);
                    if (n < N) *reinterpret_cast<__half2*>(crow + (size_t)i * ldc) = hh;
                }
            }
        }
    }

#ifdef SMAT_PROFILE
    if (lane == 0)
        for (int c = 1; c < 16; c++)
            if (prof_c[c]) atomicAdd(&g_wait_prof[c], (unsigned long long)prof_c[c]);
#endif
    tc_fence_before();
    __syncthreads();
#ifdef SMAT_PROFILE
    if (threadIdx.x == 0) { atomicAdd(&g_wait_prof[15], (unsigned long long)(clock64() - t_kernel0)); atomicAdd(&g_wait_prof[47], 1ull); }
#endif
    if (ld_shared_u32(abort_addr)) {
        // a wait ran out somewhere: give copies still in flight time to land before the CTA retires
        for (int i = 0; i < 64; i++) __nanosleep(1000);
    }
    if (warp == LW) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace

int launch_spmm_tall(const PlanView& whole, const void* B, void* C, size_t N, cudaStream_t stream, const DeviceCtx* ctx_in,
                     size_t ldc, size_t group_begin, size_t group_end) {
    const DeviceCtx* ctx = ctx_in;
    if (!ctx) {
        DeviceCtx* c = nullptr;
        if (int rc = get_device_ctx(&c)) return rc;
        ctx = c;
    }
    if (ldc == 0) ldc = N;
    if (!whole.tall || whole.rg > (size_t)kTallRows) return fail(SMAT_ERR_BAD_ARG, "not a tall plan");
    if (group_end > whole.n_groups) group_end = whole.n_groups;
    if (group_begin >= group_end) return SMAT_OK;
    const PlanView plan = plan_group_range(whole, group_begin, group_end);
    const size_t nb_rows = plan.brow_end - plan.brow_begin;
    if (nb_rows == 0 || N == 0) return SMAT_OK;
    if (plan.fix_scratch == nullptr || plan.winfo == nullptr) return fail(SMAT_ERR_BAD_ARG, "incomplete tall plan");
    const size_t sms = (size_t)ctx->sm_count;
    const uint32_t panel_rows = (uint32_t)(N < 128 ? N : 128);
    CUtensorMap mapB;
    if (int rc = encode_tensor_map_2d_f16(&mapB, B, plan.K, N, plan.K * 2, 64, panel_rows, 128, 0)) return rc;
    const int n_tiles = (int)((N + 127) / 128);
    const size_t n_items = plan.n_groups * (size_t)n_tiles;
    if (n_items > (size_t)INT_MAX) return fail(SMAT_ERR_RANGE, "too many work items (%zu)", n_items);
    size_t est_steps = plan.total_steps ? plan.total_steps / plan.n_groups : plan.K / 64;
    const int parts = (int)tail_parts_for(n_items, sms, true, est_steps);
    const int grid = (int)((parts > 1 || n_items > sms) ? sms : n_items);
    const int n_full = (int)(n_items / (size_t)grid * (size_t)grid);
    int pf = 0;  // L2 prefetch: measured to make no difference here, and it costs copy-engine time
    if (const char* ev = std::getenv("SMAT_L2_PREFETCH")) pf = std::atoi(ev) != 0;  // tuning knob
    auto launch = [&](auto kernel, int threads) -> int {
        SMAT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
        kernel<<<grid, threads, SMEM_BYTES, stream>>>(
            mapB, reinterpret_cast<const uint8_t*>(plan.packed), reinterpret_cast<const uint4*>(plan.steps),
            reinterpret_cast<const uint4*>(plan.winfo), plan.gsp, plan.rowptr, reinterpret_cast<__half*>(C), ldc, (int)plan.brow_begin,
            (int)plan.brow_end, (int)plan.rg, (int)N, n_tiles, (int)n_items, parts, panel_rows * 128u, plan.fix_scratch, ctx->d_status, pf);
        return SMAT_OK;
    };
    // the smallest shape that holds the plan's groups: fewer accumulators leave tensor memory for more panel slots
    if (plan.rg <= 16) {
        if (int rc = launch(spmm_bcsr_tall_kernel<16>, Shape<16>::kThreads)) return rc;
    } else if (plan.rg <= 20) {
        if (int rc = launch(spmm_bcsr_tall_kernel<20>, Shape<20>::kThreads)) return rc;
    } else {
        if (int rc = launch(spmm_bcsr_tall_kernel<24>, Shape<24>::kThreads)) return rc;
    }
    count_launch();
    SMAT_CUDA_TRY(cudaGetLastError());
    if (parts == 1) return SMAT_OK;
    return launch_sum_cut_items(false, (int)n_items - n_full, plan.fix_scratch, C, (int)plan.brow_begin, (int)plan.brow_end,
                                (int)plan.rg, (int)N, n_tiles, n_full, parts, ldc, stream);
}

#ifdef SMAT_PROFILE
extern "C" int smat_debug_tall_profile(unsigned long long* out64, int reset) {
    if (out64) cudaMemcpyFromSymbol(out64, g_wait_prof, sizeof(g_wait_prof));
    if (reset) { unsigned long long z[64] = {}; cudaMemcpyToSymbol(g_wait_prof, z, sizeof(z)); }
    return 0;
}
#endif

}  // namespace smat
