// Multiplication plan: the walk order of the SpMM kernel, computed on the device from the BCSR
// structure.
//
// For every group of 16 consecutive block-rows the kernel visits the group's block-columns in
// ascending order, four block-columns ("quad") at a time; per visited quad ("step") it needs the
// quad's column, which (sub-column, row) positions hold a block (a 64-bit mask) and the indices of
// those blocks.  Quads holding more than kPlanBlocksPerStep blocks are cut into several steps.
// The reference kernel has no such structure: it launches one CTA per (block-row, 8 columns of C)
// and walks bcsrColIdx directly (src/cuda_hgemm/src/mma/mmaCBT.cu:38-43), re-fetching the same B
// slab for every block-row that shares a block-column.
//
// Build: one CTA (16 warps) per group, warp w owns block-row w of the group.  Block-columns are
// processed in windows of 16384; inside a window a shared word per block-column collects the row
// mask (atomicOr), block-wide prefix sums number the steps and the blocks, then every block
// scatters its own index into the (group, column, row) order.  The number of steps per group is
// counted first (same pass without the scatter) and scanned.
#include <cuda_fp16.h>

#include <new>

#include <cstdio>
#include <cstdlib>
#include <vector>
#include <utility>
#include <queue>
#include <algorithm>

#include "smat_internal.h"

namespace smat {
namespace {

constexpr int RG = kPlanRowsPerGroup;
constexpr int kPlanThreads = RG * 32;
constexpr int kWindow = 16384;  // block-columns per pass: 64 KB of masks + 64 KB of block prefixes

// Fills masks[0..kWindow) for block-columns [w0, w0 + kWindow) of the group; cursor[] (one per warp,
// kept by lane 0 semantics via registers) walks each row once over all windows.
// A block column below the window start (columns not ascending, or negative) or beyond the matrix is not marked; the
// status word then tells the host that the structure is inconsistent.
template <int THREADS = kPlanThreads>
__device__ __forceinline__ void mark_window(const int* __restrict__ colidx, int& cur, int end, int w0, int Kb, uint32_t* masks,
                                            int warp, int lane, int* status) {
    for (int i = threadIdx.x; i < kWindow; i += THREADS) masks[i] = 0u;
    __syncthreads();
    // every lane keeps the same `cur`; lanes stride over the row until the window ends
    for (;;) {
        const int j = cur + lane;
        int cb = (j < end) ? (__ldg(colidx + j) >> 4) : INT_MAX;
        if (j < end && cb >= Kb) {  // beyond the last block-column: consume it without marking
            if (status) atomicCAS(status, 0, kStatusBadColumns);
            cb = w0 - 1;
        }
        const bool in = cb < w0 + kWindow;
        if (in && cb >= w0) atomicOr(&masks[cb - w0], 1u << warp);
        else if (in && status) atomicCAS(status, 0, kStatusBadColumns);
        const uint32_t b = __ballot_sync(0xffffffffu, in);
        cur += __popc(b);
        if (b != 0xffffffffu) break;
    }
    __syncthreads();
}

// True when row pointers [brow_begin, brow_end] cannot belong to a matrix of nnzb blocks (checked by every thread on the two
// ends; a dip in between shows up as a block-row whose end lies before its start and contributes nothing).
__device__ __forceinline__ bool range_is_bad(const int* __restrict__ rowptr, int brow_begin, int brow_end, int nnzb) {
    const int first = __ldg(rowptr + brow_begin), last = __ldg(rowptr + brow_end);
    return first < 0 || last < first || last > nnzb;
}

// Block-wide exclusive scan of one int per thread; returns the exclusive prefix, *total gets the sum.
template <int THREADS = kPlanThreads>
__device__ __forceinline__ int block_exclusive_scan(int v, int* total, int* sh) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += t;
    }
    if (lane == 31) sh[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = lane < (THREADS >> 5) ? sh[lane] : 0;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, w, d);
            if (lane >= d) w += t;
        }
        sh[32 + lane] = w;  // inclusive warp totals
    }
    __syncthreads();
    const int before = warp ? sh[32 + warp - 1] : 0;
    *total = sh[32 + (THREADS >> 5) - 1];
    __syncthreads();
    return before + inc - v;
}

template <bool FILL>
__global__ void __launch_bounds__(kPlanThreads)
plan_kernel(const int* __restrict__ rowptr, const int* __restrict__ colidx, int brow_begin, int brow_end, int rg, int CAP, int Kb,
            int n_groups, int* __restrict__ gsp, uint4* __restrict__ steps, int* __restrict__ blk, int nnzb, int* status) {
    extern __shared__ uint32_t sm[];
    uint32_t* masks = sm;                                 // [kWindow] row mask per block-column
    int* blk_pre = reinterpret_cast<int*>(sm + kWindow);  // [kWindow] exclusive block number (FILL only)
    __shared__ int scan_sh[64];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // The buffers of the plan are sized from the caller's block count: a range of row pointers that is not monotone or
    // holds more blocks than that would be written past their end.  Such a range gets an empty plan and a status code.
    if (range_is_bad(rowptr, brow_begin, brow_end, nnzb)) {
        if (!FILL) {
            for (int g = blockIdx.x * blockDim.x + threadIdx.x; g <= n_groups; g += gridDim.x * blockDim.x) gsp[g] = 0;
            if (blockIdx.x == 0 && threadIdx.x == 0 && status) atomicCAS(status, 0, kStatusBadRowptr);
        }
        return;
    }
    for (int g = blockIdx.x; g < n_groups; g += gridDim.x) {
        const int row = brow_begin + g * rg + warp;  // warps >= rg hold no row
        const bool have = warp < rg && row < brow_end;
        const int r_lo = __ldg(rowptr + brow_begin), r_hi = __ldg(rowptr + brow_end);
        const int beg = have ? min(max(__ldg(rowptr + row), r_lo), r_hi) : 0;  // clamped: a dip inside the range reads nothing outside it
        const int end = have ? min(max(__ldg(rowptr + row + 1), beg), r_hi) : 0;
        const int gfirst = min(max(__ldg(rowptr + brow_begin + g * rg), r_lo), r_hi);  // first block of the group
        const int rfirst = __ldg(rowptr + brow_begin);           // first block of the whole range
        int cur = beg;
        int steps_done = 0, blocks_done = 0;
        const int gs = FILL ? __ldg(gsp + g) : 0;
        for (int w0 = 0; w0 < Kb; w0 += kWindow) {
            const int cur_before = cur;
            mark_window(colidx, cur, end, w0, Kb, masks, warp, lane, status);
            // per-thread chunk of the window: PER consecutive block-columns = PER / 4 quads
            constexpr int PER = kWindow / kPlanThreads;
            static_assert(PER % 4 == 0, "a thread owns whole quads");
            const int i0 = threadIdx.x * PER;
            int ns = 0, nb = 0;
#pragma unroll
            for (int qd = 0; qd < PER / 4; qd++) {
                const int c = __popc(masks[i0 + 4 * qd]) + __popc(masks[i0 + 4 * qd + 1]) + __popc(masks[i0 + 4 * qd + 2]) +
                              __popc(masks[i0 + 4 * qd + 3]);
                ns += (c + CAP - 1) / CAP;
                nb += c;
            }
            int tot_s, tot_b = 0;
            const int pre_s = block_exclusive_scan(ns, &tot_s, scan_sh);
            if (FILL) {
                const int pre_b = block_exclusive_scan(nb, &tot_b, scan_sh);
                int s = steps_done + pre_s, b = blocks_done + pre_b;
                for (int qd = 0; qd < PER / 4; qd++) {
                    unsigned long long m64 = 0;
#pragma unroll
                    for (int sub = 0; sub < 4; sub++) {
                        const uint32_t mk = masks[i0 + 4 * qd + sub];
                        blk_pre[i0 + 4 * qd + sub] = b + __popcll(m64);
                        m64 |= (unsigned long long)mk << (16 * sub);
                    }
                    // cut the quad into steps of at most CAP blocks, in (sub-column, row) order
                    while (m64) {
                        unsigned long long part = 0;
                        for (int t = 0; t < CAP && m64; t++) {
                            const unsigned long long low = m64 & (~m64 + 1ull);
                            part |= low;
                            m64 ^= low;
                        }
                        // position of the step's first block in the packed stream, in 256-byte units
                        const uint32_t pos = 2u * (uint32_t)(gfirst - rfirst + b);
                        steps[gs + s] = make_uint4((uint32_t)(w0 + i0 + 4 * qd) << 4, pos, (uint32_t)part, (uint32_t)(part >> 32));
                        s++;
                        b += __popcll(part);
                    }
                }
                __syncthreads();
                // scatter: block j of this warp's row goes to its (column, row) rank inside the group
                for (int j = cur_before + lane; j < cur; j += 32) {
                    const int cbx = __ldg(colidx + j) >> 4;
                    const int cb = cbx - w0;
                    if (cb < 0 || cb >= kWindow || cbx >= Kb) continue;  // not marked above (status set there)
                    blk[gfirst + blk_pre[cb] + __popc(masks[cb] & ((1u << warp) - 1u))] = j;
                }
                blocks_done += tot_b;
            }
            steps_done += tot_s;
            __syncthreads();
        }
        if (!FILL && threadIdx.x == 0) gsp[g + 1] = steps_done;
    }
    if (!FILL && blockIdx.x == 0 && threadIdx.x == 0) gsp[0] = 0;
}

// In-place inclusive scan of data[0..n) by one CTA.
__global__ void __launch_bounds__(1024) plan_scan_kernel(int* data, int n) {
    __shared__ int warp_tot[32];
    __shared__ int carry_s, max_s;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) { carry_s = 0; max_s = 0; }
    __syncthreads();
    int vmax = 0;  // the largest entry before the scan = the most steps of any group, stored behind the scanned array
    for (int base = 0; base < n; base += 1024) {
        const int i = base + threadIdx.x;
        int v = i < n ? data[i] : 0;
        vmax = max(vmax, v);
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, v, d);
            if (lane >= d) v += t;
        }
        if (lane == 31) warp_tot[warp] = v;
        __syncthreads();
        if (warp == 0) {
            int w = warp_tot[lane];
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, w, d);
                if (lane >= d) w += t;
            }
            warp_tot[lane] = w;
        }
        __syncthreads();
        v += carry_s + (warp ? warp_tot[warp - 1] : 0);
        if (i < n) data[i] = v;
        __syncthreads();
        if (threadIdx.x == 1023) carry_s = v;
        __syncthreads();
    }
    atomicMax(&max_s, vmax);
    __syncthreads();
    if (threadIdx.x == 0) data[n] = max_s;
}

// One warp per step: copies the step's value blocks to their place in the packed stream; lane l moves
// the 16-byte chunk l of a block (row l/2, half l%2) to chunk l ^ ((l >> 3) & 1), i.e. the 32-byte swizzle.
__global__ void __launch_bounds__(256) pack_kernel(const uint4* __restrict__ vals, const int* __restrict__ blk,
                                                  const int* __restrict__ gsp, const uint4* __restrict__ steps,
                                                  uint8_t* __restrict__ packed, const int* __restrict__ rowptr, int brow_begin,
                                                  int n_groups) {
    const int rfirst = __ldg(rowptr + brow_begin);
    const int total = __ldg(gsp + n_groups);
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < total; i += warps) {
        const uint4 d = __ldg(steps + i);
        const int cnt = __popc(d.z) + __popc(d.w);
        const int first = rfirst + (int)(d.y >> 1);  // position of the step's first block in blk
        uint4* dst = reinterpret_cast<uint4*>(packed + (size_t)d.y * 256);
        for (int q = 0; q < cnt; q++) {
            const int src = __ldg(blk + first + q);
            dst[q * 32 + (lane ^ ((lane >> 3) & 1))] = __ldg(vals + (size_t)src * 32 + lane);
        }
    }
}


// ---- tall plans: groups of up to kTallRows block-rows (one warp of this kernel per block-row), 16-byte step records,
// ---- 64 bytes of per-warp words per step (the input of tall_pair_kernel below), groups padded to an even step count ----
constexpr int kTallPlanThreads = 1024;  // warp w owns block-row w of the group
static_assert(kTallRows == 24 && kTallBlocksPerStep <= 32, "the per-warp step words below are laid out for 12 warps of two rows and 5-bit block positions");

template <bool FILL>
__global__ void __launch_bounds__(kTallPlanThreads)
plan_tall_kernel(const int* __restrict__ rowptr, const int* __restrict__ colidx, int brow_begin, int brow_end, int rg, int CAP, int Kb,
                 int n_groups, int* __restrict__ gsp, uint4* __restrict__ steps, uint4* __restrict__ winfo, int* __restrict__ blk,
                 int nnzb, int* status) {
    extern __shared__ uint32_t sm[];
    uint32_t* masks = sm;                                 // [kWindow] row mask per block-column
    int* blk_pre = reinterpret_cast<int*>(sm + kWindow);  // [kWindow] exclusive block number (FILL only)
    __shared__ int scan_sh[64];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // The buffers of the plan are sized from the caller's block count: a range of row pointers that is not monotone or
    // holds more blocks than that would be written past their end.  Such a range gets an empty plan and a status code.
    if (range_is_bad(rowptr, brow_begin, brow_end, nnzb)) {
        if (!FILL) {
            for (int g = blockIdx.x * blockDim.x + threadIdx.x; g <= n_groups; g += gridDim.x * blockDim.x) gsp[g] = 0;
            if (blockIdx.x == 0 && threadIdx.x == 0 && status) atomicCAS(status, 0, kStatusBadRowptr);
        }
        return;
    }
    for (int g = blockIdx.x; g < n_groups; g += gridDim.x) {
        const int row = brow_begin + g * rg + warp;
        const bool have = warp < rg && row < brow_end;
        const int r_lo = __ldg(rowptr + brow_begin), r_hi = __ldg(rowptr + brow_end);
        const int beg = have ? min(max(__ldg(rowptr + row), r_lo), r_hi) : 0;
        const int end = have ? min(max(__ldg(rowptr + row + 1), beg), r_hi) : 0;
        const int gfirst = min(max(__ldg(rowptr + brow_begin + g * rg), r_lo), r_hi);
        const int rfirst = __ldg(rowptr + brow_begin);
        int cur = beg;
        int steps_done = 0, blocks_done = 0;
        const int gs = FILL ? __ldg(gsp + g) : 0;
        for (int w0 = 0; w0 < Kb; w0 += kWindow) {
            const int cur_before = cur;
            mark_window<kTallPlanThreads>(colidx, cur, end, w0, Kb, masks, warp, lane, status);
            constexpr int PER = kWindow / kTallPlanThreads;
            static_assert(PER % 4 == 0, "a thread owns whole quads");
            const int i0 = threadIdx.x * PER;
            int ns = 0, nb = 0;
#pragma unroll
            for (int qd = 0; qd < PER / 4; qd++) {
                const int c = __popc(masks[i0 + 4 * qd]) + __popc(masks[i0 + 4 * qd + 1]) + __popc(masks[i0 + 4 * qd + 2]) +
                              __popc(masks[i0 + 4 * qd + 3]);
                ns += (c + CAP - 1) / CAP;
                nb += c;
            }
            int tot_s, tot_b = 0;
            const int pre_s = block_exclusive_scan<kTallPlanThreads>(ns, &tot_s, scan_sh);
            if (FILL) {
                const int pre_b = block_exclusive_scan<kTallPlanThreads>(nb, &tot_b, scan_sh);
                int s = steps_done + pre_s, b = blocks_done + pre_b;
                for (int qd = 0; qd < PER / 4; qd++) {
                    uint32_t m[4];
                    int c = 0;
#pragma unroll
                    for (int sub = 0; sub < 4; sub++) {
                        m[sub] = masks[i0 + 4 * qd + sub];
                        blk_pre[i0 + 4 * qd + sub] = b + c;
                        c += __popc(m[sub]);
                    }
                    // cut the quad into steps of at most CAP blocks, in (sub-column, row) order
                    while (c > 0) {
                        uint32_t part[4] = {0u, 0u, 0u, 0u};
                        int taken = 0;
#pragma unroll
                        for (int sub = 0; sub < 4; sub++) {
                            while (m[sub] && taken < CAP) {
                                const uint32_t low = m[sub] & (~m[sub] + 1u);
                                part[sub] |= low;
                                m[sub] ^= low;
                                taken++;
                            }
                        }
                        const uint32_t pos = 2u * (uint32_t)(gfirst - rfirst + b);
                        steps[gs + s] = make_uint4((uint32_t)(w0 + i0 + 4 * qd) << 4, pos, (uint32_t)taken,
                                                    (part[0] ? 1u : 0u) | (part[1] ? 2u : 0u) | (part[2] ? 4u : 0u) | (part[3] ? 8u : 0u));
                        // what each MMA-issuing warp needs of the step: warp m owns block-rows 2m, 2m + 1
                        const uint32_t pre1 = (uint32_t)__popc(part[0]), pre2 = pre1 + (uint32_t)__popc(part[1]),
                                       pre3 = pre2 + (uint32_t)__popc(part[2]);
                        const uint32_t pre[4] = {0u, pre1, pre2, pre3};
                        uint4* wdst = winfo + 4 * (size_t)(gs + s);
#pragma unroll
                        for (int v = 0; v < 3; v++) {
                            uint32_t wi[4];
#pragma unroll
                            for (int mm = 0; mm < 4; mm++) {
                                const int m = 4 * v + mm;
                                uint32_t word = 0;
#pragma unroll
                                for (int sub = 0; sub < 4; sub++) {
                                    const uint32_t own = (part[sub] >> (2 * m)) & 3u;
                                    const uint32_t q = pre[sub] + (uint32_t)__popc(part[sub] & ((1u << (2 * m)) - 1u));
                                    word |= own << (2 * sub);
                                    word |= (q & 31u) << (8 + 5 * sub);
                                }
                                wi[mm] = word;
                            }
                            wdst[v] = make_uint4(wi[0], wi[1], wi[2], wi[3]);
                        }
                        wdst[3] = make_uint4((part[0] ? 1u : 0u) | (part[1] ? 2u : 0u) | (part[2] ? 4u : 0u) | (part[3] ? 8u : 0u), 0u, 0u, 0u);
                        s++;
                        b += taken;
                        c -= taken;
                    }
                }
                __syncthreads();
                for (int j = cur_before + lane; j < cur; j += 32) {
                    const int cbx = __ldg(colidx + j) >> 4;
                    const int cb = cbx - w0;
                    if (cb < 0 || cb >= kWindow || cbx >= Kb) continue;  // not marked above (status set there)
                    blk[gfirst + blk_pre[cb] + __popc(masks[cb] & ((1u << warp) - 1u))] = j;
                }
                blocks_done += tot_b;
            }
            steps_done += tot_s;
            __syncthreads();
        }
        // The kernel hands steps to its MMA warps two at a time: a group with an odd number of steps gets one more
        // without blocks (no panel is fetched for it).
        if (!FILL && threadIdx.x == 0) gsp[g + 1] = (steps_done + 1) & ~1;
        if (FILL && threadIdx.x == 0 && (steps_done & 1)) {
            steps[gs + steps_done] = make_uint4(0u, 2u * (uint32_t)(gfirst - rfirst + blocks_done), 0u, 0u);
            uint4* wdst = winfo + 4 * (size_t)(gs + steps_done);
            for (int v = 0; v < 4; v++) wdst[v] = make_uint4(0u, 0u, 0u, 0u);
        }
    }
    if (!FILL && blockIdx.x == 0 && threadIdx.x == 0) gsp[0] = 0;
}

// Tall plans, last pass: the kernel hands its MMA warps the steps two at a time, so what each warp has to issue for a
// pair is listed here once, ready to use.  One thread per (pair, warp m): from the two steps' words (bits 2s, 2s + 1
// = rows 2m, 2m + 1 have a block in sub-column s; bits [8 + 5s, 13 + 5s) = position of the first of them among the
// step's blocks) to four words holding up to eight 16-bit entries, one per MMA, in (step, sub-column) order:
//   bits [0, 6)  block position in the pair's two block slots (24 * step + position in the step)
//   bits [6, 9)  panel sub-column, 4 * step + s            bit 9  accumulator of row 2m + 1 (else 2m)
//   bit 10       both rows (one MMA of 32 accumulator columns)
// and the number of entries in bits [28, 32) of word 0 (the spare bits of its second entry).
__global__ void __launch_bounds__(256) tall_pair_kernel(const uint32_t* __restrict__ wstep, uint4* __restrict__ winfo,
                                                       const int* __restrict__ gsp, int n_groups) {
    const int pairs = __ldg(gsp + n_groups) >> 1;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < pairs * 16; i += gridDim.x * blockDim.x) {
        const int pr = i >> 4, m = i & 15;
        uint32_t out[4] = {0u, 0u, 0u, 0u};
        if (m < kTallRows / 2) {
            uint32_t n = 0;
            for (uint32_t st = 0; st < 2; st++) {
                const uint32_t x = __ldg(wstep + ((size_t)(2 * pr) + st) * 16 + m);
                for (uint32_t sub = 0; sub < 4; sub++) {
                    const uint32_t own = (x >> (2 * sub)) & 3u;
                    if (!own) continue;
                    const uint32_t q = (x >> (8 + 5 * sub)) & 31u;
                    const uint32_t e = (st * (uint32_t)kTallBlocksPerStep + q) | ((4 * st + sub) << 6) | ((own == 2u ? 1u : 0u) << 9) |
                                       ((own == 3u ? 1u : 0u) << 10);
                    out[n >> 1] |= e << (16 * (n & 1));
                    n++;
                }
            }
            out[0] |= n << 28;
        }
        winfo[(size_t)pr * 16 + m] = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

// One warp per step of a tall plan: copies the step's value blocks to their place in the packed stream (32-byte swizzle).
__global__ void __launch_bounds__(256) pack_tall_kernel(const uint4* __restrict__ vals, const int* __restrict__ blk,
                                                       const int* __restrict__ gsp, const uint4* __restrict__ steps,
                                                       uint8_t* __restrict__ packed, const int* __restrict__ rowptr, int brow_begin,
                                                       int n_groups) {
    const int rfirst = __ldg(rowptr + brow_begin);
    const int total = __ldg(gsp + n_groups);
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < total; i += warps) {
        const uint4 d = __ldg(steps + i);
        const int cnt = (int)d.z;
        const int first = rfirst + (int)(d.y >> 1);
        uint4* dst = reinterpret_cast<uint4*>(packed + (size_t)d.y * 256);
        for (int q = 0; q < cnt; q++) {
            const int src = __ldg(blk + first + q);
            dst[q * 32 + (lane ^ ((lane >> 3) & 1))] = __ldg(vals + (size_t)src * 32 + lane);
        }
    }
}

}  // namespace

int pack_values_async(const int* rowptr, const void* vals, const int* gsp, const void* steps, const int* blk, void* packed,
                      size_t brow_begin, size_t brow_end, size_t rg, size_t nnzb, cudaStream_t stream,
                      const DeviceCtx* ctx_in) {
    if (nnzb == 0 || brow_end == brow_begin) return SMAT_OK;
    const DeviceCtx* ctx = ctx_in;
    if (!ctx) {
        DeviceCtx* c = nullptr;
        if (int rc = get_device_ctx(&c)) return rc;
        ctx = c;
    }
    const size_t n_groups = (brow_end - brow_begin + rg - 1) / rg;
    pack_kernel<<<ctx->sm_count * 8, 256, 0, stream>>>(reinterpret_cast<const uint4*>(vals), blk, gsp,
                                                       reinterpret_cast<const uint4*>(steps), reinterpret_cast<uint8_t*>(packed),
                                                       rowptr, (int)brow_begin, (int)n_groups);
    count_launch();
    SMAT_CUDA_TRY(cudaGetLastError());
    return SMAT_OK;
}

size_t choose_rows_per_group(size_t block_rows, size_t N, int sm_count, bool can_cut, size_t nnzb, size_t K) {
    static const int forced = [] {  // tuning knob: SMAT_ROWS_PER_GROUP=4..16 overrides the choice
        const char* e = std::getenv("SMAT_ROWS_PER_GROUP");
        const int v = e ? std::atoi(e) : 0;
        return (v >= 4 && v <= kPlanRowsPerGroup) ? v : 0;
    }();
    if (forced) return (size_t)forced;
    if (N == 0 || block_rows == 0) return kPlanRowsPerGroup;
    const size_t sms = (size_t)sm_count;
    size_t best = kPlanRowsPerGroup;
    double best_cost = 0.0;
    for (size_t rg = kPlanRowsPerGroup; rg >= 8; rg--) {
        const size_t groups = (block_rows + rg - 1) / rg;
        size_t est_steps = nnzb / groups;  // steps per item: at most one per block and one per 64 columns
        if (K / 64 < est_steps) est_steps = K / 64;
        // the per-item overhead (pipeline fill, epilogue, steps that do not shrink with the height) is worth about
        // four block-rows of work
        double cost = rounds_for(groups * ((N + 127) / 128), sms, can_cut, est_steps, false) * (double)(rg + 4);
        if (N >= 256 && nnzb / groups >= 256 && est_steps >= 64) {
            const double wide = kWideItemCost * rounds_for(groups * ((N + 255) / 256), sms, can_cut, est_steps, true) * (double)(rg + 4);
            if (wide < cost) cost = wide;
        }
        if (rg == kPlanRowsPerGroup || cost < best_cost * 0.97) {  // a smaller group must pay for its lower panel reuse
            best = rg;
            best_cost = cost;
        }
    }
    return best;
}

PlanSizes plan_sizes(size_t nnzb, size_t brow_begin, size_t brow_end, size_t rg, size_t max_steps) {
    PlanSizes s;
    s.n_groups = (brow_end - brow_begin + rg - 1) / rg;
    s.gsp_bytes = ((s.n_groups + 2) * sizeof(int) + 255) / 256 * 256;  // + the largest step count of a group
    // a step holds at least one block, so nnzb bounds the number of steps
    const size_t steps = max_steps ? max_steps : (nnzb ? nnzb : 1);
    s.steps_bytes = (steps * sizeof(uint4) + 255) / 256 * 256;
    s.blk_bytes = ((nnzb ? nnzb : 1) * sizeof(int) + 255) / 256 * 256;
    s.packed_bytes = (nnzb ? nnzb : 1) * 512;
    return s;
}

static int plan_launch_setup(const DeviceCtx* ctx_in, const DeviceCtx** ctx) {
    *ctx = ctx_in;
    if (!*ctx) {
        DeviceCtx* c = nullptr;
        if (int rc = get_device_ctx(&c)) return rc;
        *ctx = c;
    }
    return SMAT_OK;
}

int plan_count_async(const int* rowptr, const int* colidx, size_t K, size_t nnzb, size_t brow_begin, size_t brow_end,
                     size_t rg, int* gsp, cudaStream_t stream, const DeviceCtx* ctx_in, size_t cap) {
    const DeviceCtx* ctx = nullptr;
    if (int rc = plan_launch_setup(ctx_in, &ctx)) return rc;
    const size_t n_groups = (brow_end - brow_begin + rg - 1) / rg;
    if (n_groups == 0) return SMAT_OK;
    if (nnzb == 0) {
        SMAT_CUDA_TRY(cudaMemsetAsync(gsp, 0, (n_groups + 1) * sizeof(int), stream));
        return SMAT_OK;
    }
    const int grid = (int)(n_groups < (size_t)ctx->sm_count ? n_groups : (size_t)ctx->sm_count);
    const size_t smem_count = (size_t)kWindow * 4;
    SMAT_CUDA_TRY(cudaFuncSetAttribute(plan_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_count));
    plan_kernel<false><<<grid, kPlanThreads, smem_count, stream>>>(rowptr, colidx, (int)brow_begin, (int)brow_end, (int)rg, (int)cap,
                                                                  (int)(K / 16), (int)n_groups, gsp, nullptr, nullptr, (int)nnzb,
                                                                  ctx->d_status);
    count_launch();
    plan_scan_kernel<<<1, 1024, 0, stream>>>(gsp, (int)n_groups + 1);
    count_launch();
    SMAT_CUDA_TRY(cudaGetLastError());
    return SMAT_OK;
}

int plan_fill_async(const int* rowptr, const int* colidx, size_t K, size_t nnzb, size_t brow_begin, size_t brow_end,
                    size_t rg, const int* gsp, void* steps, int* blk, cudaStream_t stream, const DeviceCtx* ctx_in, size_t cap) {
    const DeviceCtx* ctx = nullptr;
    if (int rc = plan_launch_setup(ctx_in, &ctx)) return rc;
    const size_t n_groups = (brow_end - brow_begin + rg - 1) / rg;
    if (n_groups == 0 || nnzb == 0) return SMAT_OK;
    const int grid = (int)(n_groups < (size_t)ctx->sm_count ? n_groups : (size_t)ctx->sm_count);
    const size_t smem_fill = (size_t)kWindow * 8;
    SMAT_CUDA_TRY(cudaFuncSetAttribute(plan_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_fill));
    plan_kernel<true><<<grid, kPlanThreads, smem_fill, stream>>>(rowptr, colidx, (int)brow_begin, (int)brow_end, (int)rg, (int)cap,
                                                                 (int)(K / 16), (int)n_groups, const_cast<int*>(gsp),
                                                                 reinterpret_cast<uint4*>(steps), blk, (int)nnzb, ctx->d_status);
    count_launch();
    SMAT_CUDA_TRY(cudaGetLastError());
    return SMAT_OK;
}


int plan_count_tall_async(const int* rowptr, const int* colidx, size_t K, size_t nnzb, size_t brow_begin, size_t brow_end,
                          size_t rg, int* gsp, cudaStream_t stream, const DeviceCtx* ctx_in) {
    const DeviceCtx* ctx = nullptr;
    if (int rc = plan_launch_setup(ctx_in, &ctx)) return rc;
    const size_t n_groups = (brow_end - brow_begin + rg - 1) / rg;
    if (n_groups == 0) return SMAT_OK;
    if (nnzb == 0) {
        SMAT_CUDA_TRY(cudaMemsetAsync(gsp, 0, (n_groups + 1) * sizeof(int), stream));
        return SMAT_OK;
    }
    const int grid = (int)(n_groups < (size_t)ctx->sm_count ? n_groups : (size_t)ctx->sm_count);
    const size_t smem_count = (size_t)kWindow * 4;
    SMAT_CUDA_TRY(cudaFuncSetAttribute(plan_tall_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_count));
    plan_tall_kernel<false><<<grid, kTallPlanThreads, smem_count, stream>>>(rowptr, colidx, (int)brow_begin, (int)brow_end, (int)rg,
                                                                           kTallBlocksPerStep, (int)(K / 16), (int)n_groups, gsp, nullptr,
                                                                           nullptr, nullptr, (int)nnzb, ctx->d_status);
    count_launch();
    plan_scan_kernel<<<1, 1024, 0, stream>>>(gsp, (int)n_groups + 1);
    count_launch();
    SMAT_CUDA_TRY(cudaGetLastError());
    return SMAT_OK;
}

int plan_fill_tall_async(const int* rowptr, const int* colidx, size_t K, size_t nnzb, size_t brow_begin, size_t brow_end,
                         size_t rg, const int* gsp, void* steps, void* wstep, void* winfo, int* blk, cudaStream_t stream,
                         const DeviceCtx* ctx_in) {
    const DeviceCtx* ctx = nullptr;
    if (int rc = plan_launch_setup(ctx_in, &ctx)) return rc;
    const size_t n_groups = (brow_end - brow_begin + rg - 1) / rg;
    if (n_groups == 0 || nnzb == 0) return SMAT_OK;
    const int grid = (int)(n_groups < (size_t)ctx->sm_count ? n_groups : (size_t)ctx->sm_count);
    const size_t smem_fill = (size_t)kWindow * 8;
    SMAT_CUDA_TRY(cudaFuncSetAttribute(plan_tall_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_fill));
    plan_tall_kernel<true><<<grid, kTallPlanThreads, smem_fill, stream>>>(rowptr, colidx, (int)brow_begin, (int)brow_end, (int)rg,
                                                                         kTallBlocksPerStep, (int)(K / 16), (int)n_groups,
                                                                         const_cast<int*>(gsp), reinterpret_cast<uint4*>(steps),
                                                                         reinterpret_cast<uint4*>(wstep), blk, (int)nnzb, ctx->d_status);
    count_launch();
    tall_pair_kernel<<<ctx->sm_count * 4, 256, 0, stream>>>(reinterpret_cast<const uint32_t*>(wstep), reinterpret_cast<uint4*>(winfo), gsp,
                                                            (int)n_groups);
    count_launch();
    SMAT_CUDA_TRY(cudaGetLastError());
    return SMAT_OK;
}

int pack_values_tall_async(const int* rowptr, const void* vals, const int* gsp, const void* steps, const int* blk, void* packed,
                           size_t brow_begin, size_t brow_end, size_t rg, size_t nnzb, cudaStream_t stream,
                           const DeviceCtx* ctx_in) {
    if (nnzb == 0 || brow_end == brow_begin) return SMAT_OK;
    const DeviceCtx* ctx = nullptr;
    if (int rc = plan_launch_setup(ctx_in, &ctx)) return rc;
    const size_t n_groups = (brow_end - brow_begin + rg - 1) / rg;
    pack_tall_kernel<<<ctx->sm_count * 8, 256, 0, stream>>>(reinterpret_cast<const uint4*>(vals), blk, gsp,
                                                            reinterpret_cast<const uint4*>(steps), reinterpret_cast<uint8_t*>(packed),
                                                            rowptr, (int)brow_begin, (int)n_groups);
    count_launch();
    SMAT_CUDA_TRY(cudaGetLastError());
    return SMAT_OK;
}

}  // namespace smat

using namespace smat;

struct smat_plan {
    PlanView v;
    void* buffer = nullptr;
    void* gsp_buffer = nullptr;
    void* fix_buffer = nullptr;  // partial tiles of cut work items
    void* sched_buffer = nullptr;  // listed schedule: offsets per CTA, then the groups
    int device = -1;
    // smat_plan_spmm_host: device staging (B and C whole), the copy streams, per-chunk and per-range events
    void* host_B = nullptr;
    void* host_C = nullptr;
    size_t host_B_bytes = 0, host_C_bytes = 0;
    cudaStream_t s_in = nullptr, s_out = nullptr;
    cudaEvent_t ev_start = nullptr;
    std::vector<cudaEvent_t> ev_in, ev_done, ev_out;
};

// A plan's memory and tuning belong to the device it was created on.
static int check_plan_device(const smat_plan* plan) {
    int dev = -1;
    SMAT_CUDA_TRY(cudaGetDevice(&dev));
    if (dev != plan->device)
        return fail(SMAT_ERR_BAD_ARG, "the plan belongs to device %d but device %d is current", plan->device, dev);
    return SMAT_OK;
}

extern "C" {

int smat_plan_create(smat_plan** out, const void* bcsrValuesA, const int* bcsrRowPtrA, const int* bcsrColIdxA, size_t M,
                     size_t K, size_t nnzb, size_t brow_begin, size_t brow_end, size_t N_hint, void* stream) {
    clear_error();
    if (!out || !bcsrRowPtrA || (nnzb && (!bcsrColIdxA || !bcsrValuesA))) return fail(SMAT_ERR_BAD_ARG, "NULL argument");
    if (M % 16 || K % 16) return fail(SMAT_ERR_BAD_ARG, "M (%zu) and K (%zu) must be multiples of 16", M, K);
    if ((uintptr_t)bcsrValuesA & 15) return fail(SMAT_ERR_BAD_ARG, "bcsrValuesA must be 16-byte aligned");
    if (brow_begin > brow_end || brow_end > M / 16)
        return fail(SMAT_ERR_BAD_ARG, "block-row range [%zu, %zu) outside [0, %zu]", brow_begin, brow_end, M / 16);
    if (nnzb * 16 >= ((size_t)1 << 31) || K >= ((size_t)1 << 31)) return fail(SMAT_ERR_RANGE, "size beyond 2^31");
    smat_plan* p = new (std::nothrow) smat_plan();
    if (!p) return fail(SMAT_ERR_NOMEM, "out of host memory");
    DeviceCtx* ctx = nullptr;
    if (int rc0 = get_device_ctx(&ctx)) {
        delete p;
        return rc0;
    }
    const size_t rg = choose_rows_per_group(brow_end - brow_begin, N_hint, ctx->sm_count, true, nnzb, K);
    // phase 1 into a small buffer of its own; the step total then sizes the rest exactly
    PlanSizes sz = plan_sizes(nnzb, brow_begin, brow_end, rg);
    cudaError_t e = cudaGetDevice(&p->device);
    if (e == cudaSuccess) e = cudaMalloc(&p->gsp_buffer, sz.gsp_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&p->fix_buffer, fix_scratch_bytes(ctx->sm_count));
    if (e != cudaSuccess) {
        cudaFree(p->gsp_buffer);
        cudaFree(p->fix_buffer);
        cudaFree(p->sched_buffer);
        delete p;
        return fail(SMAT_ERR_CUDA, "plan allocation failed: %s", cudaGetErrorString(e));
    }
    int* gsp = static_cast<int*>(p->gsp_buffer);
    int rc = plan_count_async(bcsrRowPtrA, bcsrColIdxA, K, nnzb, brow_begin, brow_end, rg, gsp, (cudaStream_t)stream);
    int total_and_max[2] = {0, 0};
    if (rc == SMAT_OK && sz.n_groups) {
        e = cudaMemcpyAsync(total_and_max, gsp + sz.n_groups, 2 * sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
        if (e != cudaSuccess) rc = fail(SMAT_ERR_CUDA, "plan build failed: %s", cudaGetErrorString(e));
    }
    // blocks of THIS range (nonzeroBlocks counts the whole arrays): what the choices below and at launch go by
    size_t range_blocks = nnzb;
    if (rc == SMAT_OK && nnzb) {
        int ends[2] = {0, 0};
        e = cudaMemcpyAsync(&ends[0], bcsrRowPtrA + brow_begin, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(&ends[1], bcsrRowPtrA + brow_end, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
        if (e != cudaSuccess) rc = fail(SMAT_ERR_CUDA, "plan build failed: %s", cudaGetErrorString(e));
        else if (ends[1] >= ends[0] && (size_t)(ends[1] - ends[0]) <= nnzb) range_blocks = (size_t)(ends[1] - ends[0]);
    }
    // Densely filled quads (dense clusters: every quad of a cluster holds all 64 blocks) are cut into pieces of at most 24
    // blocks that each fetch the B panel again; when the steps are that full on average, recount with 32 per step.
    size_t cap = kPlanBlocksPerStep;
    if (rc == SMAT_OK && total_and_max[0] > 0 && range_blocks >= 18 * (size_t)total_and_max[0]) {
        cap = kPlanBlocksPerStepDense;
        rc = plan_count_async(bcsrRowPtrA, bcsrColIdxA, K, nnzb, brow_begin, brow_end, rg, gsp, (cudaStream_t)stream, nullptr, cap);
        if (rc == SMAT_OK) {
            e = cudaMemcpyAsync(total_and_max, gsp + sz.n_groups, 2 * sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
            if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
            if (e != cudaSuccess) rc = fail(SMAT_ERR_CUDA, "plan build failed: %s", cudaGetErrorString(e));
        }
    }
    const int total_steps = total_and_max[0];  // of the 16-row plan
    // Schedule: when the heaviest group holds many times the average number of steps, items dealt out round-robin
    // leave most SMs waiting for the one with the heaviest item; such plans deal out equal step ranges instead.
    bool balanced = (size_t)total_and_max[1] * sz.n_groups > 4 * (size_t)total_steps &&
                    (size_t)total_steps >= 8 * (size_t)ctx->sm_count;
    if (rc == SMAT_OK && balanced && sz.n_groups >= 4 * (size_t)ctx->sm_count) {
        // First choice: whole groups dealt out heaviest first to the least loaded CTA (keeps every item in one piece
        // and the CTAs sweeping the block-columns the way the round-robin schedule does); taken when the heaviest
        // CTA ends up within a quarter of the average load.
        const int G = ctx->sm_count;
        std::vector<int> h_gsp(sz.n_groups + 1);
        e = cudaMemcpy(h_gsp.data(), gsp, (sz.n_groups + 1) * sizeof(int), cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) rc = fail(SMAT_ERR_CUDA, "plan build failed: %s", cudaGetErrorString(e));
        if (rc == SMAT_OK) {
            std::vector<int> order(sz.n_groups);
            for (size_t g = 0; g < sz.n_groups; g++) order[g] = (int)g;
            std::stable_sort(order.begin(), order.end(),
                             [&](int a, int b) { return h_gsp[a + 1] - h_gsp[a] > h_gsp[b + 1] - h_gsp[b]; });
            std::priority_queue<std::pair<long long, int>, std::vector<std::pair<long long, int>>, std::greater<>> heap;
            for (int c = 0; c < G; c++) heap.push({0, c});
            std::vector<std::vector<int>> lists(G);
            long long heaviest = 0;
            for (int g : order) {
                auto [load, c] = heap.top();
                heap.pop();
                load += h_gsp[g + 1] - h_gsp[g];
                lists[c].push_back(g);
                if (load > heaviest) heaviest = load;
                heap.push({load, c});
            }
            if (heaviest * 4 * G <= 5LL * total_steps) {
                std::vector<int> flat(G + 1 + sz.n_groups);
                int pos = 0;
                for (int c = 0; c < G; c++) {
                    flat[c] = pos;
                    for (int g : lists[c]) flat[G + 1 + pos++] = g;
                }
                flat[G] = pos;
                e = cudaMalloc(&p->sched_buffer, flat.size() * sizeof(int));
                if (e == cudaSuccess) e = cudaMemcpy(p->sched_buffer, flat.data(), flat.size() * sizeof(int), cudaMemcpyHostToDevice);
                if (e != cudaSuccess) rc = fail(SMAT_ERR_CUDA, "plan allocation failed: %s", cudaGetErrorString(e));
                p->v.sched_off = static_cast<const int*>(p->sched_buffer);
                p->v.sched_list = static_cast<const int*>(p->sched_buffer) + G + 1;
                p->v.sched_ctas = G;
                balanced = false;
            }
        }
    }
    // Tall plan: groups of up to 24 block-rows for the kernel that reads the B panels from tensor memory.  Its steps
    // cost a little more than those of the 16-row kernels (measured ~550 against ~470 cycles, the latter growing with
    // the blocks of the step: ~45 cycles each with the hand-overs, the shared-memory operand port), so it pays where taller groups mean
    // fewer steps: matrices whose quads mostly hold a block (a block-sparse layer, a reordered random matrix: three
    // quarters of the steps), not scattered ones (as many steps as before) and not dense clusters (steps of 32 blocks
    // already).  Both plans are counted and the estimates compared; smat_spmm_set_variant(4) forces a tall plan,
    // 1..3 exclude it.
    bool tall = false;
    size_t rg_used = rg;
    const size_t rows = brow_end - brow_begin, tiles = ((N_hint ? N_hint : 128) + 127) / 128;
    const bool tall_forced = g_spmm_variant == 4;
    const bool tall_possible = rc == SMAT_OK && !balanced && !p->v.sched_list && total_steps > 0 && rows > 0 &&
                               (tall_forced || (g_spmm_variant == 0 && cap == (size_t)kPlanBlocksPerStep && rows >= 16 && N_hint >= 128 &&
                                                (size_t)total_steps * tiles >= 64 * (size_t)ctx->sm_count));
    if (tall_possible) {
        // Height of the groups: what a launch costs is about (rounds of work items) x (steps of an item) x (bytes a
        // step moves from L2: a 16 KB panel and its blocks).  The steps of an item hardly change with the height as
        // long as most quads hold a block, so compare rounds x bytes per step.
        size_t rg_tall = kTallRows;
        double best = 0.0;
        const double steps_per_group = (double)total_steps / (double)sz.n_groups;
        for (size_t r = kTallRows; r >= 16; r -= 2) {
            const size_t groups = (rows + r - 1) / r;
            // (blocks per step of a full group: the heaviest item sets the time of a round)
            const double blocks_per_step =
                (double)range_blocks / (double)rows * (double)(r < rows ? r : rows) / (steps_per_group > 1.0 ? steps_per_group : 1.0);
            const double cost = rounds_for(groups * tiles, (size_t)ctx->sm_count, true, (size_t)steps_per_group, false) *
                                (16384.0 + 512.0 * blocks_per_step);
            if (r == (size_t)kTallRows || cost < best * 0.97) {
                best = cost;
                rg_tall = r;
            }
        }
        if (const char* ev = std::getenv("SMAT_TALL_ROWS")) {  // tuning knob
            const int v = std::atoi(ev);
            if (v >= 1 && v <= kTallRows) rg_tall = (size_t)v;
        }
        // the group count changes with the height: count into a buffer of its own, kept if the tall plan is taken
        const PlanSizes sz_tall = plan_sizes(nnzb, brow_begin, brow_end, rg_tall);
        void* gsp_tall = nullptr;
        int tall_total_and_max[2] = {0, 0};
        e = cudaMalloc(&gsp_tall, sz_tall.gsp_bytes);
        if (e != cudaSuccess) rc = fail(SMAT_ERR_CUDA, "plan allocation failed: %s", cudaGetErrorString(e));
        if (rc == SMAT_OK)
            rc = plan_count_tall_async(bcsrRowPtrA, bcsrColIdxA, K, nnzb, brow_begin, brow_end, rg_tall, static_cast<int*>(gsp_tall),
                                       (cudaStream_t)stream);
        if (rc == SMAT_OK) {
            e = cudaMemcpyAsync(tall_total_and_max, static_cast<int*>(gsp_tall) + sz_tall.n_groups, 2 * sizeof(int), cudaMemcpyDeviceToHost,
                                (cudaStream_t)stream);
            if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
            if (e != cudaSuccess) rc = fail(SMAT_ERR_CUDA, "plan build failed: %s", cudaGetErrorString(e));
        }
        if (rc == SMAT_OK) {
            const double per_step = (double)range_blocks / (double)total_steps;
            const double est16 = rounds_for(sz.n_groups * tiles, (size_t)ctx->sm_count, true, (size_t)steps_per_group, false) * steps_per_group *
                                 (per_step * 45.0 > 470.0 ? per_step * 45.0 : 470.0);
            const double steps_per_tall = (double)tall_total_and_max[0] / (double)sz_tall.n_groups;
            const double est_tall =
                rounds_for(sz_tall.n_groups * tiles, (size_t)ctx->sm_count, true, (size_t)steps_per_tall, false) * steps_per_tall * 550.0;
            tall = tall_forced || est_tall < 0.97 * est16;
            if (std::getenv("SMAT_PLAN_DEBUG"))
                fprintf(stderr, "[smat plan] estimates: 16-row %.0f cycles, tall (rg %zu, %d steps) %.0f cycles -> %s\n", est16, rg_tall,
                        tall_total_and_max[0], est_tall, tall ? "tall" : "16-row");
        }
        if (rc == SMAT_OK && tall) {
            cudaFree(p->gsp_buffer);
            p->gsp_buffer = gsp_tall;
            gsp = static_cast<int*>(gsp_tall);
            sz = sz_tall;
            rg_used = rg_tall;
            total_and_max[0] = tall_total_and_max[0];
            total_and_max[1] = tall_total_and_max[1];
            cap = kTallBlocksPerStep;
        } else {
            cudaFree(gsp_tall);
        }
    }
    const int steps_final = total_and_max[0];
    if (std::getenv("SMAT_PLAN_DEBUG"))
        fprintf(stderr, "[smat plan] rows %zu blocks %zu: 16-row plan rg %zu steps %d cap %zu balanced %d listed %d; tall %d rg %zu steps %d max/group %d\n",
                brow_end - brow_begin, range_blocks, rg, total_steps, cap, (int)balanced, p->v.sched_list != nullptr, (int)tall, rg_used,
                steps_final, total_and_max[1]);
    if (rc == SMAT_OK && balanced) {  // two partial tiles per CTA
        cudaFree(p->fix_buffer);
        p->fix_buffer = nullptr;
        e = cudaMalloc(&p->fix_buffer, 2 * fix_scratch_bytes(ctx->sm_count));
        if (e != cudaSuccess) rc = fail(SMAT_ERR_CUDA, "plan allocation failed: %s", cudaGetErrorString(e));
    }
    if (rc == SMAT_OK) {
        sz = plan_sizes(nnzb, brow_begin, brow_end, rg_used, (size_t)(steps_final > 0 ? steps_final : 1) * (tall ? 13 : 1));  // tall: + 64 bytes of per-step words + 128 bytes of the per-pair lists
        e = cudaMalloc(&p->buffer, sz.steps_bytes + sz.blk_bytes + sz.packed_bytes);
        if (e != cudaSuccess) rc = fail(SMAT_ERR_CUDA, "plan allocation failed: %s", cudaGetErrorString(e));
    }
    if (rc) {
        cudaFree(p->gsp_buffer);
        cudaFree(p->fix_buffer);
        cudaFree(p->sched_buffer);
        delete p;
        return rc;
    }
    char* b = static_cast<char*>(p->buffer);
    p->v.rowptr = bcsrRowPtrA;
    p->v.gsp = gsp;
    p->v.steps = b;
    p->v.blk = reinterpret_cast<int*>(b + sz.steps_bytes);
    p->v.packed = b + sz.steps_bytes + sz.blk_bytes;
    p->v.K = K;
    p->v.nnzb = range_blocks;  // blocks of the plan's range
    p->v.brow_begin = brow_begin;
    p->v.brow_end = brow_end;
    p->v.n_groups = sz.n_groups;
    p->v.rg = rg_used;
    p->v.fix_scratch = static_cast<float*>(p->fix_buffer);
    p->v.total_steps = (size_t)(steps_final > 0 ? steps_final : 0);
    p->v.balanced = balanced;
    p->v.cap = cap;
    p->v.tall = tall;
    if (tall) {
        // behind the step records, in the same region: the per-step words (only read while the plan is built), then the per-pair lists
        char* wstep = b + (size_t)(steps_final > 0 ? steps_final : 1) * 16;
        p->v.winfo = wstep + (size_t)(steps_final > 0 ? steps_final : 1) * 64;
        rc = plan_fill_tall_async(bcsrRowPtrA, bcsrColIdxA, K, nnzb, brow_begin, brow_end, rg_used, gsp, const_cast<void*>(p->v.steps), wstep,
                                  const_cast<void*>(p->v.winfo), const_cast<int*>(p->v.blk), (cudaStream_t)stream);
        if (rc == SMAT_OK)
            rc = pack_values_tall_async(bcsrRowPtrA, bcsrValuesA, gsp, p->v.steps, p->v.blk, const_cast<void*>(p->v.packed),
                                        brow_begin, brow_end, rg_used, nnzb, (cudaStream_t)stream);
    } else {
        rc = plan_fill_async(bcsrRowPtrA, bcsrColIdxA, K, nnzb, brow_begin, brow_end, rg, gsp, const_cast<void*>(p->v.steps),
                             const_cast<int*>(p->v.blk), (cudaStream_t)stream, nullptr, cap);
        if (rc == SMAT_OK)
            rc = pack_values_async(bcsrRowPtrA, bcsrValuesA, gsp, p->v.steps, p->v.blk, const_cast<void*>(p->v.packed), brow_begin,
                                   brow_end, rg, nnzb, (cudaStream_t)stream);
    }
    if (rc) {
        cudaFree(p->buffer);
        cudaFree(p->gsp_buffer);
        cudaFree(p->fix_buffer);
        cudaFree(p->sched_buffer);
        delete p;
        return rc;
    }
    *out = p;
    return SMAT_OK;
}

int smat_plan_set_values(smat_plan* plan, const void* bcsrValuesA, void* stream) {
    clear_error();
    if (!plan || (plan->v.nnzb && !bcsrValuesA)) return fail(SMAT_ERR_BAD_ARG, "NULL argument");
    if ((uintptr_t)bcsrValuesA & 15) return fail(SMAT_ERR_BAD_ARG, "bcsrValuesA must be 16-byte aligned");
    if (int rc = check_plan_device(plan)) return rc;
    if (plan->v.tall)
        return pack_values_tall_async(plan->v.rowptr, bcsrValuesA, plan->v.gsp, plan->v.steps, plan->v.blk,
                                      const_cast<void*>(plan->v.packed), plan->v.brow_begin, plan->v.brow_end, plan->v.rg,
                                      plan->v.nnzb, (cudaStream_t)stream);
    return pack_values_async(plan->v.rowptr, bcsrValuesA, plan->v.gsp, plan->v.steps, plan->v.blk,
                             const_cast<void*>(plan->v.packed), plan->v.brow_begin, plan->v.brow_end, plan->v.rg,
                             plan->v.nnzb, (cudaStream_t)stream);
}

int smat_plan_spmm(const smat_plan* plan, const void* B, void* C, size_t N, void* stream) {
    clear_error();
    if (!plan) return fail(SMAT_ERR_BAD_ARG, "plan is NULL");
    if (N % 8) return fail(SMAT_ERR_BAD_ARG, "N (%zu) must be a multiple of 8", N);
    if (plan->v.brow_end > plan->v.brow_begin && N && (!C || (plan->v.nnzb && !B)))
        return fail(SMAT_ERR_BAD_ARG, "B or C is NULL");
    if (((uintptr_t)B | (uintptr_t)C) & 15) return fail(SMAT_ERR_BAD_ARG, "B and C must be 16-byte aligned");
    if (N >= ((size_t)1 << 31)) return fail(SMAT_ERR_RANGE, "N beyond 2^31");
    if (int rc = check_plan_device(plan)) return rc;
    return launch_spmm(plan->v, B, C, N, (cudaStream_t)stream);
}

int smat_plan_spmm_host(smat_plan* plan, const void* B_host, void* C_host, size_t N, void* stream) {
    clear_error();
    if (!plan) return fail(SMAT_ERR_BAD_ARG, "plan is NULL");
    if (N % 8) return fail(SMAT_ERR_BAD_ARG, "N (%zu) must be a multiple of 8", N);
    if (N >= ((size_t)1 << 31)) return fail(SMAT_ERR_RANGE, "N beyond 2^31");
    const size_t rows = (plan->v.brow_end - plan->v.brow_begin) * 16, K = plan->v.K;
    if (rows == 0 || N == 0) return SMAT_OK;
    if (!B_host || !C_host) return fail(SMAT_ERR_BAD_ARG, "B_host or C_host is NULL");
    if (int rc = check_plan_device(plan)) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    // B comes in by column chunks as wide as the kernel's widest work item (rows of the [N][K] array: contiguous);
    // every chunk but the last is multiplied for all block-rows as soon as it has arrived; the last chunk is
    // multiplied group range by group range, and the rows of C that it completes go out at once (rows of the
    // row-major C: contiguous), under the multiplication of the next range.
    const size_t W = N >= 512 ? 256 : (N > 128 ? 128 : N);
    const size_t n_chunks = (N + W - 1) / W;
    const size_t n_groups = plan->v.n_groups;
    // ranges of the last chunk: each should still fill the SMs for about one round of work items (shorter launches
    // lose more to partly filled rounds than the overlap of the copy-out wins back); at most 4
    DeviceCtx* ctx = nullptr;
    if (int rc0 = get_device_ctx(&ctx)) return rc0;
    size_t n_ranges = (n_groups * ((W + 127) / 128) + (size_t)ctx->sm_count / 2) / (size_t)ctx->sm_count;
    if (plan->v.sched_list || plan->v.balanced) n_ranges = 1;  // such plans balance a launch over all their groups
    if (const char* e = std::getenv("SMAT_HOST_RANGES")) n_ranges = (size_t)std::atoi(e);  // tuning knob
    if (n_ranges > 4) n_ranges = 4;
    if (n_ranges > n_groups) n_ranges = n_groups;
    if (n_ranges < 1) n_ranges = 1;
    // staging memory and streams: created on first use and kept with the plan (grown when a later call is wider)
    if (!plan->s_in) {
        SMAT_CUDA_TRY(cudaStreamCreateWithFlags(&plan->s_in, cudaStreamNonBlocking));
        SMAT_CUDA_TRY(cudaStreamCreateWithFlags(&plan->s_out, cudaStreamNonBlocking));
        SMAT_CUDA_TRY(cudaEventCreateWithFlags(&plan->ev_start, cudaEventDisableTiming));
    }
    if (plan->host_B_bytes < N * K * 2 || plan->host_C_bytes < rows * N * 2) {
        SMAT_CUDA_TRY(cudaStreamSynchronize(plan->s_in));
        SMAT_CUDA_TRY(cudaStreamSynchronize(plan->s_out));
        SMAT_CUDA_TRY(cudaStreamSynchronize(s));
        SMAT_CUDA_TRY(cudaFree(plan->host_B));
        SMAT_CUDA_TRY(cudaFree(plan->host_C));
        plan->host_B = plan->host_C = nullptr;
        plan->host_B_bytes = plan->host_C_bytes = 0;
        SMAT_CUDA_TRY(cudaMalloc(&plan->host_B, N * K * 2));
        plan->host_B_bytes = N * K * 2;
        SMAT_CUDA_TRY(cudaMalloc(&plan->host_C, rows * N * 2));
        plan->host_C_bytes = rows * N * 2;
    }
    while (plan->ev_in.size() < n_chunks) {
        cudaEvent_t e = nullptr;
        SMAT_CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        plan->ev_in.push_back(e);
    }
    while (plan->ev_done.size() < n_ranges) {
        cudaEvent_t a = nullptr, b = nullptr;
        SMAT_CUDA_TRY(cudaEventCreateWithFlags(&a, cudaEventDisableTiming));
        plan->ev_done.push_back(a);
        SMAT_CUDA_TRY(cudaEventCreateWithFlags(&b, cudaEventDisableTiming));
        plan->ev_out.push_back(b);
    }
    // the copies start after whatever the caller had put on its stream (e.g. the previous call's use of the buffers)
    SMAT_CUDA_TRY(cudaEventRecord(plan->ev_start, s));
    SMAT_CUDA_TRY(cudaStreamWaitEvent(plan->s_in, plan->ev_start, 0));
    SMAT_CUDA_TRY(cudaStreamWaitEvent(plan->s_out, plan->ev_start, 0));
    const char* Bh = static_cast<const char*>(B_host);
    char* Ch = static_cast<char*>(C_host);
    char* Bd = static_cast<char*>(plan->host_B);
    char* Cd = static_cast<char*>(plan->host_C);
    for (size_t j = 0; j < n_chunks; j++) {
        const size_t n0 = j * W, w = (N - n0 < W) ? N - n0 : W;
        SMAT_CUDA_TRY(cudaMemcpyAsync(Bd + n0 * K * 2, Bh + n0 * K * 2, w * K * 2, cudaMemcpyHostToDevice, plan->s_in));
        SMAT_CUDA_TRY(cudaEventRecord(plan->ev_in[j], plan->s_in));
    }
    for (size_t j = 0; j < n_chunks; j++) {
        const size_t n0 = j * W, w = (N - n0 < W) ? N - n0 : W;
        SMAT_CUDA_TRY(cudaStreamWaitEvent(s, plan->ev_in[j], 0));
        if (j + 1 < n_chunks) {
            if (int rc = launch_spmm(plan->v, Bd + n0 * K * 2, Cd + n0 * 2, w, s, nullptr, N)) return rc;
            continue;
        }
        for (size_t r = 0; r < n_ranges; r++) {
            const size_t g0 = n_groups * r / n_ranges, g1 = n_groups * (r + 1) / n_ranges;
            const size_t row0 = g0 * plan->v.rg * 16;
            const size_t row1 = (g1 * plan->v.rg * 16 < rows) ? g1 * plan->v.rg * 16 : rows;
            if (int rc = launch_spmm(plan->v, Bd + n0 * K * 2, Cd + (row0 * N + n0) * 2, w, s, nullptr, N, g0, g1)) return rc;
            SMAT_CUDA_TRY(cudaEventRecord(plan->ev_done[r], s));
            SMAT_CUDA_TRY(cudaStreamWaitEvent(plan->s_out, plan->ev_done[r], 0));
            SMAT_CUDA_TRY(cudaMemcpyAsync(Ch + row0 * N * 2, Cd + row0 * N * 2, (row1 - row0) * N * 2, cudaMemcpyDeviceToHost,
                                          plan->s_out));
            SMAT_CUDA_TRY(cudaEventRecord(plan->ev_out[r], plan->s_out));
        }
    }
    // the caller's stream ends after the last copy out, so that ordering on it covers the whole call
    SMAT_CUDA_TRY(cudaStreamWaitEvent(s, plan->ev_out[n_ranges - 1], 0));
    return SMAT_OK;
}

int smat_plan_info(const smat_plan* plan, int* tall, int* rows_per_item, size_t* steps) {
    clear_error();
    if (!plan) return fail(SMAT_ERR_BAD_ARG, "NULL plan");
    if (tall) *tall = plan->v.tall ? 1 : 0;
    if (rows_per_item) *rows_per_item = (int)plan->v.rg;
    if (steps) *steps = plan->v.total_steps;
    return SMAT_OK;
}

int smat_plan_destroy(smat_plan* plan) {
    clear_error();
    if (!plan) return SMAT_OK;
    if (plan->s_in) {
        cudaStreamSynchronize(plan->s_in);
        cudaStreamSynchronize(plan->s_out);
        cudaStreamDestroy(plan->s_in);
        cudaStreamDestroy(plan->s_out);
        cudaEventDestroy(plan->ev_start);
        for (auto& v : {plan->ev_in, plan->ev_done, plan->ev_out})
            for (cudaEvent_t ev : v) cudaEventDestroy(ev);
        cudaFree(plan->host_B);
        cudaFree(plan->host_C);
    }
    cudaError_t e = cudaFree(plan->buffer);
    const cudaError_t e2 = cudaFree(plan->gsp_buffer);
    const cudaError_t e3 = cudaFree(plan->fix_buffer);
    cudaFree(plan->sched_buffer);
    if (e == cudaSuccess) e = e2;
    if (e == cudaSuccess) e = e3;
    delete plan;
    if (e != cudaSuccess) return fail(SMAT_ERR_CUDA, "cudaFree failed: %s", cudaGetErrorString(e));
    return SMAT_OK;
}

}  // extern "C"
