// Pieces shared by the SpMM kernels (spmm_sm100.cu, spmm_tall_sm100.cu): bounded mbarrier waits and the
// generator of a CTA's sequence of work-item segments.
#pragma once
#include <stdint.h>

#include "ptx_sm100.cuh"
#include "smat_internal.h"

namespace smat {
namespace {

using namespace ptx;

constexpr long long WAIT_LIMIT = 4000000000LL;  // clock cycles (about two seconds)
constexpr int RG = kPlanRowsPerGroup;           // block-rows per work item of the 16-row kernels

__device__ __forceinline__ uint32_t ld_shared_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void st_shared_u16(uint32_t addr, unsigned short v) {
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(v) : "memory");
}
__device__ __forceinline__ void st_shared_u32(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}


#ifdef SMAT_PROFILE
// Development aid (compiled out by default): cycles spent in waits per wait site, summed by the kernels at their end.
static __device__ unsigned long long g_wait_prof[64];
#endif

// Bounded mbarrier wait.  After the first time-out anywhere in the CTA every wait returns at once.
__device__ __forceinline__ void wait_bar(uint32_t bar, uint32_t parity, uint32_t abort_addr, int* status, int code,
                                         long long limit = WAIT_LIMIT) {
    if (mbar_try_wait(bar, parity)) return;
    if (ld_shared_u32(abort_addr)) return;
    const long long t0 = clock64();
    // suspended waits: the warp sleeps in hardware until the phase completes or ~2 us pass
    while (!mbar_try_wait_suspend(bar, parity, 2000u)) {
        if (ld_shared_u32(abort_addr)) return;
        if (clock64() - t0 > limit) {
            st_shared_u32(abort_addr, 1);
            atomicCAS(status, 0, code);
            return;
        }
    }
}

// A segment: steps [k0, k1) of the ns steps of work item `item` (the first step of the item is steps[gs]).
// cut: the item is computed in several segments by as many CTAs and this segment goes to scratch tile `slot`.
struct Seg {
    int item, k0, k1, ns, gs, slot;
    bool cut;
};

// The (item, step) pairs of a launch flattened in item order; position 0 is the first step of the first item.
struct Flat {
    const int* gsp;
    int n_tiles, n_groups;
    long long total;  // number of positions
    __device__ __forceinline__ long long first_of_group(int g) const { return (long long)(__ldg(gsp + g) - __ldg(gsp)) * n_tiles; }
    // first position of CTA c's range when the positions are dealt out in `parts` equal contiguous ranges
    __device__ __forceinline__ long long range_begin(int parts, int c) const { return total * c / parts; }
    // the CTA whose range holds position p: the largest c with range_begin(c) <= p
    __device__ __forceinline__ int range_owner(int parts, long long p) const { return (int)(((p + 1) * parts - 1) / total); }
    // last group whose first position is <= p (groups without steps share their successor's first position)
    __device__ __forceinline__ int group_of(long long p) const {
        int lo = 0, hi = n_groups - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (first_of_group(mid) <= p) lo = mid; else hi = mid - 1;
        }
        return lo;
    }
};

// What a CTA works on, in order.  Three schedules:
//  * round-robin (default): work items go round-robin over the CTAs as long as there is one for every CTA.  The
//    items left for the last round (fewer than CTAs) are each cut into P = #CTAs / #items-left segments of equal
//    step count, one per CTA, so that the last round keeps every SM busy and takes 1/P of an item's time.  All
//    items are cut at the same fractions and consecutive CTAs take consecutive segments, so the CTAs of a round
//    still walk the block-columns in step (what they fetch is shared through L2).
//  * listed (plans whose heaviest group holds many times the average number of steps): every CTA has a fixed list
//    of whole groups, dealt out at plan time heaviest first to the least loaded CTA;
//  * balanced (such plans when whole groups cannot be dealt out evenly, e.g. one group outweighs a CTA's share): the flattened
//    (item, step) sequence is dealt out in equal contiguous ranges, one per CTA, whatever the number and the
//    length of the items; an item that a range boundary falls into is computed in segments.
// A cut item is assembled from fp32 partial tiles: each CTA stores its segment's result to a scratch tile (one
// per CTA, two in the balanced schedule: the head and the tail of its range) and a small second kernel adds them.
// SCHED: 0 = round-robin with a cut last round, 1 = listed, 2 = balanced ranges.
template <int SCHED>
struct SegGen {
    const int* gsp;
    int n_tiles, n_items, n_ctas, cta, item, n_full, P;
    int quantum = 1;  // round-robin schedule: cut items at multiples of this many steps
    bool tail_done;
    Flat flat;
    long long p, p_begin, p_end;
    int g;
    const int* list;      // listed schedule: the groups of this CTA, else null
    int li, li_end, lt;   // position in the list, its end, next tile of the current group
    __device__ __forceinline__ bool next(Seg& s) {
        if (SCHED == 1) {
            if (li >= li_end) return false;
            const int gg = __ldg(list + li);
            const int gs = __ldg(gsp + gg), ns = __ldg(gsp + gg + 1) - gs;
            s.item = gg * n_tiles + lt; s.k0 = 0; s.k1 = ns; s.ns = ns; s.gs = gs; s.cut = false; s.slot = 0;
            if (++lt == n_tiles) { lt = 0; li++; }
            return true;
        }
        if (SCHED == 2) {
            if (p >= p_end) return false;
            while (flat.first_of_group(g + 1) <= p) g++;  // groups without steps are passed over
            const int gs = __ldg(gsp + g), ns = __ldg(gsp + g + 1) - gs;
            const long long item_p0 = flat.first_of_group(g);
            const long long off = p - item_p0;
            const int t = (int)(off / ns), k0 = (int)(off - (long long)t * ns);
            const long long left = p_end - p;
            const int k1 = (left < (long long)(ns - k0)) ? k0 + (int)left : ns;
            s.item = g * n_tiles + t; s.k0 = k0; s.k1 = k1; s.ns = ns; s.gs = gs;
            s.cut = k0 != 0 || k1 != ns;
            // the tail of this CTA's range (the item began inside the range) goes to its second tile
            s.slot = cta * 2 + ((p_begin < item_p0 + (long long)t * ns) ? 1 : 0);
            p += k1 - k0;
            return true;
        }
        if (item < n_full) {
            const int gg = item / n_tiles;
            const int gs = __ldg(gsp + gg), ns = __ldg(gsp + gg + 1) - gs;
            s.item = item; s.k0 = 0; s.k1 = ns; s.ns = ns; s.gs = gs; s.cut = false; s.slot = 0;
            item += n_ctas;
            return true;
        }
        if (tail_done) return false;
        tail_done = true;
        if (cta >= (n_items - n_full) * P) return false;
        const int i = cta / P, j = cta - i * P;
        const int gg = (n_full + i) / n_tiles;
        const int gs = __ldg(gsp + gg), ns = __ldg(gsp + gg + 1) - gs;
        s.item = n_full + i; s.gs = gs; s.ns = ns; s.cut = P > 1; s.slot = cta;
        const unsigned nq = (unsigned)(ns / quantum);  // P <= kMaxTailParts: the products fit 32 bits
        s.k0 = (int)(nq * (unsigned)j / (unsigned)P) * quantum;
        s.k1 = (j + 1 == P) ? ns : (int)(nq * (unsigned)(j + 1) / (unsigned)P) * quantum;
        return true;
    }
};

constexpr int kFixSlotFloats = 2 * RG * 16 * 128;  // one partial tile: up to 2 halves x 16 block-rows x 16 rows x 128 columns
static_assert((size_t)kFixSlotFloats * sizeof(float) == (2 * 16 * 16 * 128) * sizeof(float), "fix_scratch_bytes() assumes this tile size");


}  // namespace
}  // namespace smat
