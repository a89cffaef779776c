// Block-sparse SpMM  C = A_bcsr x B  for NVIDIA B200 (sm_100a): TMA-fed, tcgen05.mma with fp32
// accumulators in tensor memory, persistent warp-specialised CTAs.
//
// Replaces the reference's one-warp-per-tile mma.sync kernel and its launcher
// (mmaCBTKernelSparse / mmaCBTKernel, src/cuda_hgemm/src/mma/mmaCBT.cu:13-88) behind the same
// argument convention and memory layouts.
//
// Mapping onto the tensor core.  A nonzero block is a dense 16x16 contraction, far below the
// 128-row minimum of tcgen05.mma, so the product is computed transposed:
//     C^T[n0:n0+128, 16 rows of block-row r]  +=  B^T[n0:n0+128, 16 k of block-column c] * A_blk^T
//   * MMA "A" operand = a panel of B: 128 n x 16 k, K-major -- exactly how the boundary stores B
//     (element (k, n) at B[n*K + k]); one TMA box {16 k, 128 n} at x = colidx fetches it;
//   * MMA "B" operand = the 16x16 block of A, row-major = N(16 rows) x K(16) K-major -- exactly how
//     BCSR stores it; one TMA box {16, 16} over the value array viewed as [nnzb*16][16];
//   * D = 128 lanes (columns of C) x 16 fp32 columns (rows of the block-row) in tensor memory.
//
// Work decomposition.  A work item is (group of RG consecutive block-rows) x (128 columns of C).
// All RG accumulators of an item live in tensor memory at once (RG*16 columns, NBUF buffers), and
// the item walks the UNION of the group's block-columns in ascending order: each B panel is
// fetched once per item and used by every block of the group in that block-column.  The walk is a
// RG-way merge of the sorted colidx lists done by the producer warp with warp votes
// (min-reduction + ballot), so no auxiliary work list is read from memory.
//
// Warps: 0 = producer (merge + TMA issue), 1 = MMA issuer (one thread) and tensor-memory owner,
// 2..5 = epilogue (tcgen05.ld -> fp16 -> paired, coalesced stores).  Pipelines (mbarrier rings):
// B panels (SP stages), A blocks (SA chunks of 8 blocks), accumulator buffers (NBUF).
//
// Every wait is bounded: when a wait runs out the kernel records a status code, stops waiting
// anywhere in the CTA, and runs to completion (results are then invalid and the host reports
// SMAT_ERR_DEVICE_WAIT).
#include <cuda_fp16.h>
#include <limits.h>

#include "ptx_sm100.cuh"
#include "smat_internal.h"

namespace smat {

using namespace ptx;

namespace {

constexpr int kThreads = 192;
constexpr int NT = 128;      // columns of C per work item = tensor-memory lanes = MMA M
constexpr int SP = 16;       // B-panel pipeline stages
constexpr int SA = 16;       // A-block pipeline chunks
constexpr int CHUNK = 8;     // A blocks per chunk
constexpr int KEYRING = 8;   // per-row colidx prefetch depth (cp.async ring)
constexpr uint32_t PANEL_BYTES = NT * 16 * 2;
constexpr uint32_t ABLK_BYTES = 16 * 16 * 2;
constexpr long long WAIT_LIMIT = 4000000000LL;  // clock cycles (about two seconds)

constexpr uint32_t OFF_PANEL = 0;
constexpr uint32_t OFF_ABLK = OFF_PANEL + SP * PANEL_BYTES;
constexpr uint32_t OFF_KEYS = OFF_ABLK + SA * CHUNK * ABLK_BYTES;
constexpr uint32_t OFF_META = OFF_KEYS + 32 * KEYRING * 4;
constexpr uint32_t OFF_BAR = OFF_META + SP * 8;
constexpr uint32_t N_BARS = 2 * SP + 2 * SA + 4;
constexpr uint32_t OFF_MISC = OFF_BAR + N_BARS * 8;
constexpr uint32_t SMEM_USED = OFF_MISC + 16;
constexpr uint32_t SMEM_BYTES = SMEM_USED + 1024;  // slack for the manual 1024-byte alignment

constexpr uint32_t IDESC = idesc_f16_f32(128, 16);

__device__ __forceinline__ uint32_t ld_shared_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void st_shared_u32(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

// Bounded mbarrier wait.  After the first time-out anywhere in the CTA every wait returns at once.
__device__ __forceinline__ void wait_bar(uint32_t bar, uint32_t parity, uint32_t abort_addr, int* status, int code) {
    if (mbar_try_wait(bar, parity)) return;
    if (ld_shared_u32(abort_addr)) return;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (ld_shared_u32(abort_addr)) return;
        if (clock64() - t0 > WAIT_LIMIT) {
            st_shared_u32(abort_addr, 1);
            atomicCAS(status, 0, code);
            return;
        }
    }
}

template <int RG, int NBUF>
__global__ void __launch_bounds__(kThreads, 1)
spmm_bcsr_tc_kernel(const __grid_constant__ CUtensorMap mapB, const __grid_constant__ CUtensorMap mapA,
                    const int* __restrict__ rowptr, const int* __restrict__ colidx, __half* __restrict__ C,
                    int brow_begin, int brow_end, int N, int n_tiles, int n_items, uint32_t panel_bytes,
                    int* status) {
    static_assert(RG * NBUF * 16 <= 512, "accumulators must fit the 512 tensor-memory columns");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar0 = base + OFF_BAR;
    auto full_p = [&](uint32_t s) { return bar0 + 8 * s; };
    auto empty_p = [&](uint32_t s) { return bar0 + 8 * (SP + s); };
    auto full_a = [&](uint32_t s) { return bar0 + 8 * (2 * SP + s); };
    auto empty_a = [&](uint32_t s) { return bar0 + 8 * (2 * SP + SA + s); };
    auto acc_full = [&](uint32_t b) { return bar0 + 8 * (2 * SP + 2 * SA + b); };
    auto acc_empty = [&](uint32_t b) { return bar0 + 8 * (2 * SP + 2 * SA + 2 + b); };
    const uint32_t tmem_slot = base + OFF_MISC;
    const uint32_t abort_addr = base + OFF_MISC + 4;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < SP; s++) { mbar_init(full_p(s), 1); mbar_init(empty_p(s), 1); }
        for (uint32_t s = 0; s < SA; s++) { mbar_init(full_a(s), 1); mbar_init(empty_a(s), 1); }
        for (uint32_t b = 0; b < 2; b++) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), 4); }
        st_shared_u32(abort_addr, 0);
        fence_barrier_init();
        fence_proxy_async();
        prefetch_tensormap(&mapA);
        prefetch_tensormap(&mapB);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ld_shared_u32(tmem_slot);

    if (warp == 0) {
        // ------------------------------ producer: RG-way merge + TMA issue ------------------------------
        uint32_t ps = 0, cs_base = 0;
        const uint32_t ring = base + OFF_KEYS + (uint32_t)lane * KEYRING * 4;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
            const int g = item / n_tiles, t = item - g * n_tiles;
            const int row = brow_begin + g * RG + lane;
            const bool valid = lane < RG && row < brow_end;
            int p = valid ? __ldg(rowptr + row) : 0;
            const int end = valid ? __ldg(rowptr + row + 1) : 0;
            const int total = __reduce_add_sync(0xffffffffu, end - p);
            if (total == 0) continue;
#pragma unroll
            for (int k = 0; k < KEYRING; k++) {
                if (p + k < end) cp_async_4(ring + (uint32_t)((p + k) % KEYRING) * 4, colidx + p + k);
                cp_async_commit();
            }
            cp_async_wait<KEYRING - 1>();
            int key = (p < end) ? (int)ld_shared_u32(ring + (uint32_t)(p % KEYRING) * 4) : INT_MAX;
            int a_pos = 0;
            const int n0 = t * NT;
            for (;;) {
                const int c = __reduce_min_sync(0xffffffffu, key);
                if (c == INT_MAX) break;
                const bool has = key == c;
                const uint32_t mask = __ballot_sync(0xffffffffu, has);
                const int cnt = __popc(mask);
                const uint32_t s = ps % SP;
                if (lane == 0) {
                    wait_bar(empty_p(s), ((ps / SP) & 1) ^ 1, abort_addr, status, 1);
                    for (int ch = (a_pos + CHUNK - 1) / CHUNK; ch <= (a_pos + cnt - 1) / CHUNK; ++ch) {
                        const uint32_t gc = cs_base + (uint32_t)ch, slot = gc % SA;
                        wait_bar(empty_a(slot), ((gc / SA) & 1) ^ 1, abort_addr, status, 2);
                        const int nb = min(CHUNK, total - CHUNK * ch);
                        mbar_arrive_expect_tx(full_a(slot), (uint32_t)nb * ABLK_BYTES);
                    }
                    st_shared_u32(base + OFF_META + s * 8, mask);
                    st_shared_u32(base + OFF_META + s * 8 + 4, (uint32_t)a_pos);
                    mbar_arrive_expect_tx(full_p(s), panel_bytes);
                    tma_load_2d(base + OFF_PANEL + s * PANEL_BYTES, &mapB, c, n0, full_p(s));
                }
                __syncwarp();
                if (has) {
                    const int q = a_pos + __popc(mask & ((1u << lane) - 1u));
                    const uint32_t gc = cs_base + (uint32_t)(q / CHUNK), slot = gc % SA;
                    tma_load_2d(base + OFF_ABLK + (slot * CHUNK + (uint32_t)(q % CHUNK)) * ABLK_BYTES, &mapA, 0, p * 16,
                                full_a(slot));
                    if (p + KEYRING < end) cp_async_4(ring + (uint32_t)(p % KEYRING) * 4, colidx + p + KEYRING);
                    cp_async_commit();
                    p++;
                    cp_async_wait<KEYRING - 1>();
                    key = (p < end) ? (int)ld_shared_u32(ring + (uint32_t)(p % KEYRING) * 4) : INT_MAX;
                }
                __syncwarp();
                a_pos += cnt;
                ps++;
            }
            cp_async_wait<0>();
            cs_base += (uint32_t)((total + CHUNK - 1) / CHUNK);
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (one thread) ------------------------------
        if (lane == 0) {
            uint32_t ps = 0, cs_base = 0, it = 0;
            for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++it) {
                const int g = item / n_tiles;
                const int r0 = brow_begin + g * RG;
                const int r1 = min(r0 + RG, brow_end);
                const int total = __ldg(rowptr + r1) - __ldg(rowptr + r0);
                const uint32_t buf = it % NBUF;
                wait_bar(acc_empty(buf), ((it / NBUF) & 1) ^ 1, abort_addr, status, 3);
                tc_fence_after();
                uint32_t started = 0;
                int a_done = 0;
                while (a_done < total) {
                    const uint32_t s = ps % SP;
                    wait_bar(full_p(s), (ps / SP) & 1, abort_addr, status, 4);
                    uint32_t mask = ld_shared_u32(base + OFF_META + s * 8);
                    if (ld_shared_u32(abort_addr)) mask = mask ? mask : 1u;  // guarantee progress after a time-out
                    tc_fence_after();
                    const uint64_t adesc = smem_desc_k_sw32(base + OFF_PANEL + s * PANEL_BYTES);
                    while (mask && a_done < total) {
                        const int r = __ffs(mask) - 1;
                        mask &= mask - 1;
                        const uint32_t gc = cs_base + (uint32_t)(a_done / CHUNK), slot = gc % SA;
                        if (a_done % CHUNK == 0) {
                            wait_bar(full_a(slot), (gc / SA) & 1, abort_addr, status, 5);
                            tc_fence_after();
                        }
                        const uint64_t bdesc =
                            smem_desc_k_sw32(base + OFF_ABLK + (slot * CHUNK + (uint32_t)(a_done % CHUNK)) * ABLK_BYTES);
                        mma_f16_ss(tmem_base + (buf * RG + (uint32_t)r) * 16, adesc, bdesc, IDESC, (started >> r) & 1u);
                        started |= 1u << r;
                        a_done++;
                        if (a_done % CHUNK == 0 || a_done == total) tc_commit(empty_a(slot));
                    }
                    tc_commit(empty_p(s));
                    ps++;
                }
                tc_commit(acc_full(buf));
                cs_base += (uint32_t)((total + CHUNK - 1) / CHUNK);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------ epilogue: tensor memory -> fp16 -> C ------------------------------
        const int quarter = warp & 3;  // a warp may only read tensor-memory lanes [32*(warp%4), +32)
        const bool odd = lane & 1;
        uint32_t it = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++it) {
            const int g = item / n_tiles, t = item - g * n_tiles;
            const int r0 = brow_begin + g * RG;
            const int nrows = min(RG, brow_end - r0);
            const int lo = (lane < nrows) ? __ldg(rowptr + r0 + lane) : 0;
            const int hi = (lane < nrows) ? __ldg(rowptr + r0 + lane + 1) : 0;
            const uint32_t nonempty = __ballot_sync(0xffffffffu, hi > lo);
            const uint32_t buf = it % NBUF;
            wait_bar(acc_full(buf), (it / NBUF) & 1, abort_addr, status, 6);
            tc_fence_after();
            const int n = t * NT + quarter * 32 + lane;
            __half* cbase = C + ((size_t)(r0 - brow_begin) * 16 + (odd ? 8 : 0)) * (size_t)N + (size_t)(n & ~1);
            for (int r = 0; r < nrows; r++) {
                uint32_t v[16];
                if ((nonempty >> r) & 1u) {
                    tmem_ld_x16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (buf * RG + (uint32_t)r) * 16, v);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 16; i++) v[i] = 0u;
                }
                if (r == nrows - 1) {
                    // every accumulator of this buffer has been read: hand it back to the MMA warp
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty(buf));
                }
                __half* crow = cbase + (size_t)r * 16 * (size_t)N;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    // lane pairs exchange halves: even lanes keep rows 0..7, odd lanes rows 8..15,
                    // each for the two adjacent columns (n & ~1, n | 1) -> one 4-byte store per row
                    const float keep = __uint_as_float(odd ? v[i + 8] : v[i]);
                    const float send = __uint_as_float(odd ? v[i] : v[i + 8]);
                    const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
                    const __half2 h = odd ? __floats2half2_rn(recv, keep) : __floats2half2_rn(keep, recv);
                    if (n < N) *reinterpret_cast<__half2*>(crow + (size_t)i * (size_t)N) = h;
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (ld_shared_u32(abort_addr)) {
        // a wait ran out somewhere: give copies still in flight time to land before the CTA retires
        for (int i = 0; i < 64; i++) __nanosleep(1000);
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

__global__ void zero_rows_kernel(uint4* dst, size_t n16) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n16; i += stride) dst[i] = make_uint4(0, 0, 0, 0);
}

}  // namespace

int g_spmm_variant = 0;

int launch_spmm(const void* vals, const int* rowptr, const int* colidx, const void* B, void* C, size_t M, size_t N,
                size_t K, size_t nnzb, size_t brow_begin, size_t brow_end, cudaStream_t stream) {
    DeviceCtx* ctx = nullptr;
    if (int rc = get_device_ctx(&ctx)) return rc;
    const size_t nb_rows = brow_end - brow_begin;
    if (nb_rows == 0 || N == 0) return SMAT_OK;
    (void)M;
    if (nnzb == 0) {
        const size_t n16 = nb_rows * 16 * N * 2 / 16;
        zero_rows_kernel<<<ctx->sm_count * 4, 256, 0, stream>>>(reinterpret_cast<uint4*>(C), n16);
        count_launch();
        SMAT_CUDA_TRY(cudaGetLastError());
        return SMAT_OK;
    }
    const uint32_t panel_rows = (uint32_t)(N < (size_t)NT ? N : (size_t)NT);
    CUtensorMap mapB, mapA;
    if (int rc = encode_tensor_map_2d_f16(&mapB, B, K, N, K * 2, 16, panel_rows, 1, 0)) return rc;
    if (int rc = encode_tensor_map_2d_f16(&mapA, vals, 16, nnzb * 16, 32, 16, 16, 1, 256)) return rc;

    const int n_tiles = (int)((N + NT - 1) / NT);
    int variant = g_spmm_variant;
    if (variant == 0) {
        const size_t items32 = ((nb_rows + 31) / 32) * (size_t)n_tiles;
        variant = (items32 >= (size_t)ctx->sm_count && nnzb / (nb_rows ? nb_rows : 1) >= 32) ? 2 : 1;
    }
    const int rg = (variant == 2) ? 32 : 16;
    const size_t n_items = ((nb_rows + rg - 1) / rg) * (size_t)n_tiles;
    if (n_items > (size_t)INT_MAX) return fail(SMAT_ERR_RANGE, "too many work items (%zu)", n_items);
    const int grid = (int)(n_items < (size_t)ctx->sm_count ? n_items : (size_t)ctx->sm_count);
    const uint32_t panel_bytes = panel_rows * 32u;

    auto launch = [&](auto kernel) -> int {
        SMAT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
        kernel<<<grid, kThreads, SMEM_BYTES, stream>>>(mapB, mapA, rowptr, colidx, reinterpret_cast<__half*>(C),
                                                       (int)brow_begin, (int)brow_end, (int)N, n_tiles, (int)n_items,
                                                       panel_bytes, ctx->d_status);
        count_launch();
        SMAT_CUDA_TRY(cudaGetLastError());
        return SMAT_OK;
    };
    if (variant == 2) return launch(spmm_bcsr_tc_kernel<32, 1>);
    return launch(spmm_bcsr_tc_kernel<16, 2>);
}

}  // namespace smat
