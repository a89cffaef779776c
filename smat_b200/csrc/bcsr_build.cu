// Device-side CSR -> 16x16 BCSR builder.
//
// Replaces the host routine SparseMatrix::csrToBcsr and the uploads that follow it
// (src/cuda_hgemm/src/common/matrix.h:376-502, 185-199).  The result is bit-identical to the
// reference's arrays:
//   * a block exists iff it holds at least one stored CSR entry, whatever its value (:388-404);
//   * blocks of a block-row appear in ascending block-column order, and bcsrColIdx holds the ELEMENT
//     column of the block's left edge (:441-460);
//   * values are zero-filled and entry (row, col) lands at block*256 + (row%16)*16 + col%16 (:482);
//     of several entries with the same (row, col) the last one in CSR order wins (:470-487).
// The reference's two dense Mb*Kb int maps (:381, :425-431) are not materialised: one CTA owns one
// block-row at a time and keeps that block-row's column-block bitmap in shared memory.
//
// One CTA of 512 threads per block-row (grid-stride); warp w walks CSR row 16*blockrow + w.
#include <cuda_fp16.h>

#include "smat_internal.h"

namespace smat {
namespace {

constexpr int kBuildThreads = 512;

// Marks the block-columns touched by the 16 rows of block-row `br` in the shared bitmap.
__device__ __forceinline__ void mark_block_columns(const int* __restrict__ rowptr, const int* __restrict__ colidx, int br,
                                                   uint32_t* bitmap, int words) {
    for (int w = threadIdx.x; w < words; w += blockDim.x) bitmap[w] = 0u;
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = br * 16 + warp;
    const int beg = __ldg(rowptr + row), end = __ldg(rowptr + row + 1);
    for (int j = beg + lane; j < end; j += 32) {
        const int bc = __ldg(colidx + j) >> 4;
        atomicOr(&bitmap[bc >> 5], 1u << (bc & 31));
    }
    __syncthreads();
}

__device__ __forceinline__ int block_sum(int v, int* scratch) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    v = __reduce_add_sync(0xffffffffu, v);
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    int total = 0;
    if (warp == 0) {
        int x = lane < (int)(blockDim.x >> 5) ? scratch[lane] : 0;
        total = __reduce_add_sync(0xffffffffu, x);
        if (lane == 0) scratch[32] = total;
    }
    __syncthreads();
    total = scratch[32];
    __syncthreads();
    return total;
}

// counts[br + 1] = number of nonzero blocks of block-row br (counts[0] is set to 0).
__global__ void __launch_bounds__(kBuildThreads)
bcsr_count_kernel(const int* __restrict__ rowptr, const int* __restrict__ colidx, int Mb, int words, int* counts) {
    extern __shared__ uint32_t sm[];
    uint32_t* bitmap = sm;
    __shared__ int red[33];
    for (int br = blockIdx.x; br < Mb; br += gridDim.x) {
        mark_block_columns(rowptr, colidx, br, bitmap, words);
        int c = 0;
        for (int w = threadIdx.x; w < words; w += blockDim.x) c += __popc(bitmap[w]);
        c = block_sum(c, red);
        if (threadIdx.x == 0) counts[br + 1] = c;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) counts[0] = 0;
}

// In-place inclusive scan of data[0..n) by a single CTA (n = Mb + 1 is small next to nnz).
__global__ void __launch_bounds__(1024) scan_inplace_kernel(int* data, int n) {
    __shared__ int warp_tot[32];
    __shared__ int carry_s;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    for (int base = 0; base < n; base += 1024) {
        const int i = base + threadIdx.x;
        int v = i < n ? data[i] : 0;
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
        const int carry = carry_s;
        v += carry + (warp ? warp_tot[warp - 1] : 0);
        if (i < n) data[i] = v;
        __syncthreads();
        if (threadIdx.x == 1023) carry_s = v;
        __syncthreads();
    }
}

__global__ void __launch_bounds__(kBuildThreads)
bcsr_fill_kernel(const int* __restrict__ rowptr, const int* __restrict__ colidx, const __half* __restrict__ vals, int Mb,
                 int words, const int* __restrict__ brp, int* __restrict__ bcol, __half* __restrict__ bvals) {
    extern __shared__ uint32_t sm[];
    uint32_t* bitmap = sm;          // [words]
    uint32_t* prefix = sm + words;  // [words] exclusive prefix of popcounts
    __shared__ int warp_tot[16];
    __shared__ int carry_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int br = blockIdx.x; br < Mb; br += gridDim.x) {
        mark_block_columns(rowptr, colidx, br, bitmap, words);
        const int first = __ldg(brp + br);
        const int nblk = __ldg(brp + br + 1) - first;
        if (nblk == 0) { __syncthreads(); continue; }
        // exclusive scan of popcounts over the bitmap words
        if (threadIdx.x == 0) carry_s = 0;
        __syncthreads();
        for (int base = 0; base < words; base += kBuildThreads) {
            const int w = base + threadIdx.x;
            const int c = w < words ? __popc(bitmap[w]) : 0;
            int v = c;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, v, d);
                if (lane >= d) v += t;
            }
            if (lane == 31) warp_tot[warp] = v;
            __syncthreads();
            int woff = 0;
            for (int k = 0; k < warp; k++) woff += warp_tot[k];
            const int carry = carry_s;
            if (w < words) prefix[w] = (uint32_t)(carry + woff + v - c);
            __syncthreads();
            if (threadIdx.x == kBuildThreads - 1) carry_s = carry + woff + v;
            __syncthreads();
        }
        // column index of every block, ascending
        for (int w = threadIdx.x; w < words; w += blockDim.x) {
            uint32_t bits = bitmap[w];
            int pos = first + (int)prefix[w];
            while (bits) {
                const int b = __ffs(bits) - 1;
                bits &= bits - 1;
                bcol[pos++] = ((w << 5) + b) << 4;
            }
        }
        // zero this block-row's values (nblk * 512 bytes, 16-byte stores)
        uint4* z = reinterpret_cast<uint4*>(bvals + (size_t)first * 256);
        for (int i = threadIdx.x; i < nblk * 32; i += blockDim.x) z[i] = make_uint4(0, 0, 0, 0);
        __syncthreads();
        // scatter: warp w owns CSR row 16*br + w and walks it in order, 32 entries at a time; inside
        // a 32-entry step the highest lane holding a given column stores, so the last entry wins
        const int row = br * 16 + warp;
        const int beg = __ldg(rowptr + row), end = __ldg(rowptr + row + 1);
        for (int j0 = beg; j0 < end; j0 += 32) {
            const int j = j0 + lane;
            const bool act = j < end;
            const int col = act ? __ldg(colidx + j) : -1 - lane;
            const uint32_t same = __match_any_sync(0xffffffffu, col);
            if (act && lane == 31 - __clz(same)) {
                const int bc = col >> 4;
                const int slot = first + (int)prefix[bc >> 5] + __popc(bitmap[bc >> 5] & ((1u << (bc & 31)) - 1u));
                bvals[(size_t)slot * 256 + warp * 16 + (col & 15)] = vals[j];
            }
            __syncwarp();
        }
        __syncthreads();
    }
}

int bitmap_words(size_t K, int* words, size_t factor) {
    const size_t Kb = K / 16;
    const size_t w = (Kb + 31) / 32;
    if (w * 4 * factor > 192 * 1024) return fail(SMAT_ERR_RANGE, "K = %zu exceeds the builder's limit of 12582912", K);
    *words = (int)(w ? w : 1);
    return SMAT_OK;
}

}  // namespace
}  // namespace smat

using namespace smat;

extern "C" {

int smat_bcsr_count(const int* csr_rowptr, const int* csr_colidx, size_t M, size_t K, size_t nnz, int* bcsr_rowptr,
                    size_t* nnzb_out, void* stream_) {
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    if (M % 16 || K % 16) return fail(SMAT_ERR_BAD_ARG, "M (%zu) and K (%zu) must be multiples of 16", M, K);
    if (!csr_rowptr || !bcsr_rowptr || !nnzb_out || (nnz && !csr_colidx)) return fail(SMAT_ERR_BAD_ARG, "NULL argument");
    if (M / 16 >= ((size_t)1 << 31) - 1 || nnz >= ((size_t)1 << 31)) return fail(SMAT_ERR_RANGE, "size beyond 2^31");
    DeviceCtx* ctx = nullptr;
    if (int rc = get_device_ctx(&ctx)) return rc;
    int words = 1;
    if (int rc = bitmap_words(K, &words, 2)) return rc;
    const int Mb = (int)(M / 16);
    if (Mb > 0) {
        const size_t smem = (size_t)words * 4;
        SMAT_CUDA_TRY(cudaFuncSetAttribute(bcsr_count_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        const int grid = Mb < ctx->sm_count * 4 ? Mb : ctx->sm_count * 4;
        bcsr_count_kernel<<<grid, kBuildThreads, smem, stream>>>(csr_rowptr, csr_colidx, Mb, words, bcsr_rowptr);
        count_launch();
        SMAT_CUDA_TRY(cudaGetLastError());
    } else {
        SMAT_CUDA_TRY(cudaMemsetAsync(bcsr_rowptr, 0, sizeof(int), stream));
    }
    scan_inplace_kernel<<<1, 1024, 0, stream>>>(bcsr_rowptr, Mb + 1);
    count_launch();
    SMAT_CUDA_TRY(cudaGetLastError());
    // the total is the last entry of the scanned array (the caller's own buffer: concurrent calls do not meet)
    int total = 0;
    SMAT_CUDA_TRY(cudaMemcpyAsync(&total, bcsr_rowptr + Mb, sizeof(total), cudaMemcpyDeviceToHost, stream));
    SMAT_CUDA_TRY(cudaStreamSynchronize(stream));
    *nnzb_out = (size_t)total;
    return SMAT_OK;
}

int smat_bcsr_fill(const int* csr_rowptr, const int* csr_colidx, const void* csr_vals, size_t M, size_t K, size_t nnz,
                   const int* bcsr_rowptr, int* bcsr_colidx, void* bcsr_vals, size_t nnzb, void* stream_) {
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    if (M % 16 || K % 16) return fail(SMAT_ERR_BAD_ARG, "M (%zu) and K (%zu) must be multiples of 16", M, K);
    if (nnzb == 0 || M == 0) return SMAT_OK;
    if (!csr_rowptr || !csr_colidx || !csr_vals || !bcsr_rowptr || !bcsr_colidx || !bcsr_vals || nnz == 0)
        return fail(SMAT_ERR_BAD_ARG, "NULL argument");
    if ((uintptr_t)bcsr_vals & 15) return fail(SMAT_ERR_BAD_ARG, "bcsr_vals must be 16-byte aligned");
    DeviceCtx* ctx = nullptr;
    if (int rc = get_device_ctx(&ctx)) return rc;
    int words = 1;
    if (int rc = bitmap_words(K, &words, 2)) return rc;
    const int Mb = (int)(M / 16);
    const size_t smem = (size_t)words * 8;
    SMAT_CUDA_TRY(cudaFuncSetAttribute(bcsr_fill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int grid = Mb < ctx->sm_count * 4 ? Mb : ctx->sm_count * 4;
    bcsr_fill_kernel<<<grid, kBuildThreads, smem, stream>>>(csr_rowptr, csr_colidx, reinterpret_cast<const __half*>(csr_vals),
                                                            Mb, words, bcsr_rowptr, bcsr_colidx,
                                                            reinterpret_cast<__half*>(bcsr_vals));
    count_launch();
    SMAT_CUDA_TRY(cudaGetLastError());
    return SMAT_OK;
}

}  // extern "C"
