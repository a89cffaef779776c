// extern "C" entry points of libsmat_b200.so that touch the GPU, plus the shared host plumbing
// (per-thread error text, per-device context, tensor-map encoding).
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "smat_internal.h"
#include "spmm_sched.cuh"

namespace smat {

namespace {
thread_local char t_error[512] = "";
std::atomic<long long> g_launches{0};
std::mutex g_ctx_mutex;
constexpr int kMaxDevices = 64;
DeviceCtx g_ctx[kMaxDevices];
}  // namespace

namespace {
// One thread waits, with the kernels' bounded wait and a short limit, on a barrier that nothing ever completes.
__global__ void wait_selftest_kernel(int* status, long long limit) {
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        ptx::mbar_init(ptx::smem_u32(&bar), 1);
        abort_flag = 0;
        ptx::fence_barrier_init();
        wait_bar(ptx::smem_u32(&bar), 0, ptx::smem_u32(&abort_flag), status, 90, limit);
    }
}
}  // namespace

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
    return code;
}
void clear_error() { t_error[0] = 0; }
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int get_device_ctx(DeviceCtx** out) {
    int dev = -1;
    SMAT_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(SMAT_ERR_RANGE, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_ctx_mutex);
    DeviceCtx& c = g_ctx[dev];
    if (c.device != dev) {
        cudaDeviceProp prop;
        SMAT_CUDA_TRY(cudaGetDeviceProperties(&prop, dev));
        if (prop.major != 10)
            return fail(SMAT_ERR_CUDA, "device %d is sm_%d%d; this library holds sm_100a code only", dev, prop.major,
                        prop.minor);
        // Stream-ordered scratch (the per-call plans of smat_spmm_bcsr_f16) comes from a pool of the library's own,
        // which keeps what it has been given; the process's default pool is left as the application configured it.
        cudaMemPoolProps props = {};
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = dev;
        cudaMemPool_t pool = nullptr;
        SMAT_CUDA_TRY(cudaMemPoolCreate(&pool, &props));
        unsigned long long keep = ~0ull;
        SMAT_CUDA_TRY(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
        c.pool = pool;
        int* st = nullptr;
        SMAT_CUDA_TRY(cudaMalloc(&st, 64));
        SMAT_CUDA_TRY(cudaMemset(st, 0, 64));
        c.sm_count = prop.multiProcessorCount;
        c.d_status = st;
        c.device = dev;
    }
    *out = &c;
    return SMAT_OK;
}

int encode_tensor_map_2d_f16(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_pitch_bytes,
                             uint32_t box_inner, uint32_t box_outer, int swizzle_bytes, int l2_promo_bytes) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        SMAT_CUDA_TRY(cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000, cudaEnableDefault, &qres));
        if (qres != cudaDriverEntryPointSuccess || !fn)
            return fail(SMAT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
        encode = (EncodeFn)fn;
    }
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {row_pitch_bytes};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    const CUtensorMapL2promotion promo = l2_promo_bytes >= 256   ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B
                                         : l2_promo_bytes >= 128 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                                         : l2_promo_bytes >= 64  ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
                                                                 : CU_TENSOR_MAP_L2_PROMOTION_NONE;
    const CUresult r =
        encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE,
               swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
               : swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                     : CU_TENSOR_MAP_SWIZZLE_NONE,
               promo,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(SMAT_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (dims %llu x %llu, pitch %llu, box %u x %u)",
                    (int)r, (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)row_pitch_bytes,
                    box_inner, box_outer);
    return SMAT_OK;
}

int check_spmm_args(const void* vals, const int* rowptr, const int* colidx, const void* B, const void* C, size_t M,
                           size_t N, size_t K, size_t nnzb) {
    if (M % 16 || K % 16) return fail(SMAT_ERR_BAD_ARG, "M (%zu) and K (%zu) must be multiples of 16", M, K);
    if (N % 8) return fail(SMAT_ERR_BAD_ARG, "N (%zu) must be a multiple of 8", N);
    if (!rowptr) return fail(SMAT_ERR_BAD_ARG, "bcsrRowPtrA is NULL");
    if (nnzb && (!vals || !colidx)) return fail(SMAT_ERR_BAD_ARG, "bcsrValuesA / bcsrColIdxA is NULL with nonzeroBlocks > 0");
    if (M && N && (!C || (nnzb && !B))) return fail(SMAT_ERR_BAD_ARG, "B or C is NULL");
    if (((uintptr_t)vals | (uintptr_t)B | (uintptr_t)C) & 15)
        return fail(SMAT_ERR_BAD_ARG, "bcsrValuesA, B and C must be 16-byte aligned");
    if (nnzb * 16 >= ((size_t)1 << 31)) return fail(SMAT_ERR_RANGE, "nonzeroBlocks (%zu) exceeds 2^27 - 1", nnzb);
    if (K >= ((size_t)1 << 31) || N >= ((size_t)1 << 31) || M / 16 >= ((size_t)1 << 31))
        return fail(SMAT_ERR_RANGE, "dimension beyond 2^31");
    return SMAT_OK;
}

}  // namespace smat

using namespace smat;

extern "C" {

// One multiplication with a plan (walk order + packed copy of the blocks) built on the fly in
// stream-ordered scratch memory.
static int spmm_transient_plan(const void* vals, const int* rowptr, const int* colidx, const void* B, void* C, size_t N,
                               size_t K, size_t nnzb, size_t brow_begin, size_t brow_end, cudaStream_t stream) {
    if (brow_end == brow_begin || N == 0) return SMAT_OK;
    PlanView v;
    v.rowptr = rowptr;
    v.K = K;
    v.nnzb = nnzb;
    v.brow_begin = brow_begin;
    v.brow_end = brow_end;
    DeviceCtx* ctx = nullptr;
    if (int rc0 = get_device_ctx(&ctx)) return rc0;
    const size_t rg = choose_rows_per_group(brow_end - brow_begin, N, ctx->sm_count, true, nnzb, K);
    const PlanSizes sz = plan_sizes(nnzb, brow_begin, brow_end, rg);
    v.n_groups = sz.n_groups;
    v.rg = rg;
    if (nnzb == 0) return launch_spmm(v, B, C, N, stream);
    void* buf = nullptr;
    const size_t plan_bytes = (sz.gsp_bytes + sz.steps_bytes + sz.blk_bytes + sz.packed_bytes + 255) / 256 * 256;
    SMAT_CUDA_TRY(cudaMallocFromPoolAsync(&buf, plan_bytes + fix_scratch_bytes(ctx->sm_count), ctx->pool, stream));
    char* b = static_cast<char*>(buf);
    v.fix_scratch = reinterpret_cast<float*>(b + plan_bytes);
    v.gsp = reinterpret_cast<int*>(b);
    v.steps = b + sz.gsp_bytes;
    v.blk = reinterpret_cast<int*>(b + sz.gsp_bytes + sz.steps_bytes);
    v.packed = b + sz.gsp_bytes + sz.steps_bytes + sz.blk_bytes;
    int rc = plan_count_async(rowptr, colidx, K, nnzb, brow_begin, brow_end, rg, reinterpret_cast<int*>(b), stream);
    if (rc == SMAT_OK)
        rc = plan_fill_async(rowptr, colidx, K, nnzb, brow_begin, brow_end, rg, v.gsp, b + sz.gsp_bytes,
                             reinterpret_cast<int*>(b + sz.gsp_bytes + sz.steps_bytes), stream);
    if (rc == SMAT_OK)
        rc = pack_values_async(rowptr, vals, v.gsp, v.steps, v.blk, b + sz.gsp_bytes + sz.steps_bytes + sz.blk_bytes, brow_begin,
                               brow_end, rg, nnzb, stream);
    if (rc == SMAT_OK) rc = launch_spmm(v, B, C, N, stream);
    const cudaError_t e = cudaFreeAsync(buf, stream);
    if (rc == SMAT_OK && e != cudaSuccess) return fail(SMAT_ERR_CUDA, "cudaFreeAsync failed: %s", cudaGetErrorString(e));
    return rc;
}

int smat_spmm_bcsr_f16(const void* vals, const int* rowptr, const int* colidx, const void* B, void* C, size_t M, size_t N,
                       size_t K, size_t nnzb, const int* blockInfo, const int* relMap, void* stream) {
    (void)blockInfo;
    (void)relMap;
    clear_error();
    if (int rc = check_spmm_args(vals, rowptr, colidx, B, C, M, N, K, nnzb)) return rc;
    return spmm_transient_plan(vals, rowptr, colidx, B, C, N, K, nnzb, 0, M / 16, (cudaStream_t)stream);
}

int smat_spmm_bcsr_f16_rows(const void* vals, const int* rowptr, const int* colidx, const void* B, void* C, size_t M,
                            size_t N, size_t K, size_t nnzb, size_t brow_begin, size_t brow_end, void* stream) {
    clear_error();
    if (int rc = check_spmm_args(vals, rowptr, colidx, B, C, M, N, K, nnzb)) return rc;
    if (brow_begin > brow_end || brow_end > M / 16)
        return fail(SMAT_ERR_BAD_ARG, "block-row range [%zu, %zu) outside [0, %zu]", brow_begin, brow_end, M / 16);
    return spmm_transient_plan(vals, rowptr, colidx, B, C, N, K, nnzb, brow_begin, brow_end, (cudaStream_t)stream);
}

int smat_spmm_set_variant(int variant) {
    clear_error();
    if (variant < 0 || variant > 4) return fail(SMAT_ERR_BAD_ARG, "unknown SpMM variant %d", variant);
    g_spmm_variant = variant;
    return SMAT_OK;
}

int smat_device_status(void* stream) {
    clear_error();
    DeviceCtx* ctx = nullptr;
    if (int rc = get_device_ctx(&ctx)) return rc;
    SMAT_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    int st = 0;
    SMAT_CUDA_TRY(cudaMemcpy(&st, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (st != 0) SMAT_CUDA_TRY(cudaMemset(ctx->d_status, 0, sizeof(int)));
    int st_static = 0;  // the word of the allocation-free entry point lives in its fixed array
    if (int rc = static_status_take(&st_static)) return rc;
    if (st == 0) st = st_static;
    if (st >= 100)
        return fail(SMAT_ERR_RANGE, "the BCSR arrays are inconsistent (device check %d: %s); the output is invalid", st,
                    st == kStatusBadRowptr ? "bcsrRowPtr disagrees with nonzeroBlocks"
                                           : "a block column is out of range or a block-row's columns are not ascending");
    if (st != 0) return fail(SMAT_ERR_DEVICE_WAIT, "a kernel gave up a bounded wait (site code %d); its output is invalid", st);
    return SMAT_OK;
}

int smat_selftest_wait_timeout(void* stream) {
    clear_error();
    DeviceCtx* ctx = nullptr;
    if (int rc = get_device_ctx(&ctx)) return rc;
    wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(ctx->d_status, 400000LL);  // about 0.2 ms
    count_launch();
    SMAT_CUDA_TRY(cudaGetLastError());
    return SMAT_OK;
}

long long smat_launch_count(void) { return g_launches.load(); }

const char* smat_last_error_string(void) { return t_error; }

}  // extern "C"
