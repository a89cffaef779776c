// smat_spmm_bcsr_f16_static: the one-call SpMM for hosts that must not allocate device memory.
//
// Who needs it: code that runs where cudaMalloc / cudaFree (also the stream-ordered allocator and
// any framework allocator on top of them) is off limits -- a latency-critical serving loop whose
// memory budget is fixed at start-up, a library callback invoked while another component holds the
// allocator or device-synchronising locks, a process that has handed all remaining device memory
// to a pool it does not own.  smat_spmm_bcsr_f16 builds its plan (walk order plus a copy of the
// blocks in that order) in freshly allocated scratch on every call; this variant builds the same
// plan in a fixed array that is part of the library image, so the call itself allocates nothing
// and frees nothing.
//
// Cost and limits: the array occupies kStaticScratchBytes (17.5 MB) on every GPU that loads
// the library, until the process exits, and therefore bounds the problem: at most
// SMAT_STATIC_MAX_BLOCKS nonzero blocks and SMAT_STATIC_MAX_ROWS rows.  Larger inputs are refused
// with SMAT_ERR_RANGE; use the plan API for them.
//
// Sharing: all calls on a device use the same array.  It keeps whatever the previous call left; the
// plan build overwrites every entry the multiplication reads, so nothing stale is consumed -- but two
// calls that overlap on the GPU (different streams, or different host threads without external
// ordering) race on it.  Calls on one stream are safe back to back.
//
// Errors found on the device (a bounded wait that ran out, a row pointer that disagrees with
// nonzeroBlocks) are recorded in a status word inside the array.  The word starts at zero when the
// library is loaded and stays set until smat_device_status reads it, which reports and clears it
// together with the word of the allocating entry points; a later static call never clears it.
//
// First call per device: looks up the device address of the array (cudaGetSymbolAddress, with that
// device current) and the SM count.  No allocation happens, but it is a set-up step: make it before
// beginning a stream capture.
#include <mutex>

#include "smat_internal.h"

namespace smat {
namespace {

constexpr size_t kMaxBlocks = 32768;          // SMAT_STATIC_MAX_BLOCKS
constexpr size_t kMaxRows = 1048576;          // SMAT_STATIC_MAX_ROWS
constexpr size_t kMaxGroups = kMaxRows / 16 / 4;  // the smallest group height (SMAT_ROWS_PER_GROUP override) is 4 block-rows
constexpr size_t kGspBytes = ((kMaxGroups + 2) * sizeof(int) + 255) / 256 * 256;  // prefix of step counts + the largest count
constexpr size_t kStepsBytes = kMaxBlocks * 16;   // a group never has more steps than blocks
constexpr size_t kBlkBytes = kMaxBlocks * sizeof(int);
constexpr size_t kPackedBytes = kMaxBlocks * 512;  // the blocks in walk order
constexpr size_t kStatusBytes = 256;
constexpr size_t kStaticScratchBytes = kGspBytes + kStepsBytes + kBlkBytes + kPackedBytes + kStatusBytes;

// In host code this name is only a handle for cudaGetSymbolAddress; the device address it yields is
// what the kernels receive.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
struct StaticDev {
    bool ready = false;
    unsigned char* base = nullptr;
    DeviceCtx ctx;
} g_dev[kMaxDevices];

// Per-device set-up with that device current.  Allocates nothing.
int static_device(StaticDev** out) {
    int dev = -1;
    SMAT_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(SMAT_ERR_RANGE, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_mutex);
    StaticDev& d = g_dev[dev];
    if (!d.ready) {
        void* p = nullptr;
        SMAT_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
        int major = 0, sms = 0;
        SMAT_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        SMAT_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        if (major != 10) return fail(SMAT_ERR_CUDA, "device %d is not sm_100; this library holds sm_100a code only", dev);
        d.base = static_cast<unsigned char*>(p);
        d.ctx.device = dev;
        d.ctx.sm_count = sms;
        d.ctx.d_status = reinterpret_cast<int*>(d.base + kGspBytes + kStepsBytes + kBlkBytes + kPackedBytes);
        d.ready = true;
    }
    *out = &d;
    return SMAT_OK;
}

}  // namespace

// Reads (and, when set, clears) the status word of the fixed array on the current device; 0 when the static entry
// point has not been used on it.  The caller has synchronised the stream.  Allocates nothing.
int static_status_take(int* out) {
    *out = 0;
    int dev = -1;
    SMAT_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return SMAT_OK;
    int* word = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (!g_dev[dev].ready) return SMAT_OK;
        word = g_dev[dev].ctx.d_status;
    }
    SMAT_CUDA_TRY(cudaMemcpy(out, word, sizeof(int), cudaMemcpyDeviceToHost));
    if (*out != 0) SMAT_CUDA_TRY(cudaMemset(word, 0, sizeof(int)));
    return SMAT_OK;
}

}  // namespace smat

using namespace smat;

extern "C" int smat_spmm_bcsr_f16_static(const void* vals, const int* rowptr, const int* colidx, const void* B, void* C,
                                         size_t M, size_t N, size_t K, size_t nnzb, void* stream_) {
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    if (int rc = check_spmm_args(vals, rowptr, colidx, B, C, M, N, K, nnzb)) return rc;
    if (nnzb > kMaxBlocks)
        return fail(SMAT_ERR_RANGE,
                    "smat_spmm_bcsr_f16_static holds at most %zu nonzero blocks in its fixed scratch (got %zu); "
                    "use smat_plan_create for larger matrices",
                    kMaxBlocks, nnzb);
    if (M > kMaxRows)
        return fail(SMAT_ERR_RANGE, "smat_spmm_bcsr_f16_static handles at most %zu rows (got %zu)", kMaxRows, M);
    if (M == 0 || N == 0) return SMAT_OK;
    StaticDev* d = nullptr;
    if (int rc = static_device(&d)) return rc;

    const size_t Mb = M / 16;
    PlanView v;
    v.rowptr = rowptr;
    v.K = K;
    v.nnzb = nnzb;
    v.brow_begin = 0;
    v.brow_end = Mb;
    const size_t rg = choose_rows_per_group(Mb, N, d->ctx.sm_count, false, nnzb, K);
    v.rg = rg;
    v.n_groups = (Mb + rg - 1) / rg;
    int* gsp = reinterpret_cast<int*>(d->base);
    void* steps = d->base + kGspBytes;
    int* blk = reinterpret_cast<int*>(d->base + kGspBytes + kStepsBytes);
    void* packed = d->base + kGspBytes + kStepsBytes + kBlkBytes;
    v.gsp = gsp;
    v.steps = steps;
    v.blk = blk;
    v.packed = packed;
    if (int rc = plan_count_async(rowptr, colidx, K, nnzb, 0, Mb, rg, gsp, stream, &d->ctx)) return rc;
    if (int rc = plan_fill_async(rowptr, colidx, K, nnzb, 0, Mb, rg, gsp, steps, blk, stream, &d->ctx)) return rc;
    if (int rc = pack_values_async(rowptr, vals, gsp, steps, blk, packed, 0, Mb, rg, nnzb, stream, &d->ctx)) return rc;
    return launch_spmm(v, B, C, N, stream, &d->ctx);
}
