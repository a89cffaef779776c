// Internal declarations shared by the translation units of libsmat_b200.so.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/smat_b200.h"

namespace smat {

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
};
int get_device_ctx(DeviceCtx** out);

void count_launch();

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup (no link against libcuda).
int encode_tensor_map_2d_f16(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_pitch_bytes,
                             uint32_t box_inner, uint32_t box_outer, int swizzle32, int l2_promo_bytes);

// Launch of the SpMM kernels (spmm_sm100.cu).
int launch_spmm(const void* vals, const int* rowptr, const int* colidx, const void* B, void* C, size_t M, size_t N,
                size_t K, size_t nnzb, size_t brow_begin, size_t brow_end, cudaStream_t stream);

extern int g_spmm_variant;

}  // namespace smat
