// TEST / BENCHMARK INFRASTRUCTURE ONLY -- doorway onto GPU baselines that are timed beside the product:
//   * the reference's own sm_80-style kernels, UNMODIFIED, compiled from the reference tree for sm_100a
//     (mmaCBTKernel, src/cuda_hgemm/src/mma/mmaCBT.cu:83-88; mmaBTKernel, src/cuda_hgemm/src/mma/mmaBT.cu),
//   * cuSPARSE CSR SpMM configured as the reference's baseline does it
//     (preprocess/src/cuda/cuda_utilities.cpp:1326-1393: CSR, fp16 in, fp32 compute, ALG_DEFAULT).
// No algorithm of its own.  Built by oracle/Makefile (target ref_gpu) into oracle/_ref/; never linked
// into the product.  Note: mmaCBT copies a contiguous 256-byte slab of B per tile, which is the intended
// 8 x 16 tile only when K == 16 (mmaCBT.cu:46-53), so its numbers are timing-only.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cusparse.h>
#include <stddef.h>

void mmaCBTKernel(half*, int*, int*, half*, half*, size_t, size_t, size_t, size_t, int*, int*);
void mmaBTKernel(half*, int*, int*, half*, half*, size_t, size_t, size_t, size_t, int*, int*);

extern "C" {

// Launches the reference kernel `iters` times on the default stream and returns the mean milliseconds
// per launch (CUDA events), or a negative CUDA error code.
float ref_gpu_launch(int which, void* vals, int* rowptr, int* colidx, void* B, void* C, size_t M, size_t N, size_t K,
                     size_t nnzb, int* blockInfo, int* relMap, int warmup, int iters) {
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    auto run = [&]() {
        if (which == 0) mmaCBTKernel((half*)vals, rowptr, colidx, (half*)B, (half*)C, M, N, K, nnzb, blockInfo, relMap);
        else mmaBTKernel((half*)vals, rowptr, colidx, (half*)B, (half*)C, M, N, K, nnzb, blockInfo, relMap);
    };
    for (int i = 0; i < warmup; i++) run();
    cudaEventRecord(e0);
    for (int i = 0; i < iters; i++) run();
    cudaEventRecord(e1);
    cudaError_t e = cudaEventSynchronize(e1);
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (e != cudaSuccess || cudaGetLastError() != cudaSuccess) return -(float)(int)e - 1.0f;
    return ms / iters;
}

// C[M x N] (row-major fp16) = A_csr[M x K] (fp16) * B, with B given as the [N][K] array of the kernel
// boundary, i.e. the column-major K x N matrix.  Returns mean ms per call or a negative status.
float cusparse_csr_spmm_f16(int* rowptr, int* colidx, void* vals, size_t nnz, void* B_nk, void* C, size_t M, size_t N,
                            size_t K, int warmup, int iters) {
    cusparseHandle_t h;
    if (cusparseCreate(&h) != CUSPARSE_STATUS_SUCCESS) return -1;
    cusparseSpMatDescr_t A;
    cusparseDnMatDescr_t Bd, Cd;
    cusparseCreateCsr(&A, M, K, nnz, rowptr, colidx, vals, CUSPARSE_INDEX_32I, CUSPARSE_INDEX_32I, CUSPARSE_INDEX_BASE_ZERO,
                      CUDA_R_16F);
    cusparseCreateDnMat(&Bd, K, N, K, B_nk, CUDA_R_16F, CUSPARSE_ORDER_COL);
    cusparseCreateDnMat(&Cd, M, N, N, C, CUDA_R_16F, CUSPARSE_ORDER_ROW);
    float alpha = 1.0f, beta = 0.0f;
    size_t ws = 0;
    cusparseStatus_t st = cusparseSpMM_bufferSize(h, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha, A,
                                                  Bd, &beta, Cd, CUDA_R_32F, CUSPARSE_SPMM_ALG_DEFAULT, &ws);
    if (st != CUSPARSE_STATUS_SUCCESS) return -2 - (float)st;
    void* buf = nullptr;
    cudaMalloc(&buf, ws ? ws : 16);
    auto run = [&]() {
        return cusparseSpMM(h, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha, A, Bd, &beta, Cd,
                            CUDA_R_32F, CUSPARSE_SPMM_ALG_DEFAULT, buf);
    };
    for (int i = 0; i < warmup; i++) st = run();
    if (st != CUSPARSE_STATUS_SUCCESS) { cudaFree(buf); return -100 - (float)st; }
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaEventRecord(e0);
    for (int i = 0; i < iters; i++) run();
    cudaEventRecord(e1);
    cudaEventSynchronize(e1);
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(buf);
    cusparseDestroySpMat(A);
    cusparseDestroyDnMat(Bd);
    cusparseDestroyDnMat(Cd);
    cusparseDestroy(h);
    return ms / iters;
}

}  // extern "C"

// ---- the reference's own reader + blocked-format builder, run unmodified -------------------------------------------
// SparseMatrix(name, file) (src/cuda_hgemm/src/common/matrix.h:145-202) reads the .mtx file with mmio_allinone
// (mmio_highlevel.h:619-786), converts CSR -> BCSR with csrToBcsr (matrix.h:376-502) and uploads both.  Its arrays are
// private and have no host getters, so the class is compiled here with its access specifiers opened; nothing else changes.
#define private public
#include "matrix.h"
#undef private

#include <stdlib.h>
#include <string.h>

extern "C" {

// Builds a SparseMatrix from `mtx_path` and hands back malloc'ed copies of its host arrays (free them with
// ref_free).  host_only == 0: through the class's constructor, which also uploads everything (needs a GPU).
// host_only != 0: the two host steps the constructor performs, readCsr() and csrToBcsr(), on a zero-filled object
// whose constructor is not run -- neither step touches CUDA, so this works on a machine without a GPU.
// With export_magicube != 0 it also calls SparseMatrix::outputCsr (matrix.h:321-348), which writes
// ./data/magicube_cop20k_A.mtx relative to the current directory.  The object is leaked on purpose: its destructor frees
// only part of what the constructor allocates and the process is short-lived.
int ref_sparse_matrix_load(const char* mtx_path, int host_only, int export_magicube, size_t* M, size_t* K, size_t* nnz,
                           size_t* nnzb, int** csr_rowptr, int** csr_colidx, unsigned short** csr_vals, int** bcsr_rowptr,
                           int** bcsr_colidx, unsigned short** bcsr_vals) {
    SparseMatrix* sm;
    if (host_only) {
        sm = static_cast<SparseMatrix*>(calloc(1, sizeof(SparseMatrix)));
        sm->filename = const_cast<char*>(mtx_path);
        sm->readCsr();
        // host_only == 2: the alternative, gap-skipping blocking the reference keeps beside csrToBcsr
        // (csrToBcsrKnapsacking, matrix.h:504-671; its call in the constructor is commented out, matrix.h:174)
        if (host_only == 2) sm->csrToBcsrKnapsacking();
        else sm->csrToBcsr();
    } else {
        sm = new SparseMatrix("A", const_cast<char*>(mtx_path));
    }
    if (export_magicube) sm->outputCsr();
    *M = sm->m_row;
    *K = sm->m_col;
    *nnz = sm->nnz;
    *nnzb = sm->nonzeroBlocks;
    auto dup = [](const void* src, size_t bytes) {
        void* p = malloc(bytes ? bytes : 1);
        memcpy(p, src, bytes);
        return p;
    };
    *csr_rowptr = (int*)dup(sm->csrRowPtr_host, (sm->m_row + 1) * sizeof(int));
    *csr_colidx = (int*)dup(sm->csrColIdx_host, sm->nnz * sizeof(int));
    *csr_vals = (unsigned short*)dup(sm->csrVal_host, sm->nnz * sizeof(half));
    *bcsr_rowptr = (int*)dup(sm->bcsrRowPtr_host, (sm->m_row / 16 + 1) * sizeof(int));
    *bcsr_colidx = (int*)dup(sm->bcsrColIdx_host, sm->nonzeroBlocks * sizeof(int));
    *bcsr_vals = (unsigned short*)dup(sm->bcsrVal_host, sm->nonzeroBlocks * 256 * sizeof(half));
    return 0;
}

void ref_free(void* p) { free(p); }

}  // extern "C"
