"""smat_b200: B200-native block-sparse SpMM engine behind SMaT's kernel-launcher boundary.

The product is the C-ABI shared library ``libsmat_b200.so`` (declared in ``include/smat_b200.h``,
sources in ``smat_b200/csrc``).  This Python package is the host-side mirror of the reference's
harness objects (``SparseMatrix``, ``Matrix``, ``Tester``; src/cuda_hgemm/src/common/matrix.h,
tester.h) on top of that library, using torch only for device memory and streams.

There is no CPU fallback: every compute entry point goes through the CUDA library and raises if it is
missing or if no sm_100 device is present.
"""
from .api import (  # noqa: F401
    Matrix,
    Plan,
    SmatError,
    SparseMatrix,
    Tester,
    all_gather_rows,
    apply_col_permutation,
    apply_row_permutation,
    b_slice_of_rank,
    gather_b_slices,
    bcsr_knapsack,
    jaccard_group,
    knapsack_to_csr,
    cluster_rows,
    vbr_from_csr,
    vbr_to_csr,
    launch_count,
    lib,
    partition_block_rows,
    permute_rows_of_B,
    read_mtx,
    reorder_cols,
    reorder_rows,
    set_variant,
    spmm,
    spmm_rows,
)
