"""TEST INFRASTRUCTURE ONLY: ctypes doorway onto the CPU oracle (oracle/libsmat_oracle.so) and, when it
was built, onto the unmodified reference CPU code (oracle/_ref/libsmat_ref.so).

Only tests, the smoke check and the benchmark's CPU-baseline leg import this package; the product
package never does.  Build with ``make -C oracle`` (and ``make -C oracle ref`` where the reference
tree is present).
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None

i64p = np.ctypeslib.ndpointer(dtype=np.int64, flags="C_CONTIGUOUS")
i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
u16p = np.ctypeslib.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")
f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")


def build(ref_root=None):
    """Compile the oracle; also the reference-backed libraries/programs when a reference tree is named (argument, or
    the SMAT_REFERENCE environment variable) and exists."""
    subprocess.check_call(["make", "-s", "-C", _HERE, "all"])
    ref_root = ref_root or os.environ.get("SMAT_REFERENCE")
    if not ref_root:
        return
    if os.path.isdir(os.path.join(ref_root, "preprocess", "src", "general")):
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref", f"REF={ref_root}"])
    if os.path.isdir(os.path.join(ref_root, "src", "cuda_hgemm", "src", "mma")):
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref_gpu", f"REF={ref_root}"])


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libsmat_oracle.so")
        if not os.path.exists(path):
            build()
        L = C.CDLL(path)
        L.orc_double_to_half_bits.restype = C.c_uint16
        L.orc_double_to_half_bits.argtypes = [C.c_double]
        L.orc_read_mtx.argtypes = [C.c_char_p, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int64),
                                   C.POINTER(C.c_int), C.POINTER(C.POINTER(C.c_int)), C.POINTER(C.POINTER(C.c_int)),
                                   C.POINTER(C.POINTER(C.c_uint16))]
        L.orc_free.argtypes = [C.c_void_p]
        L.orc_csr_to_bcsr.argtypes = [C.c_int64, C.c_int64, i32p, i32p, u16p, C.POINTER(C.c_int64), i32p,
                                      C.c_void_p, C.c_void_p]
        L.orc_bcsr_spmm_f32.argtypes = [u16p, i32p, i32p, u16p, f32p, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                        C.c_int64, C.c_int]
        L.orc_jaccard_group.restype = C.c_float
        L.orc_jaccard_group.argtypes = [i64p, C.c_int64, C.c_int64, i64p, C.c_int64, C.c_int64, C.c_int64]
        L.orc_hamming_group.restype = C.c_float
        L.orc_hamming_group.argtypes = [i64p, C.c_int64, C.c_int64, i64p, C.c_int64, C.c_int64, C.c_int64]
        L.orc_keeper_grouping.argtypes = [C.c_int64, i64p, i64p, C.c_float, C.c_int64, C.c_int64, C.c_int, i64p]
        L.orc_get_permutation.argtypes = [C.c_int64, i64p, i64p]
        L.orc_fixed_size_grouping.argtypes = [C.c_int64, i64p, C.c_int64, i64p]
        L.orc_reorder_rows.argtypes = [C.c_int64, i64p, i64p, C.c_float, C.c_int64, C.c_int64, i64p, i64p]
        _LIB = L
    return _LIB


def ref_dir():
    return os.path.join(_HERE, "_ref")


def have_ref():
    return os.path.exists(os.path.join(ref_dir(), "libsmat_ref.so"))


def ref():
    """The unmodified reference CPU code (None if oracle/_ref was not built)."""
    global _REF
    if _REF is None and have_ref():
        L = C.CDLL(os.path.join(ref_dir(), "libsmat_ref.so"))
        L.ref_jaccard_group.restype = C.c_float
        L.ref_jaccard_group.argtypes = [i64p, C.c_long, C.c_long, i64p, C.c_long, C.c_long, C.c_long]
        L.ref_hamming_group.restype = C.c_float
        L.ref_hamming_group.argtypes = [i64p, C.c_long, C.c_long, i64p, C.c_long, C.c_long, C.c_long]
        L.ref_group_and_permute.restype = C.c_long
        L.ref_group_and_permute.argtypes = [C.c_char_p, C.c_float, C.c_long, C.c_long, C.c_int, C.c_long, i64p, i64p]
        L.ref_get_permutation.restype = C.c_long
        L.ref_get_permutation.argtypes = [C.c_long, i64p, i64p]
        L.ref_fixed_size_grouping.restype = C.c_long
        L.ref_fixed_size_grouping.argtypes = [C.c_long, i64p, C.c_long, i64p]
        L.ref_vbr_multiply.argtypes = [C.c_long, C.c_long, C.c_long, C.c_long, i64p, i64p, f32p, C.c_long, C.c_long,
                                       f32p, C.c_int, f32p]
        if hasattr(L, "ref_vbr_from_csr"):
            L.ref_vbr_from_csr.restype = C.c_long
            L.ref_vbr_from_csr.argtypes = [C.c_long, C.c_long, i32p, i32p, f32p, C.c_long, C.c_long, C.c_long, i64p, i64p, f32p]
        if hasattr(L, "ref_vbr_from_grouping"):
            L.ref_vbr_from_grouping.restype = C.c_long
            L.ref_vbr_from_grouping.argtypes = [C.c_long, C.c_long, i32p, i32p, f32p, i64p, C.c_long, C.c_long, C.c_long, C.c_long,
                                                i64p, i64p, i64p, i64p, i64p, f32p]
        _REF = L
    return _REF


_REF_GPU = None


def ref_gpu():
    """GPU baselines (the reference's kernels compiled unmodified for sm_100a, cuSPARSE CSR SpMM);
    None if oracle/_ref/libsmat_ref_gpu.so was not built."""
    global _REF_GPU
    path = os.path.join(ref_dir(), "libsmat_ref_gpu.so")
    if _REF_GPU is None and os.path.exists(path):
        L = C.CDLL(path)
        vp, sz = C.c_void_p, C.c_size_t
        L.ref_gpu_launch.restype = C.c_float
        L.ref_gpu_launch.argtypes = [C.c_int, vp, vp, vp, vp, vp, sz, sz, sz, sz, vp, vp, C.c_int, C.c_int]
        L.cusparse_csr_spmm_f16.restype = C.c_float
        L.cusparse_csr_spmm_f16.argtypes = [vp, vp, vp, sz, vp, vp, sz, sz, sz, C.c_int, C.c_int]
        if hasattr(L, "ref_sparse_matrix_load"):
            psz, pip, pup = C.POINTER(sz), C.POINTER(C.POINTER(C.c_int)), C.POINTER(C.POINTER(C.c_uint16))
            L.ref_sparse_matrix_load.argtypes = [C.c_char_p, C.c_int, C.c_int, psz, psz, psz, psz, pip, pip, pup, pip, pip, pup]
            L.ref_free.argtypes = [vp]
        _REF_GPU = L
    return _REF_GPU


# ----------------------------------------------------------------------------------------------
# numpy-level helpers
# ----------------------------------------------------------------------------------------------
def read_mtx(path):
    """mmio_allinone restatement -> (M, K, rowptr int32, colidx int32, vals float16, is_symmetric)."""
    L = lib()
    M, N, nnz, sym = C.c_int64(), C.c_int64(), C.c_int64(), C.c_int()
    rp, ci, vv = C.POINTER(C.c_int)(), C.POINTER(C.c_int)(), C.POINTER(C.c_uint16)()
    rc = L.orc_read_mtx(path.encode(), C.byref(M), C.byref(N), C.byref(nnz), C.byref(sym), C.byref(rp), C.byref(ci),
                        C.byref(vv))
    if rc != 0:
        raise IOError(f"orc_read_mtx({path}) -> {rc}")
    rowptr = np.ctypeslib.as_array(rp, shape=(M.value + 1,)).copy()
    colidx = np.ctypeslib.as_array(ci, shape=(max(nnz.value, 1),))[: nnz.value].copy()
    vals = np.ctypeslib.as_array(vv, shape=(max(nnz.value, 1),))[: nnz.value].copy().view(np.float16)
    for p in (rp, ci, vv):
        L.orc_free(C.cast(p, C.c_void_p))
    return M.value, N.value, rowptr, colidx, vals, bool(sym.value)


def csr_to_bcsr(M, K, rowptr, colidx, vals):
    """csrToBcsr restatement -> (bcsr_rowptr int32[M/16+1], bcsr_colidx int32[nnzb], bcsr_vals float16[nnzb*256])."""
    L = lib()
    rowptr = np.ascontiguousarray(rowptr, dtype=np.int32)
    colidx = np.ascontiguousarray(colidx, dtype=np.int32)
    v16 = np.ascontiguousarray(vals, dtype=np.float16).view(np.uint16)
    if colidx.size == 0:
        colidx = np.zeros(1, np.int32)
        v16 = np.zeros(1, np.uint16)
    nnzb = C.c_int64()
    brp = np.zeros(M // 16 + 1, np.int32)
    L.orc_csr_to_bcsr(M, K, rowptr, colidx, v16, C.byref(nnzb), brp, None, None)
    bci = np.zeros(max(nnzb.value, 1), np.int32)
    bv = np.zeros(max(nnzb.value, 1) * 256, np.uint16)
    L.orc_csr_to_bcsr(M, K, rowptr, colidx, v16, C.byref(nnzb), brp, bci.ctypes.data, bv.ctypes.data)
    return brp, bci[: nnzb.value], bv[: nnzb.value * 256].view(np.float16)


def bcsr_spmm(bvals, browptr, bcolidx, B_nk, M, N, K, brow_begin=0, brow_end=None, threads=1):
    """fp32 blocked multiply (VBR::multiply arithmetic). B_nk is the [N][K] fp16 array. Returns fp32 C rows."""
    L = lib()
    if brow_end is None:
        brow_end = M // 16
    out = np.zeros(((brow_end - brow_begin) * 16, N), np.float32)
    bv = np.ascontiguousarray(bvals, dtype=np.float16).view(np.uint16)
    if bv.size == 0:
        bv = np.zeros(1, np.uint16)
    bc = np.ascontiguousarray(bcolidx, dtype=np.int32)
    if bc.size == 0:
        bc = np.zeros(1, np.int32)
    Bu = np.ascontiguousarray(B_nk, dtype=np.float16).view(np.uint16).reshape(-1)
    L.orc_bcsr_spmm_f32(bv, np.ascontiguousarray(browptr, dtype=np.int32), bc, Bu, out.reshape(-1), M, N, K,
                        brow_begin, brow_end, threads)
    return out


def _i64(a):
    a = np.ascontiguousarray(a, dtype=np.int64)
    return a if a.size else np.zeros(1, np.int64)


def jaccard_group(rowA, gA, rowB, gB, bs):
    return float(lib().orc_jaccard_group(_i64(rowA), len(rowA), gA, _i64(rowB), len(rowB), gB, bs))


def hamming_group(rowA, gA, rowB, gB, bs):
    return float(lib().orc_hamming_group(_i64(rowA), len(rowA), gA, _i64(rowB), len(rowB), gB, bs))


def keeper_grouping(rowptr, cols, tau=0.5, col_block=16, row_block=16):
    rows = len(rowptr) - 1
    g = np.zeros(max(rows, 1), np.int64)
    lib().orc_keeper_grouping(rows, _i64(rowptr), _i64(cols), tau, col_block, row_block, 1, g)
    return g[:rows]


def reorder_rows(rowptr, cols, tau=0.5, col_block=16, row_block=16):
    """-> (fixed-size grouping, permutation) as Matrix_Blocking -a 5 -F 1 produces them."""
    rows = len(rowptr) - 1
    g = np.zeros(max(rows, 1), np.int64)
    p = np.zeros(max(rows, 1), np.int64)
    lib().orc_reorder_rows(rows, _i64(rowptr), _i64(cols), tau, col_block, row_block, g, p)
    return g[:rows], p[:rows]


def ref_vbr_from_grouping(M, K, rowptr, colidx, vals, grouping, col_block):
    """Variable-height blocking by the UNMODIFIED reference code VBR::fill_from_CSR_inplace(cmat, grouping, col_block)
    (oracle/_ref): dict of row_part, nzcount, jab (int64), mab (float32, column-major blocks) and row_perm (the
    reference's get_permutation of the grouping).  Costs O(nnz * K / col_block) in the reference: small matrices only."""
    R = ref()
    if R is None or not hasattr(R, "ref_vbr_from_grouping"):
        raise RuntimeError("oracle/_ref/libsmat_ref.so with ref_vbr_from_grouping is not built")
    rowptr = np.ascontiguousarray(rowptr, dtype=np.int32)
    colidx = np.ascontiguousarray(colidx, dtype=np.int32)
    vals32 = np.ascontiguousarray(np.asarray(vals, dtype=np.float16).astype(np.float32))
    if colidx.size == 0:
        colidx, vals32 = np.zeros(1, np.int32), np.zeros(1, np.float32)
    g = np.ascontiguousarray(grouping, dtype=np.int64)
    Kb = (K - 1) // col_block + 1
    max_blocks = int(min(len(colidx), M * Kb)) + 1
    max_vals = max_blocks * M * col_block if M * col_block * max_blocks < (1 << 26) else (1 << 26)
    br, nv = np.zeros(1, np.int64), np.zeros(1, np.int64)
    part, nzc = np.zeros(M + 1, np.int64), np.zeros(M, np.int64)
    jab, mab = np.zeros(max_blocks, np.int64), np.zeros(max_vals, np.float32)
    nb = R.ref_vbr_from_grouping(M, K, rowptr, colidx, vals32, g, col_block, M, max_blocks, max_vals, br, part, nzc, jab, nv, mab)
    if nb < 0:
        raise RuntimeError("ref_vbr_from_grouping: bound too small")
    perm = np.zeros(M, np.int64)
    R.ref_get_permutation(M, g, perm)
    n_br = int(br[0])
    return {"col_block": col_block, "row_part": part[: n_br + 1].copy(), "row_perm": perm, "nzcount": nzc[:n_br].copy(),
            "jab": jab[:nb].copy(), "mab": mab[: int(nv[0])].copy()}


def ref_bcsr_via_vbr(M, K, rowptr, colidx, vals):
    """16x16 blocking of a CSR matrix by the UNMODIFIED reference code VBR::fill_from_CSR_inplace (oracle/_ref), restated
    in the BCSR layout of the GPU path: (bcsr_rowptr int32, bcsr_colidx int32 = element columns, bcsr_vals float16
    row-major blocks).  The reference stores a block column-major with its rows in the order of its own (unstable)
    argsort of the grouping i // 16; that order is obtained from the reference's get_permutation and undone here.
    Costs O(nnz * K / 16) in the reference (a std::count per entry): small matrices only."""
    R = ref()
    if R is None or not hasattr(R, "ref_vbr_from_csr"):
        raise RuntimeError("oracle/_ref/libsmat_ref.so with ref_vbr_from_csr is not built")
    rowptr = np.ascontiguousarray(rowptr, dtype=np.int32)
    colidx = np.ascontiguousarray(colidx, dtype=np.int32)
    vals32 = np.ascontiguousarray(np.asarray(vals, dtype=np.float16).astype(np.float32))
    if colidx.size == 0:
        colidx, vals32 = np.zeros(1, np.int32), np.zeros(1, np.float32)
    Mb = M // 16
    max_blocks = int(min(len(colidx), Mb * (K // 16))) + 1
    nzc = np.zeros(max(Mb, 1), np.int64)
    jab = np.zeros(max_blocks, np.int64)
    mab = np.zeros(max_blocks * 256, np.float32)
    nb = R.ref_vbr_from_csr(M, K, rowptr, colidx, vals32, 16, 16, max_blocks, nzc, jab, mab)
    if nb < 0:
        raise RuntimeError("ref_vbr_from_csr: block bound too small")
    perm = np.zeros(M, np.int64)
    R.ref_get_permutation(M, np.ascontiguousarray(np.arange(M, dtype=np.int64) // 16), perm)
    brp = np.zeros(Mb + 1, np.int32)
    brp[1:] = np.cumsum(nzc[:Mb])
    bci = (jab[:nb] * 16).astype(np.int32)
    blocks = mab[: nb * 256].reshape(nb, 16, 16)  # [block][column][position of the row in the reference's order]
    out = np.zeros((nb, 16, 16), np.float32)       # [block][row][column]
    brow_of_block = np.repeat(np.arange(Mb), nzc[:Mb])
    for pos in range(16):
        rows_here = perm[brow_of_block * 16 + pos] - brow_of_block * 16  # the original row (within the block) at this position
        out[np.arange(nb), rows_here, :] = blocks[:, :, pos]
    return brp, bci, out.reshape(-1).astype(np.float16)


def ref_sparse_matrix(path, host_only=True, export_magicube=False, knapsack=False):
    """Runs the reference's own reader and blocked-format builder, unmodified: mmio_allinone
    (src/cuda_hgemm/src/common/mmio_highlevel.h:619-786) + SparseMatrix::csrToBcsr (matrix.h:376-502).  host_only: just
    those two host steps (no GPU needed); else the class's full constructor, which also uploads (needs a GPU).
    knapsack (host_only): csrToBcsrKnapsacking (matrix.h:504-671) in place of csrToBcsr -- blocks start at any column.
    Returns (M, K, csr_rowptr, csr_colidx, csr_vals f16, bcsr_rowptr, bcsr_colidx, bcsr_vals f16)."""
    G = ref_gpu()
    if G is None or not hasattr(G, "ref_sparse_matrix_load"):
        raise RuntimeError("oracle/_ref/libsmat_ref_gpu.so with ref_sparse_matrix_load is not built")
    sz = C.c_size_t
    M, K, nnz, nnzb = sz(), sz(), sz(), sz()
    ip, up = C.POINTER(C.c_int), C.POINTER(C.c_uint16)
    crp, cci, cv, brp, bci, bv = ip(), ip(), up(), ip(), ip(), up()
    rc = G.ref_sparse_matrix_load(path.encode(), (2 if knapsack else 1) if host_only else 0, 1 if export_magicube else 0, C.byref(M), C.byref(K), C.byref(nnz), C.byref(nnzb),
                                  C.byref(crp), C.byref(cci), C.byref(cv), C.byref(brp), C.byref(bci), C.byref(bv))
    if rc != 0:
        raise RuntimeError(f"ref_sparse_matrix_load -> {rc}")

    def take(ptr, n, dtype):
        a = np.ctypeslib.as_array(ptr, shape=(max(n, 1),))[:n].copy()
        G.ref_free(C.cast(ptr, C.c_void_p))
        return a.view(dtype) if dtype is not None else a
    out = (M.value, K.value, take(crp, M.value + 1, None), take(cci, nnz.value, None), take(cv, nnz.value, np.float16),
           take(brp, M.value // 16 + 1, None), take(bci, nnzb.value, None), take(bv, nnzb.value * 256, np.float16))
    return out


def csr_to_bcsr_knapsack(M, K, rowptr, colidx, vals):
    """Restatement of SparseMatrix::csrToBcsrKnapsacking (src/cuda_hgemm/src/common/matrix.h:504-671), the reference's
    gap-skipping blocking: inside a block-row the stored columns are walked in ascending order and a new 16-wide block
    is opened at the first column the current one does not cover (:583-606), so blocks start at ANY column; the start
    of a block is moved left when the columns still to come would otherwise leave a ragged last block (:551-570,
    :586-600).  Returns (rowptr int32[M/16+1], colidx int32 = start column of every block, vals float16[nnzb*256]).
    Plain Python loops: for fixtures and small cases."""
    rowptr = np.asarray(rowptr, dtype=np.int64)
    colidx = np.asarray(colidx, dtype=np.int64)
    v16 = np.asarray(vals, dtype=np.float16)
    brp = np.zeros(M // 16 + 1, np.int32)
    starts, blocks = [], []
    nb = 0
    for br in range(M // 16):
        brp[br] = nb
        lo, hi = rowptr[br * 16], rowptr[br * 16 + 16]
        if hi == lo:
            continue
        cols = colidx[lo:hi]
        rows = np.repeat(np.arange(br * 16, br * 16 + 16), np.diff(rowptr[br * 16:br * 16 + 17]))
        order = np.argsort(cols, kind="stable")
        cols, rows, vv = cols[order], rows[order], v16[lo:hi][order]
        first, last = int(cols[0]), int(cols[-1])
        add_right = K - last - 1

        def place(col, add_left):
            span = last - col + 1
            to_add = 16 - span % 16
            if span % 16 == 0 or add_right >= to_add:
                return col
            if add_left >= to_add:
                return col - to_add
            return col - add_left
        start = place(first, first)
        starts.append(start)
        blocks.append(np.zeros((16, 16), np.float16))
        end = start + 16
        for c, r, x in zip(cols.tolist(), rows.tolist(), vv):
            if c >= end:
                start = place(c, c - end)
                starts.append(start)
                blocks.append(np.zeros((16, 16), np.float16))
                end = start + 16
                nb += 1
            blocks[nb][r % 16, c - start] = x
        nb += 1
    brp[M // 16] = nb
    bv = np.stack(blocks).reshape(-1) if blocks else np.zeros(0, np.float16)
    return brp, np.asarray(starts, np.int32), bv
