"""Host-side mirror of the reference's harness objects on top of the C-ABI library.

Names and argument meaning follow the reference (src/cuda_hgemm/src/common/matrix.h,
src/cuda_hgemm/src/common/tester.h, src/reorder.py); compute always goes through
``libsmat_b200.so``.  torch provides device memory and streams only.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


class SmatError(RuntimeError):
    def __init__(self, code, text):
        super().__init__(f"smat_b200 error {code}: {text}")
        self.code = code


def lib():
    """Loads libsmat_b200.so (built in-tree by ``smat_b200._build``).  Raises if it is missing."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = os.environ.get("SMAT_LIB", os.path.join(_HERE, "libsmat_b200.so"))
    if not os.path.exists(path):
        raise SmatError(-2, f"{path} is missing: build it with `python -m smat_b200._build` "
                            "(there is no CPU fallback)")
    L = C.CDLL(path)
    vp, sz, ip = C.c_void_p, C.c_size_t, C.c_void_p
    L.smat_spmm_bcsr_f16.argtypes = [vp, ip, ip, vp, vp, sz, sz, sz, sz, ip, ip, vp]
    L.smat_spmm_bcsr_f16_rows.argtypes = [vp, ip, ip, vp, vp, sz, sz, sz, sz, sz, sz, vp]
    L.smat_spmm_bcsr_f16_static.argtypes = [vp, ip, ip, vp, vp, sz, sz, sz, sz, vp]
    L.smat_plan_create.argtypes = [C.POINTER(vp), vp, ip, ip, sz, sz, sz, sz, sz, sz, vp]
    L.smat_plan_set_values.argtypes = [vp, vp, vp]
    L.smat_plan_spmm.argtypes = [vp, vp, vp, sz, vp]
    L.smat_plan_spmm_host.argtypes = [vp, vp, vp, sz, vp]
    L.smat_plan_destroy.argtypes = [vp]
    L.smat_plan_info.argtypes = [vp, vp, vp, vp]
    L.smat_spmm_set_variant.argtypes = [C.c_int]
    L.smat_device_status.argtypes = [vp]
    L.smat_selftest_wait_timeout.argtypes = [vp]
    L.smat_launch_count.restype = C.c_longlong
    L.smat_bcsr_count.argtypes = [ip, ip, sz, sz, sz, ip, C.POINTER(sz), vp]
    L.smat_bcsr_fill.argtypes = [ip, ip, vp, sz, sz, sz, ip, ip, vp, sz, vp]
    L.smat_read_mtx.argtypes = [C.c_char_p, C.POINTER(sz), C.POINTER(sz), C.POINTER(sz), C.POINTER(C.c_int),
                                C.POINTER(C.POINTER(C.c_int)), C.POINTER(C.POINTER(C.c_int)),
                                C.POINTER(C.POINTER(C.c_uint16))]
    L.smat_free_host.argtypes = [vp]
    L.smat_free_host.restype = None
    L.smat_reorder_rows.argtypes = [sz, vp, vp, C.c_float, C.c_int, C.c_int, C.c_int, vp, vp]
    L.smat_jaccard_group.argtypes = [vp, sz, C.c_int64, vp, sz, C.c_int64, C.c_int64]
    L.smat_jaccard_group.restype = C.c_float
    L.smat_partition_block_rows.argtypes = [vp, sz, C.c_int, vp]
    L.smat_last_error_string.restype = C.c_char_p
    _LIB = L
    return L


def _check(rc):
    if rc != 0:
        raise SmatError(rc, lib().smat_last_error_string().decode())


def launch_count():
    return int(lib().smat_launch_count())


def set_variant(v):
    """0 = automatic, 1 = shared-memory-operand kernel, 2 = tensor-memory-operand kernel."""
    _check(lib().smat_spmm_set_variant(int(v)))


def _stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


# ------------------------------------------------------------------------------------------------
# host-side steps
# ------------------------------------------------------------------------------------------------
def read_mtx(path):
    """Matrix-Market file -> (M, K, rowptr int32, colidx int32, vals float16, is_symmetric);
    the behaviour of mmio_allinone (src/cuda_hgemm/src/common/mmio_highlevel.h:619-786)."""
    L = lib()
    M, K, nnz, sym = C.c_size_t(), C.c_size_t(), C.c_size_t(), C.c_int()
    rp, ci, vv = C.POINTER(C.c_int)(), C.POINTER(C.c_int)(), C.POINTER(C.c_uint16)()
    _check(L.smat_read_mtx(os.fsencode(path), C.byref(M), C.byref(K), C.byref(nnz), C.byref(sym), C.byref(rp),
                           C.byref(ci), C.byref(vv)))
    try:
        rowptr = np.ctypeslib.as_array(rp, shape=(M.value + 1,)).copy()
        colidx = np.ctypeslib.as_array(ci, shape=(nnz.value + 1,))[: nnz.value].copy()
        vals = np.ctypeslib.as_array(vv, shape=(nnz.value + 1,))[: nnz.value].copy().view(np.float16)
    finally:
        for p in (rp, ci, vv):
            L.smat_free_host(C.cast(p, C.c_void_p))
    return M.value, K.value, rowptr, colidx, vals, bool(sym.value)


def jaccard_group(rowA, gA, rowB, gB, block_size):
    a = np.ascontiguousarray(rowA, dtype=np.int64)
    b = np.ascontiguousarray(rowB, dtype=np.int64)
    return float(lib().smat_jaccard_group(a.ctypes.data, a.size, gA, b.ctypes.data, b.size, gB, block_size))


def reorder_rows(rowptr, colidx, tau=0.5, col_block=16, row_block=16, threads=0):
    """Similarity row reordering as `Matrix_Blocking -a 5 -b col_block -B row_block -F 1 -t tau`
    (src/reorder.py:107-139).  Columns must be ascending inside each row.
    Returns (grouping int64[rows], perm int64[rows]) with new row r = old row perm[r]."""
    rp = np.ascontiguousarray(rowptr, dtype=np.int64)
    ci = np.ascontiguousarray(colidx, dtype=np.int32)
    rows = rp.size - 1
    grouping = np.zeros(max(rows, 1), np.int64)
    perm = np.zeros(max(rows, 1), np.int64)
    _check(lib().smat_reorder_rows(rows, rp.ctypes.data, ci.ctypes.data if ci.size else None, tau, col_block,
                                   row_block, threads, grouping.ctypes.data, perm.ctypes.data))
    return grouping[:rows], perm[:rows]


def cluster_rows(rowptr, colidx, tau=0.5, col_block=16, max_group_rows=16, threads=0):
    """The clustering of ``reorder_rows`` without the fixed-size regrouping (`Matrix_Blocking` without -F 1): the
    grouping as BlockingEngine::GetGrouping returns it (groups of unequal size, full groups numbered below zero) and
    get_permutation of it.  Feed it to ``vbr_from_csr`` for the reference's variable-height blocking."""
    rp = np.ascontiguousarray(rowptr, dtype=np.int64)
    ci = np.ascontiguousarray(colidx, dtype=np.int32)
    rows = rp.size - 1
    grouping = np.zeros(max(rows, 1), np.int64)
    perm = np.zeros(max(rows, 1), np.int64)
    L = lib()
    L.smat_cluster_rows.argtypes = L.smat_reorder_rows.argtypes
    _check(L.smat_cluster_rows(rows, rp.ctypes.data, ci.ctypes.data if ci.size else None, tau, col_block, max_group_rows, threads,
                               grouping.ctypes.data, perm.ctypes.data))
    return grouping[:rows], perm[:rows]


def apply_row_permutation(rowptr, colidx, vals, perm):
    """CSR with rows permuted: new row r = old row perm[r] (CSR::permute_rows,
    preprocess/src/general/csr.cpp:65-74).  Unlike the reference's text round trip, which drops the
    values (preprocess/test/general/Matrix_Blocking.cpp:46, src/reorder.py:39-40), values are carried."""
    rowptr = np.asarray(rowptr, dtype=np.int64)
    perm = np.asarray(perm, dtype=np.int64)
    lens = np.diff(rowptr)[perm]
    new_rp = np.zeros(rowptr.size, np.int64)
    np.cumsum(lens, out=new_rp[1:])
    starts = rowptr[:-1][perm]
    idx = np.repeat(starts - new_rp[:-1], lens) + np.arange(new_rp[-1], dtype=np.int64)
    return new_rp.astype(np.int32), np.asarray(colidx)[idx], np.asarray(vals)[idx]


def apply_col_permutation(rowptr, colidx, vals, perm):
    """CSR with columns permuted, values carried: new column c = old column perm[c], i.e. an entry in old column j
    moves to column inv(perm)[j]; columns are re-sorted inside every row.  This is what the reference's column pass
    amounts to (src/reorder.py:143-182: transpose, reorder the rows of the transpose, which it leaves transposed and
    without values).  With A' = this matrix and B' = permute_rows_of_B(B, perm):  A' x B' == A x B."""
    rowptr = np.asarray(rowptr, dtype=np.int64)
    perm = np.asarray(perm, dtype=np.int64)
    inv = np.empty_like(perm)
    inv[perm] = np.arange(perm.size, dtype=np.int64)
    rows = np.repeat(np.arange(rowptr.size - 1, dtype=np.int64), np.diff(rowptr))
    new_cols = inv[np.asarray(colidx, dtype=np.int64)]
    order = np.lexsort((new_cols, rows))
    return rowptr.astype(np.int32), new_cols[order].astype(np.int32), np.asarray(vals)[order]


def permute_rows_of_B(B_nk, perm):
    """The dense operand that goes with apply_col_permutation: row k of the new B is row perm[k] of the old one.
    B_nk is the [N][K] array of the boundary (k contiguous), so the permutation acts on its second axis."""
    return np.ascontiguousarray(np.asarray(B_nk)[:, np.asarray(perm, dtype=np.int64)])


def reorder_cols(rowptr, colidx, K, tau=0.5, col_block=16, row_block=16, threads=0):
    """Column permutation by the reference's recipe (src/reorder.py:143-182, 206-219): the similarity reorder applied
    to the rows of the transpose.  Returns (grouping, perm) over the K columns."""
    rowptr = np.asarray(rowptr, dtype=np.int64)
    colidx = np.asarray(colidx, dtype=np.int64)
    rows = np.repeat(np.arange(rowptr.size - 1, dtype=np.int64), np.diff(rowptr))
    order = np.lexsort((rows, colidx))
    t_rp = np.zeros(K + 1, np.int64)
    np.cumsum(np.bincount(colidx, minlength=K), out=t_rp[1:])
    return reorder_rows(t_rp, rows[order].astype(np.int32), tau=tau, col_block=col_block, row_block=row_block, threads=threads)


def _take(ptr, n, ctype, dtype):
    a = np.ctypeslib.as_array(ptr, shape=(max(n, 1),))[:n].copy()
    lib().smat_free_host(C.cast(ptr, C.c_void_p))
    return a.view(dtype)


def bcsr_knapsack(M, K, rowptr, colidx, vals, threads=0):
    """Gap-skipping blocking (csrToBcsrKnapsacking, src/cuda_hgemm/src/common/matrix.h:504-671): 16x16 blocks that may
    start at any column.  Returns (bcsr_rowptr int32, start column per block int32, bcsr_vals float16)."""
    rp = np.ascontiguousarray(rowptr, dtype=np.int32)
    ci = np.ascontiguousarray(colidx, dtype=np.int32)
    v = np.ascontiguousarray(vals, dtype=np.float16).view(np.uint16)
    nnzb = C.c_size_t()
    prp, pci, pv = C.POINTER(C.c_int)(), C.POINTER(C.c_int)(), C.POINTER(C.c_uint16)()
    L = lib()
    L.smat_bcsr_knapsack.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_int, C.POINTER(C.c_size_t),
                                     C.POINTER(C.POINTER(C.c_int)), C.POINTER(C.POINTER(C.c_int)), C.POINTER(C.POINTER(C.c_uint16))]
    _check(L.smat_bcsr_knapsack(rp.ctypes.data, ci.ctypes.data if ci.size else None, v.ctypes.data if v.size else None, M, K,
                                threads, C.byref(nnzb), C.byref(prp), C.byref(pci), C.byref(pv)))
    return (_take(prp, M // 16 + 1, C.c_int, np.int32), _take(pci, nnzb.value, C.c_int, np.int32),
            _take(pv, nnzb.value * 256, C.c_uint16, np.float16))


def knapsack_to_csr(M, K, bcsr_rowptr, bcsr_colidx, bcsr_vals):
    """Back from the gap-skipping blocking to CSR (columns ascending; zero entries of a block are dropped)."""
    rp = np.ascontiguousarray(bcsr_rowptr, dtype=np.int32)
    ci = np.ascontiguousarray(bcsr_colidx, dtype=np.int32)
    v = np.ascontiguousarray(bcsr_vals, dtype=np.float16).view(np.uint16)
    nnz = C.c_size_t()
    prp, pci, pv = C.POINTER(C.c_int)(), C.POINTER(C.c_int)(), C.POINTER(C.c_uint16)()
    L = lib()
    L.smat_knapsack_to_csr.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.POINTER(C.c_size_t),
                                       C.POINTER(C.POINTER(C.c_int)), C.POINTER(C.POINTER(C.c_int)), C.POINTER(C.POINTER(C.c_uint16))]
    _check(L.smat_knapsack_to_csr(rp.ctypes.data, ci.ctypes.data if ci.size else None, v.ctypes.data if v.size else None, M, K,
                                  C.byref(nnz), C.byref(prp), C.byref(pci), C.byref(pv)))
    return (_take(prp, M + 1, C.c_int, np.int32), _take(pci, nnz.value, C.c_int, np.int32),
            _take(pv, nnz.value, C.c_uint16, np.float16))


def vbr_from_csr(M, K, rowptr, colidx, vals, grouping, col_block=16):
    """Variable-height blocking (VBR::fill_from_CSR_inplace with a grouping, preprocess/src/general/vbr.cpp:135-237):
    every group of rows becomes a block-row of its own height.  Returns a dict with the reference's arrays: row_part,
    row_perm, nzcount, jab (int64) and mab (float16, blocks column-major), plus col_block."""
    rp = np.ascontiguousarray(rowptr, dtype=np.int32)
    ci = np.ascontiguousarray(colidx, dtype=np.int32)
    v = np.ascontiguousarray(vals, dtype=np.float16).view(np.uint16)
    g = np.ascontiguousarray(grouping, dtype=np.int64)
    assert g.size == M
    i64pp, szp = C.POINTER(C.POINTER(C.c_int64)), C.POINTER(C.c_size_t)
    br, nb, nv = C.c_size_t(), C.c_size_t(), C.c_size_t()
    ppart, pperm, pnz, pjab, pmab = (C.POINTER(C.c_int64)(), C.POINTER(C.c_int64)(), C.POINTER(C.c_int64)(),
                                     C.POINTER(C.c_int64)(), C.POINTER(C.c_uint16)())
    L = lib()
    L.smat_vbr_from_csr.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t, szp, i64pp,
                                    i64pp, i64pp, szp, i64pp, szp, C.POINTER(C.POINTER(C.c_uint16))]
    _check(L.smat_vbr_from_csr(rp.ctypes.data, ci.ctypes.data if ci.size else None, v.ctypes.data if v.size else None, M, K,
                               g.ctypes.data, col_block, C.byref(br), C.byref(ppart), C.byref(pperm), C.byref(pnz), C.byref(nb),
                               C.byref(pjab), C.byref(nv), C.byref(pmab)))
    return {"col_block": col_block, "row_part": _take(ppart, br.value + 1, C.c_int64, np.int64),
            "row_perm": _take(pperm, M, C.c_int64, np.int64), "nzcount": _take(pnz, br.value, C.c_int64, np.int64),
            "jab": _take(pjab, nb.value, C.c_int64, np.int64), "mab": _take(pmab, nv.value, C.c_uint16, np.float16)}


def vbr_to_csr(M, K, vbr):
    """Back from the variable-height blocking to CSR (columns ascending; zero entries of a block are dropped)."""
    part = np.ascontiguousarray(vbr["row_part"], dtype=np.int64)
    perm = np.ascontiguousarray(vbr["row_perm"], dtype=np.int64)
    nz = np.ascontiguousarray(vbr["nzcount"], dtype=np.int64)
    jab = np.ascontiguousarray(vbr["jab"], dtype=np.int64)
    mab = np.ascontiguousarray(vbr["mab"], dtype=np.float16).view(np.uint16)
    nnz = C.c_size_t()
    prp, pci, pv = C.POINTER(C.c_int)(), C.POINTER(C.c_int)(), C.POINTER(C.c_uint16)()
    L = lib()
    L.smat_vbr_to_csr.argtypes = [C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                  C.c_void_p, C.POINTER(C.c_size_t), C.POINTER(C.POINTER(C.c_int)), C.POINTER(C.POINTER(C.c_int)),
                                  C.POINTER(C.POINTER(C.c_uint16))]
    _check(L.smat_vbr_to_csr(M, K, int(vbr["col_block"]), part.size - 1, part.ctypes.data, perm.ctypes.data,
                             nz.ctypes.data if nz.size else None, jab.ctypes.data if jab.size else None,
                             mab.ctypes.data if mab.size else None, C.byref(nnz), C.byref(prp), C.byref(pci), C.byref(pv)))
    return (_take(prp, M + 1, C.c_int, np.int32), _take(pci, nnz.value, C.c_int, np.int32),
            _take(pv, nnz.value, C.c_uint16, np.float16))


def b_slice_of_rank(N, world, rank):
    """Which rows of the [N][K] array B (= columns of the logical K x N matrix) a rank uploads in the sharded
    host-buffer product: (first, last + 1, rows per rank before the last one = the padded slice height).  Slices are
    multiples of 8 rows wide, like N itself."""
    per = ((N + world - 1) // world + 7) // 8 * 8
    lo = min(N, rank * per)
    hi = min(N, lo + per)
    return lo, hi, per


def gather_b_slices(B_host, staging, group=None):
    """Every rank copies its slice of B_host ([N][K], see b_slice_of_rank) into its part of ``staging``
    ([world * slice height][K], on the device the collective runs on), one all_gather fills the rest, and the [N][K]
    matrix is returned (a view of ``staging`` when the slices need no padding)."""
    import torch
    import torch.distributed as dist
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    N = B_host.shape[0]
    lo, hi, pad = b_slice_of_rank(N, world, rank)
    mine = staging[rank * pad:(rank + 1) * pad]
    mine[:hi - lo].copy_(B_host[lo:hi], non_blocking=True)
    # NCCL gathers in place (the rank's slice already sits where it belongs); other backends want a separate input
    # (as bytes: not every backend knows 16-bit element types)
    dist.all_gather_into_tensor(staging.view(torch.uint8), (mine if staging.is_cuda else mine.clone()).view(torch.uint8), group=group)
    if world * pad == N:
        return staging
    parts = []
    for r in range(world):
        a, b, _ = b_slice_of_rank(N, world, r)
        parts.append(staging[r * pad:r * pad + (b - a)])
    return torch.cat(parts)


def partition_block_rows(bcsr_rowptr_host, parts):
    """nnzb-balanced contiguous block-row ranges -> bounds int64[parts+1]."""
    rp = np.ascontiguousarray(bcsr_rowptr_host, dtype=np.int32)
    bounds = np.zeros(parts + 1, np.uint64)
    _check(lib().smat_partition_block_rows(rp.ctypes.data, rp.size - 1, parts, bounds.ctypes.data))
    return bounds.astype(np.int64)


def all_gather_rows(C_shard, bounds, out=None, group=None):
    """Optional exchange step after a sharded SpMM: every rank ends up with all rows of C.

    ``C_shard`` holds this rank's rows (block-rows [bounds[rank], bounds[rank + 1]) of the partition, 16 rows each);
    shards differ in height, so each is padded to the tallest one for one all_gather (NCCL over NVLink for CUDA
    tensors; any torch.distributed backend works) and the pieces are copied into ``out`` ([bounds[-1] * 16, N]).
    Not part of the timed SpMM: C is left sharded unless the caller asks for this."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    rows = [int(bounds[r + 1] - bounds[r]) * 16 for r in range(world)]
    N = C_shard.shape[1]
    assert C_shard.shape[0] == rows[dist.get_rank(group)]
    tallest = max(rows)
    padded = C_shard if C_shard.shape[0] == tallest else torch.cat(
        [C_shard, C_shard.new_zeros((tallest - C_shard.shape[0], N))])
    pieces = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(pieces, padded.contiguous(), group=group)
    if out is None:
        out = C_shard.new_empty((sum(rows), N))
    at = 0
    for r in range(world):
        out[at:at + rows[r]].copy_(pieces[r][:rows[r]])
        at += rows[r]
    return out


# ------------------------------------------------------------------------------------------------
# device objects
# ------------------------------------------------------------------------------------------------
class Matrix:
    """Dense fp16 device matrix (src/cuda_hgemm/src/common/matrix.h:18-139).  ``data`` is a torch
    CUDA tensor; for B it has shape [N, K] (K contiguous), for C shape [M, N]."""

    def __init__(self, rows, cols, name="Matrix", device="cuda", fill=None):
        import torch
        self.rows, self.cols, self.name = rows, cols, name
        self.data = torch.empty((rows, cols), dtype=torch.float16, device=device)
        if fill is not None:
            self.data.fill_(fill)

    @classmethod
    def from_host(cls, array, name="Matrix", device="cuda"):
        import torch
        m = cls.__new__(cls)
        a = np.ascontiguousarray(array, dtype=np.float16)
        m.rows, m.cols, m.name = a.shape[0], a.shape[1], name
        m.data = torch.from_numpy(a.view(np.int16)).to(device).view(torch.float16)
        return m

    def getDevPtr(self):
        return self.data.data_ptr()

    def checkValue(self, other):
        """max / average absolute difference (matrix.h:103-121)."""
        d = (self.data.float() - other.data.float()).abs()
        return float(d.max()), float(d.mean())


class SparseMatrix:
    """Sparse matrix blocked on the device (src/cuda_hgemm/src/common/matrix.h:143-721).

    Built from a host CSR (``from_csr``) or a Matrix-Market file (``from_file``, the reference's
    constructor path readCsr -> csrToBcsr -> upload, matrix.h:145-202).  The CSR is uploaded and the
    16x16 BCSR is built ON THE DEVICE by the library (smat_bcsr_count / smat_bcsr_fill)."""

    def __init__(self):
        self.M = self.K = self.nnz = self.nnzb = 0
        self.bcsrRowPtr = self.bcsrColIdx = self.bcsrVal = None

    @classmethod
    def from_csr(cls, M, K, rowptr, colidx, vals, device="cuda", keep_csr=False):
        import torch
        self = cls()
        self.M, self.K, self.nnz = int(M), int(K), int(len(colidx))
        dev = torch.device(device)
        with torch.cuda.device(dev):
            d_rp = torch.from_numpy(np.ascontiguousarray(rowptr, dtype=np.int32)).to(dev)
            d_ci = torch.from_numpy(np.ascontiguousarray(colidx, dtype=np.int32)).to(dev)
            d_v = torch.from_numpy(np.ascontiguousarray(vals, dtype=np.float16).view(np.int16)).to(dev)
            self.bcsrRowPtr = torch.empty(self.M // 16 + 1, dtype=torch.int32, device=dev)
            nnzb = C.c_size_t()
            L = lib()
            _check(L.smat_bcsr_count(d_rp.data_ptr(), d_ci.data_ptr(), self.M, self.K, self.nnz,
                                     self.bcsrRowPtr.data_ptr(), C.byref(nnzb), _stream()))
            self.nnzb = int(nnzb.value)
            self.bcsrColIdx = torch.empty(max(self.nnzb, 1), dtype=torch.int32, device=dev)
            self.bcsrVal = torch.empty(max(self.nnzb, 1) * 256, dtype=torch.float16, device=dev)
            _check(L.smat_bcsr_fill(d_rp.data_ptr(), d_ci.data_ptr(), d_v.data_ptr(), self.M, self.K, self.nnz,
                                    self.bcsrRowPtr.data_ptr(), self.bcsrColIdx.data_ptr(), self.bcsrVal.data_ptr(),
                                    self.nnzb, _stream()))
            torch.cuda.current_stream().synchronize()
            if keep_csr:
                self.csrRowPtr, self.csrColIdx, self.csrVal = d_rp, d_ci, d_v
        return self

    @classmethod
    def from_bcsr(cls, M, K, bcsr_rowptr, bcsr_colidx, bcsr_vals, device="cuda"):
        """Upload host BCSR arrays that are already in the kernel's layout."""
        import torch
        self = cls()
        self.M, self.K, self.nnzb = int(M), int(K), int(len(bcsr_colidx))
        dev = torch.device(device)
        self.bcsrRowPtr = torch.from_numpy(np.ascontiguousarray(bcsr_rowptr, dtype=np.int32)).to(dev)
        ci = np.ascontiguousarray(bcsr_colidx, dtype=np.int32)
        v = np.ascontiguousarray(bcsr_vals, dtype=np.float16).view(np.int16)
        if self.nnzb == 0:
            ci, v = np.zeros(1, np.int32), np.zeros(256, np.int16)
        self.bcsrColIdx = torch.from_numpy(ci).to(dev)
        self.bcsrVal = torch.from_numpy(v).to(dev).view(torch.float16)
        return self

    @classmethod
    def from_file(cls, filename, device="cuda"):
        M, K, rowptr, colidx, vals, _ = read_mtx(filename)
        return cls.from_csr(M, K, rowptr, colidx, vals, device=device)

    # getters named as in matrix.h:228-262
    def getRow(self):
        return self.M

    def getCol(self):
        return self.K

    def getNonzeroblocks(self):
        return self.nnzb

    def getBcsrValues(self):
        return self.bcsrVal.data_ptr()

    def getBcsrRowPtr(self):
        return self.bcsrRowPtr.data_ptr()

    def getBcsrColIdx(self):
        return self.bcsrColIdx.data_ptr()

    def host_arrays(self):
        rp = self.bcsrRowPtr.cpu().numpy()
        ci = self.bcsrColIdx.cpu().numpy()[: self.nnzb]
        v = self.bcsrVal.view(dtype=__import__("torch").int16).cpu().numpy().view(np.float16)[: self.nnzb * 256]
        return rp, ci, v


def spmm(A, B, Cout, check=False):
    """C = A x B through smat_spmm_bcsr_f16 (the mmaCBTKernel signature, mmaCBT.cu:83-88).
    B: Matrix / tensor [N, K]; Cout: Matrix / tensor [M, N]."""
    Bt = B.data if isinstance(B, Matrix) else B
    Ct = Cout.data if isinstance(Cout, Matrix) else Cout
    N = Bt.shape[0]
    assert Bt.shape[1] == A.K and tuple(Ct.shape) == (A.M, N) and Bt.is_contiguous() and Ct.is_contiguous()
    _check(lib().smat_spmm_bcsr_f16(A.getBcsrValues(), A.getBcsrRowPtr(), A.getBcsrColIdx(), Bt.data_ptr(),
                                    Ct.data_ptr(), A.M, N, A.K, A.nnzb, None, None, _stream()))
    if check:
        _check(lib().smat_device_status(_stream()))


def spmm_rows(A, B, Cshard, brow_begin, brow_end, check=False):
    """Block-rows [brow_begin, brow_end) of C = A x B into ``Cshard`` ([16*(end-begin), N])."""
    Bt = B.data if isinstance(B, Matrix) else B
    Ct = Cshard.data if isinstance(Cshard, Matrix) else Cshard
    N = Bt.shape[0]
    assert tuple(Ct.shape) == ((brow_end - brow_begin) * 16, N)
    _check(lib().smat_spmm_bcsr_f16_rows(A.getBcsrValues(), A.getBcsrRowPtr(), A.getBcsrColIdx(), Bt.data_ptr(),
                                         Ct.data_ptr(), A.M, N, A.K, A.nnzb, brow_begin, brow_end, _stream()))
    if check:
        _check(lib().smat_device_status(_stream()))


class Plan:
    """Reusable multiplication plan for block-rows [brow_begin, brow_end) of A (smat_plan_*)."""

    def __init__(self, A, brow_begin=0, brow_end=None, n_hint=0):
        self.A = A
        self.brow_begin = brow_begin
        self.brow_end = A.M // 16 if brow_end is None else brow_end
        h = C.c_void_p()
        _check(lib().smat_plan_create(C.byref(h), A.getBcsrValues(), A.getBcsrRowPtr(), A.getBcsrColIdx(), A.M, A.K,
                                      A.nnzb, self.brow_begin, self.brow_end, int(n_hint), _stream()))
        self._h = h

    def set_values(self):
        """Re-reads A's value array after it changed (same structure)."""
        _check(lib().smat_plan_set_values(self._h, self.A.getBcsrValues(), _stream()))

    def info(self):
        """{'tall': bool, 'rows_per_item': int, 'steps': int, 'kernel': name of the CUDA kernel that multiplies}."""
        t, r, n = C.c_int(0), C.c_int(0), C.c_size_t(0)
        _check(lib().smat_plan_info(self._h, C.addressof(t), C.addressof(r), C.addressof(n)))
        return {"tall": bool(t.value), "rows_per_item": r.value, "steps": n.value,
                "kernel": "spmm_bcsr_tall_kernel" if t.value else "spmm_bcsr_tc_kernel"}

    def spmm(self, B, Cout, check=False):
        Bt = B.data if isinstance(B, Matrix) else B
        Ct = Cout.data if isinstance(Cout, Matrix) else Cout
        N = Bt.shape[0]
        assert Bt.shape[1] == self.A.K and tuple(Ct.shape) == ((self.brow_end - self.brow_begin) * 16, N)
        assert Bt.is_contiguous() and Ct.is_contiguous()
        _check(lib().smat_plan_spmm(self._h, Bt.data_ptr(), Ct.data_ptr(), N, _stream()))
        if check:
            _check(lib().smat_device_status(_stream()))

    def spmm_host(self, B_host, C_host):
        """B_host [N][K], C_host [rows][N]: CPU tensors (pinned for overlap); copies pipelined with the multiply."""
        N = B_host.shape[0]
        assert B_host.shape[1] == self.A.K and tuple(C_host.shape) == ((self.brow_end - self.brow_begin) * 16, N)
        assert B_host.is_contiguous() and C_host.is_contiguous() and not B_host.is_cuda and not C_host.is_cuda
        assert B_host.element_size() == 2 and C_host.element_size() == 2
        _check(lib().smat_plan_spmm_host(self._h, B_host.data_ptr(), C_host.data_ptr(), N, _stream()))

    def spmm_host_sharded(self, B_host, C_host, group=None):
        """The host-buffer product for a plan that is one rank's shard of a multi-GPU run.  B is replicated on the
        device side, but every rank taking all of it over PCIe each step makes G ranks pull G copies through the host;
        here a rank uploads only its 1/G of B's columns (a contiguous row range of the [N][K] array, see
        ``b_slice_of_rank``), the slices are exchanged on the device with one all_gather (NCCL over NVLink for CUDA
        tensors; every kernel still reads local memory only), then the shard is multiplied and its rows of C copied out.
        B_host / C_host as in ``spmm_host``; every rank passes the same B_host."""
        import torch
        import torch.distributed as dist
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        N, K = B_host.shape
        rows = (self.brow_end - self.brow_begin) * 16
        assert K == self.A.K and tuple(C_host.shape) == (rows, N) and B_host.element_size() == 2
        dev = torch.device("cuda", torch.cuda.current_device())
        _, _, pad = b_slice_of_rank(N, world, rank)
        if getattr(self, "_sh", None) is None or self._sh[0].shape != (world * pad, K) or self._sh[0].dtype != B_host.dtype:
            self._sh = (torch.empty((world * pad, K), dtype=B_host.dtype, device=dev),
                        torch.empty((rows, N), dtype=C_host.dtype, device=dev))
        Bd, Cd = self._sh
        B_full = gather_b_slices(B_host, Bd, group)
        _check(lib().smat_plan_spmm(self._h, B_full.data_ptr(), Cd.data_ptr(), N, _stream()))
        C_host.copy_(Cd, non_blocking=True)

    def close(self):
        if self._h is not None:
            lib().smat_plan_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Tester:
    """Timing harness (src/cuda_hgemm/src/common/tester.h:12-73, 166-209, 338-377): warm-up
    launches, then ``profiling_iterations`` launches timed as one region.  Differences: CUDA events
    on the launch stream instead of gettimeofday (tester.h:339-361), and the throughput counts N:
    2*16*16*N*nnzb / t (the reference's print omits N, tester.h:362-363)."""

    def __init__(self, A, N, warmup_iterations=1, profiling_iterations=10, B=None):
        import torch
        assert warmup_iterations > 0 and profiling_iterations > 0  # HGEMM_CHECK_GT, tester.h:24-29
        self.A, self.N = A, N
        self.warmup_iterations, self.profiling_iterations = warmup_iterations, profiling_iterations
        self.B = B if B is not None else Matrix(N, A.K, "Matrix B", fill=1.0)  # all ones, matrix.h:38
        self.C = Matrix(A.M, N, "Matrix C")
        self.profiling_time_ms = 0.0
        self.throughput_tflops = 0.0
        self.plan = Plan(A, n_hint=N)
        self._torch = torch

    def evaluateSparse2(self, name="smat_b200"):
        torch = self._torch
        for _ in range(self.warmup_iterations):
            self.plan.spmm(self.B, self.C)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(self.profiling_iterations):
            self.plan.spmm(self.B, self.C)
        e1.record()
        torch.cuda.synchronize()
        _check(lib().smat_device_status(_stream()))
        self.profiling_time_ms = e0.elapsed_time(e1) / self.profiling_iterations
        flops = 2.0 * 256.0 * self.N * self.A.nnzb
        self.throughput_tflops = flops * 1e-12 / (self.profiling_time_ms * 1e-3)
        return self.profiling_time_ms, self.throughput_tflops
