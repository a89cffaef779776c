"""smat_spmm_bcsr_f16_static -- the SpMM entry point for hosts that must not allocate device memory
(fixed-budget serving loops, callbacks running under an allocator lock).  It keeps its per-call plan
in a fixed array inside the library image, shared by all calls.  The test drives it through the C ABI
twice in a row, with different inputs, and requires the same bits as the allocating entry point
(both run the same kernels, so the tolerance is zero), then checks that oversize inputs are refused.
Collected last on purpose: a failure here cannot hide failures elsewhere in a run that stops early."""
import ctypes

import numpy as np
import pytest

import oracle
import smat_b200 as S
from smat_b200 import generators as gen

pytestmark = pytest.mark.gpu


def _device_memory_in_use():
    """(bytes in use on the device as the driver sees it, bytes handed out by the device's default stream-ordered
    pool): neither may move across a call that claims to allocate nothing."""
    import torch
    free, total = torch.cuda.mem_get_info()
    rt = None
    for name in ("libcudart.so.12", "libcudart.so"):
        try:
            rt = ctypes.CDLL(name)
            break
        except OSError:
            continue
    used_pool = -1
    if rt is not None:
        pool = ctypes.c_void_p()
        if rt.cudaDeviceGetDefaultMemPool(ctypes.byref(pool), torch.cuda.current_device()) == 0:
            val = ctypes.c_uint64(0)
            if rt.cudaMemPoolGetAttribute(pool, 7, ctypes.byref(val)) == 0:  # cudaMemPoolAttrUsedMemCurrent
                used_pool = int(val.value)
    return total - free, used_pool


def _both(p, brp, bci, bv, B_nk):
    import torch
    A = S.SparseMatrix.from_bcsr(p.M, p.K, brp, bci, bv)
    B = S.Matrix.from_host(B_nk)
    N = B_nk.shape[0]
    want = S.Matrix(p.M, N, fill=float("nan"))
    S.spmm(A, B, want, check=True)
    got = S.Matrix(p.M, N, fill=float("nan"))
    L = S.lib()
    args = (A.getBcsrValues(), A.getBcsrRowPtr(), A.getBcsrColIdx(), B.data.data_ptr(), got.data.data_ptr(), p.M, N, p.K,
            A.nnzb, torch.cuda.current_stream().cuda_stream)
    rc = L.smat_spmm_bcsr_f16_static(*args)  # the first call on a device also looks up the array's address
    assert rc == 0, L.smat_last_error_string()
    torch.cuda.synchronize()
    # a further call with everything set up: device memory in use must not move, neither during nor after it
    before = _device_memory_in_use()
    rc = L.smat_spmm_bcsr_f16_static(*args)
    assert rc == 0, L.smat_last_error_string()
    during = _device_memory_in_use()
    torch.cuda.synchronize()
    after = _device_memory_in_use()
    assert before == during == after, (before, during, after)
    # device-side errors of the static entry point are visible through smat_device_status
    assert L.smat_device_status(torch.cuda.current_stream().cuda_stream) == 0, L.smat_last_error_string()
    return want.data.cpu().numpy(), got.data.cpu().numpy()


def _same(a, b):
    """The allocating entry point may compute a work item in parts (fp32 partial tiles added up afterwards),
    the static one never does: equal up to the one rounding of differently grouped fp32 sums to fp16."""
    a = a.astype(np.float32)
    b = b.astype(np.float32)
    return bool(np.all(np.abs(a - b) <= 2.0 ** -9 * np.maximum(np.abs(a), np.abs(b)) + 1e-3 * float(np.abs(a).max())))


def test_static_scratch_entry_matches_allocating_entry_twice():
    rng = np.random.default_rng(5)
    # first call: the band configuration (2284 blocks)
    p = gen.make_config("band")
    brp, bci, bv = oracle.csr_to_bcsr(p.M, p.K, p.rowptr, p.colidx, p.vals)
    want, got = _both(p, brp, bci, bv, p.B_nk)
    assert _same(want, got)
    # second call right after it: another matrix and width, so leftovers of the first call in the
    # shared array would show
    p2 = gen.make_config("uniform", scale=0.03)
    brp2, bci2, bv2 = oracle.csr_to_bcsr(p2.M, p2.K, p2.rowptr, p2.colidx, p2.vals)
    B2 = rng.standard_normal((136, p2.K)).astype(np.float16)
    want2, got2 = _both(p2, brp2, bci2, bv2, B2)
    assert _same(want2, got2)
    # and against the oracle, like every other parity test (max relative error 1e-2)
    ref = oracle.bcsr_spmm(bv2, brp2, bci2, B2, p2.M, 136, p2.K)
    mag = oracle.bcsr_spmm(np.abs(bv2), brp2, bci2, np.abs(B2), p2.M, 136, p2.K)
    ref16 = ref.astype(np.float16).astype(np.float32)
    err = np.max(np.abs(got2.astype(np.float32) - ref16) / (np.maximum(np.abs(ref16), 1e-2 * mag) + 1e-30))
    assert err <= 1e-2


def test_static_scratch_entry_refuses_oversize_inputs():
    L = S.lib()
    buf = (ctypes.c_int * 64)()
    a = ctypes.addressof(buf) & ~15
    rc = L.smat_spmm_bcsr_f16_static(a, a, a, a, a, 16, 8, 16, 32769, None)
    assert rc == -6 and b"32768" in L.smat_last_error_string()
    rc = L.smat_spmm_bcsr_f16_static(a, a, a, a, a, 1048576 + 16, 8, 16, 1, None)
    assert rc == -6
