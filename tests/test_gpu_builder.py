"""Device-side BCSR builder (through the C ABI) against the reference's csrToBcsr -- fixtures made by running the
unmodified reference, the reference itself where it was built, and the oracle's restatement for the larger cases: row
pointers, column indices and values must be bit-identical."""
import glob
import os

import numpy as np
import pytest

import oracle
import smat_b200 as S
from smat_b200 import generators as gen

pytestmark = pytest.mark.gpu


def _same(A, brp, bci, bv):
    rp, ci, v = A.host_arrays()
    assert A.nnzb == len(bci)
    assert np.array_equal(rp, brp)
    assert np.array_equal(ci, bci)
    assert np.array_equal(v.view(np.uint16), bv.view(np.uint16))


@pytest.mark.parametrize("name,scale", [("band", 1.0), ("uniform", 0.05), ("powerlaw", 0.03), ("clustered", 0.01),
                                        ("llm", 0.125)])
def test_builder_matches_oracle_on_configs(name, scale):
    p = gen.make_config(name, scale=scale)
    A = S.SparseMatrix.from_csr(p.M, p.K, p.rowptr, p.colidx, p.vals)
    _same(A, *oracle.csr_to_bcsr(p.M, p.K, p.rowptr, p.colidx, p.vals))


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "reader_*.npz"))),
                         ids=lambda p: os.path.basename(p)[7:-4])
def test_file_to_bcsr_matches_reference_run(path, tmp_path):
    """The product's whole front end -- smat_read_mtx, upload, smat_bcsr_count / smat_bcsr_fill on the device -- against
    what the reference's own SparseMatrix(file) (mmio_allinone + csrToBcsr) produced for the same Matrix-Market text."""
    z = np.load(path)
    mtx = str(tmp_path / "m.mtx")
    with open(mtx, "wb") as f:
        f.write(z["mtx"].tobytes())
    A = S.SparseMatrix.from_file(mtx)
    assert (A.M, A.K) == (int(z["M"]), int(z["K"]))
    _same(A, z["bcsr_rowptr"], z["bcsr_colidx"], z["bcsr_vals"])


def test_file_to_bcsr_matches_live_reference_constructor(tmp_path):
    """Where the reference's SparseMatrix was compiled for this GPU (oracle/_ref/libsmat_ref_gpu.so): run its real
    constructor -- reader, csrToBcsr, uploads -- on a fresh file and compare the product's device-built arrays with it."""
    G = oracle.ref_gpu()
    if G is None or not hasattr(G, "ref_sparse_matrix_load"):
        pytest.skip("oracle/_ref/libsmat_ref_gpu.so is not built here")
    p = gen.make_config("uniform", scale=0.02)
    path = str(tmp_path / "u.mtx")
    gen.write_mtx(path, p.M, p.K, p.rowptr, p.colidx, p.vals)
    M, K, crp, cci, cv, brp, bci, bv = oracle.ref_sparse_matrix(path, host_only=False)
    A = S.SparseMatrix.from_file(path)
    assert (A.M, A.K) == (M, K)
    _same(A, brp, bci, bv)


def test_builder_unsorted_columns_duplicates_and_explicit_zeros():
    rng = np.random.default_rng(3)
    M, K, n = 160, 4096, 30000
    r = np.sort(rng.integers(0, M, n))
    r[r // 16 == 3] = 2 * 16  # block-row 3 empty
    r = np.sort(r)
    c = rng.integers(0, K, n)
    c[:4000] = rng.integers(0, 64, 4000)  # many duplicates in the first rows
    v = rng.standard_normal(n).astype(np.float16)
    v[::5] = 0
    rowptr = np.zeros(M + 1, np.int32)
    rowptr[1:] = np.cumsum(np.bincount(r, minlength=M))
    A = S.SparseMatrix.from_csr(M, K, rowptr, c.astype(np.int32), v)
    _same(A, *oracle.csr_to_bcsr(M, K, rowptr, c.astype(np.int32), v))


def test_builder_empty_and_tiny():
    A = S.SparseMatrix.from_csr(32, 32, np.zeros(33, np.int32), np.zeros(0, np.int32), np.zeros(0, np.float16))
    assert A.nnzb == 0 and A.bcsrRowPtr.cpu().tolist() == [0, 0, 0]
    rowptr = np.zeros(17, np.int32)
    rowptr[16:] = 1
    A = S.SparseMatrix.from_csr(16, 16, rowptr, np.array([15], np.int32), np.array([2.5], np.float16))
    rp, ci, v = A.host_arrays()
    assert rp.tolist() == [0, 1] and ci.tolist() == [0] and v[255] == np.float16(2.5) and np.count_nonzero(v) == 1


def test_builder_from_mtx_file(tmp_path):
    p = gen.make_config("band", scale=0.05)
    path = str(tmp_path / "b.mtx")
    gen.write_mtx(path, p.M, p.K, p.rowptr, p.colidx, p.vals)
    A = S.SparseMatrix.from_file(path)
    _same(A, *oracle.csr_to_bcsr(p.M, p.K, p.rowptr, p.colidx, p.vals))


def test_builder_full_size_llm_structure():
    """The block-sparse weight layer at full size: exact block count and a checksum of the value array."""
    p = gen.make_config("llm")
    A = S.SparseMatrix.from_csr(p.M, p.K, p.rowptr, p.colidx, p.vals)
    assert A.nnzb == 183501
    rp, ci, v = A.host_arrays()
    assert rp[-1] == 183501 and np.all(np.diff(ci.astype(np.int64))[np.diff(np.repeat(np.arange(p.M // 16), np.diff(rp))) == 0] > 0)
    assert int(v.view(np.uint16).astype(np.uint64).sum()) == int(p.vals.view(np.uint16).astype(np.uint64).sum())
