"""The CPU oracle against the reference's own known answers and against fixtures generated from the
unmodified reference (tests/golden/make_golden.py)."""
import glob
import json
import os

import numpy as np
import pytest

import oracle
from smat_b200 import generators as gen


def test_half_rounding_matches_ieee():
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(5000) * 10.0 ** rng.integers(-9, 6, 5000),
                        [0.0, -0.0, 65504, 65519.99, 65520, 1e-8, 5.96e-8, 2.9802322387695312e-08, 6.1e-5, 1e30]])
    L = oracle.lib()
    got = np.array([L.orc_double_to_half_bits(float(v)) for v in x], np.uint16)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(got, want)


def test_similarity_known_answers(golden_dir):
    """TEST_similarities' fixed rows (preprocess/test/general/TEST_similarities.cpp:14-16)."""
    kat = json.load(open(os.path.join(golden_dir, "similarities.json")))
    A, B = kat["row_A"], kat["row_B"]
    for b in ("1", "3", "4", "16"):
        assert oracle.hamming_group(A, 1, B, 1, int(b)) == pytest.approx(kat[b]["Hamming"], abs=1e-6)
        assert oracle.jaccard_group(A, 1, B, 1, int(b)) == pytest.approx(kat[b]["Jaccard"], abs=1e-6)


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "reorder_*.npz"))),
                         ids=lambda p: os.path.basename(p)[8:-4])
def test_reorder_matches_reference_program(path):
    z = np.load(path)
    g, p = oracle.reorder_rows(z["rowptr"], z["cols"].astype(np.int64), tau=float(z["tau"]),
                               col_block=int(z["col_block"]), row_block=int(z["row_block"]))
    assert np.array_equal(g, z["grouping"])
    assert np.array_equal(p, z["perm"])


@pytest.mark.parametrize("name", ["band", "uniform", "llm"])
def test_multiply_matches_reference_vbr(golden_dir, name):
    z = np.load(os.path.join(golden_dir, f"multiply_{name}.npz"))
    M, K, N = int(z["M"]), int(z["K"]), int(z["N"])
    brp, bci, bv = oracle.csr_to_bcsr(M, K, z["rowptr"], z["colidx"], z["vals"])
    assert np.array_equal(brp, z["bcsr_rowptr"]) and np.array_equal(bci, z["bcsr_colidx"])
    assert np.array_equal(bv.view(np.uint16), z["bcsr_vals"].view(np.uint16))
    C = oracle.bcsr_spmm(bv, brp, bci, z["B_nk"], M, N, K)
    # same fp32 operations in the same order as VBR::multiply -> identical bits
    assert np.array_equal(C.view(np.uint32), z["C_f32"].view(np.uint32))


READER_FIXTURES = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "reader_*.npz")))


@pytest.mark.parametrize("path", READER_FIXTURES, ids=lambda p: os.path.basename(p)[7:-4])
def test_reader_and_blocking_match_reference_run(path, tmp_path):
    """The reference's own mmio_allinone + SparseMatrix::csrToBcsr were run on these Matrix-Market texts (fixtures made
    by tests/golden/make_golden.py): the oracle's reader and blocked-format builder must give the same arrays, bit for bit."""
    z = np.load(path)
    mtx = str(tmp_path / "m.mtx")
    with open(mtx, "wb") as f:
        f.write(z["mtx"].tobytes())
    M, K, rp, ci, v, _ = oracle.read_mtx(mtx)
    assert (M, K) == (int(z["M"]), int(z["K"]))
    assert np.array_equal(rp, z["csr_rowptr"]) and np.array_equal(ci, z["csr_colidx"])
    assert np.array_equal(v.view(np.uint16), z["csr_vals"].view(np.uint16))
    brp, bci, bv = oracle.csr_to_bcsr(M, K, rp, ci, v)
    assert np.array_equal(brp, z["bcsr_rowptr"]) and np.array_equal(bci, z["bcsr_colidx"])
    assert np.array_equal(bv.view(np.uint16), z["bcsr_vals"].view(np.uint16))
    if oracle.have_ref() and hasattr(oracle.ref(), "ref_vbr_from_csr"):
        # a second, independent piece of the reference: its CPU blocking code (VBR::fill_from_CSR_inplace)
        vrp, vci, vv = oracle.ref_bcsr_via_vbr(M, K, rp, ci, v)
        assert np.array_equal(vrp, brp) and np.array_equal(vci, bci)
        if len(np.unique(np.stack([np.repeat(np.arange(M), np.diff(rp)), ci]), axis=1).T) == len(ci):  # no duplicate entries
            assert np.array_equal(vv.view(np.uint16), bv.view(np.uint16))


def test_reader_and_blocking_match_live_reference(tmp_path):
    """Where oracle/_ref holds the reference's reader and builder (compiled from its sources): fuzz against them."""
    G = oracle.ref_gpu()
    if G is None or not hasattr(G, "ref_sparse_matrix_load"):
        pytest.skip("oracle/_ref/libsmat_ref_gpu.so is not built here")
    rng = np.random.default_rng(5)
    for case in range(6):
        M, K = int(rng.integers(1, 200)), int(rng.integers(1, 200))
        n = int(rng.integers(1, 800))
        rows, cols = rng.integers(0, M, n), rng.integers(0, K, n)
        rows[-1], cols[-1] = M - 1, K - 1
        path = str(tmp_path / f"f{case}.mtx")
        with open(path, "w") as f:
            f.write(f"%%MatrixMarket matrix coordinate real general\n{M} {K} {n}\n")
            f.write("".join(f"{r + 1} {c + 1} {v!r}\n" for r, c, v in zip(rows.tolist(), cols.tolist(), rng.standard_normal(n).tolist())))
        ref = oracle.ref_sparse_matrix(path, host_only=True)
        Mo, Ko, rp, ci, v, _ = oracle.read_mtx(path)
        assert (Mo, Ko) == ref[:2] and np.array_equal(rp, ref[2]) and np.array_equal(ci, ref[3])
        assert np.array_equal(v.view(np.uint16), ref[4].view(np.uint16))
        brp, bci, bv = oracle.csr_to_bcsr(Mo, Ko, rp, ci, v)
        assert np.array_equal(brp, ref[5]) and np.array_equal(bci, ref[6])
        assert np.array_equal(bv.view(np.uint16), ref[7].view(np.uint16))


def _dense_bcsr(M, K, rowptr, colidx, vals):
    """Independent numpy construction of the BCSR arrays from a dense scatter."""
    D = np.zeros((M, K), np.float16)
    present = np.zeros((M // 16, K // 16), bool)
    rows = np.repeat(np.arange(M), np.diff(rowptr))
    for r, c, v in zip(rows, colidx, vals):  # sequential: last duplicate wins
        D[r, c] = v
        present[r // 16, c // 16] = True
    brp = np.zeros(M // 16 + 1, np.int32)
    brp[1:] = np.cumsum(present.sum(1))
    br, bc = np.nonzero(present)
    bv = np.stack([D[16 * r:16 * r + 16, 16 * c:16 * c + 16] for r, c in zip(br, bc)]).reshape(-1) if len(br) else \
        np.zeros(0, np.float16)
    return brp, (bc * 16).astype(np.int32), bv


def test_csr_to_bcsr_against_dense_construction():
    rng = np.random.default_rng(3)
    M, K = 96, 160
    n = 700
    r = np.sort(rng.integers(0, M, n))
    c = rng.integers(0, K, n)  # unsorted columns, duplicates likely
    v = rng.standard_normal(n).astype(np.float16)
    v[::7] = 0  # explicit zeros still create blocks (matrix.h:388-404)
    rowptr = np.zeros(M + 1, np.int32)
    rowptr[1:] = np.cumsum(np.bincount(r, minlength=M))
    got = oracle.csr_to_bcsr(M, K, rowptr, c.astype(np.int32), v)
    want = _dense_bcsr(M, K, rowptr, c, v)
    for a, b in zip(got, want):
        assert np.array_equal(np.asarray(a).view(np.uint16) if a.dtype == np.float16 else a,
                              np.asarray(b).view(np.uint16) if b.dtype == np.float16 else b)


def test_band_config_block_count():
    """The band matrix (n = 4096, half-bandwidth 64): 9 blocks per block-row minus the 20 cut off at the two edges."""
    p = gen.make_config("band")
    brp, bci, _ = oracle.csr_to_bcsr(p.M, p.K, p.rowptr, p.colidx, p.vals)
    assert len(bci) == 2284 and brp[-1] == 2284


def test_mtx_reader_symmetric_pattern_and_padding(tmp_path):
    f = tmp_path / "s.mtx"
    f.write_text("%%MatrixMarket matrix coordinate pattern symmetric\n% comment\n5 5 4\n1 1\n3 1\n5 2\n4 4\n")
    M, K, rowptr, colidx, vals, sym = oracle.read_mtx(str(f))
    assert (M, K, sym) == (16, 16, True)
    assert rowptr[:6].tolist() == [0, 2, 3, 4, 5, 6] and rowptr[-1] == 6
    assert colidx.tolist() == [0, 2, 4, 0, 3, 1]  # file order with mirrors interleaved
    assert np.all(vals == np.float16(1.0))


@pytest.mark.skipif(not oracle.have_ref(), reason="oracle/_ref not built (reference tree absent)")
def test_live_reference_fuzz(tmp_path):
    """Restated Keeper clustering vs the real reference code on random patterns with merges."""
    R = oracle.ref()
    rng = np.random.default_rng(11)
    for case in range(40):
        n = int(rng.integers(8, 150))
        ncols = int(rng.integers(8, 300))
        rb, cb, tau = [(4, 16, 0.5), (16, 16, 0.5), (16, 4, 0.3), (3, 3, 0.6), (16, 16, 0.8)][case % 5]
        rows, cols = [], []
        for i in range(n):
            c = np.unique(rng.integers(0, ncols, rng.integers(0, 9)))
            if i == n - 1:
                c = np.unique(np.append(c, ncols - 1))
            rows += [i] * len(c)
            cols += list(c)
        rowptr = np.zeros(n + 1, np.int64)
        rowptr[1:] = np.cumsum(np.bincount(np.array(rows, dtype=np.int64), minlength=n))
        cols = np.array(cols, dtype=np.int64)
        el = tmp_path / f"m{case}.el"
        np.savetxt(el, np.stack([np.array(rows), cols], 1), fmt="%d")
        G, P = np.zeros(n, np.int64), np.zeros(n, np.int64)
        assert R.ref_group_and_permute(str(el).encode(), tau, cb, rb, 1, n, G, P) == n
        g, p = oracle.reorder_rows(rowptr, cols, tau=tau, col_block=cb, row_block=rb)
        assert np.array_equal(G, g) and np.array_equal(P, p), case
        # without -F 1: the clustering's own grouping (unequal groups) and its permutation, from the product
        import smat_b200 as S
        assert R.ref_group_and_permute(str(el).encode(), tau, cb, rb, 0, n, G, P) == n
        g, p = S.cluster_rows(rowptr, cols, tau=tau, col_block=cb, max_group_rows=rb)
        assert np.array_equal(G, g) and np.array_equal(P, p), case
        g2, p2 = S.reorder_rows(rowptr, cols, tau=tau, col_block=cb, row_block=rb)
        fixed = np.zeros(n, np.int64)
        R.ref_fixed_size_grouping(n, G, rb, fixed)
        assert np.array_equal(fixed, g2), case


@pytest.mark.skipif(not (oracle.have_ref() and hasattr(oracle.ref(), "ref_vbr_from_grouping")),
                    reason="oracle/_ref not built (reference tree absent)")
def test_variable_height_blocking_matches_live_reference():
    """smat_vbr_from_csr against the unmodified VBR::fill_from_CSR_inplace(cmat, grouping, col_block) run here, on
    random matrices and groupings (many equal keys: the order inside a group is the unstable sort's)."""
    import smat_b200 as S
    rng = np.random.default_rng(77)
    for _ in range(25):
        M, K = int(rng.integers(1, 120)), int(rng.integers(1, 90))
        cb = int(rng.integers(1, 20))
        mask = rng.random((M, K)) < rng.uniform(0.02, 0.4)
        vals = (rng.standard_normal((M, K)) * mask).astype(np.float16)
        mask = vals != 0
        rowptr = np.zeros(M + 1, np.int32)
        rowptr[1:] = np.cumsum(mask.sum(axis=1))
        colidx = np.nonzero(mask)[1].astype(np.int32)
        g = rng.integers(0, max(1, M // int(rng.integers(1, 20))) + 1, M).astype(np.int64)
        want = oracle.ref_vbr_from_grouping(M, K, rowptr, colidx, vals[mask], g, cb)
        got = S.vbr_from_csr(M, K, rowptr, colidx, vals[mask], g, cb)
        for key in ("row_part", "row_perm", "nzcount", "jab"):
            assert np.array_equal(got[key], want[key]), key
        assert np.array_equal(got["mab"].astype(np.float32), want["mab"])
