"""Generates the golden fixtures in this directory FROM THE UNMODIFIED REFERENCE.

Run in a container that has the reference tree (it is not needed to run the tests):

    make -C oracle ref REF=<reference tree>
    SMAT_REFERENCE=<reference tree> python tests/golden/make_golden.py

It drives the reference's own code through oracle/_ref (built from the reference sources by
oracle/Makefile): the Matrix_Blocking / TEST_similarities programs and, through the thin ctypes
doorway libsmat_ref.so, BlockingEngine::GetGrouping, get_permutation and VBR::multiply.  The inputs
are small seeded matrices, so the fixtures stay a few hundred KB.

Outputs:
  similarities.json     stdout figures of TEST_similarities for -b 1, 3, 4, 16
  reorder_<name>.npz    CSR pattern + reference grouping (.g file of Matrix_Blocking) + permutation
                        (from its *_reordered.el) for -a 5 -F 1 runs
  multiply_<name>.npz   BCSR arrays (blocked by the reference's VBR::fill_from_CSR_inplace) + B + fp32 C of the
                        reference's VBR::multiply
  reader_<name>.npz     a Matrix-Market text + the CSR and BCSR arrays that the reference's mmio_allinone and
                        SparseMatrix::csrToBcsr make of it, the arrays of its csrToBcsrKnapsacking, and for small cases
                        the bytes of its outputCsr export (needs `make -C oracle ref_gpu REF=...` too)
  formats/*             outputs of the reference's Python glue (src/reorder.py: mtx2el, el2mtx, row pass,
                        transpose, column pass) on a small pattern matrix
"""
import json
import os
import re
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from smat_b200 import generators as gen  # noqa: E402

REFDIR = oracle.ref_dir()


def similarities():
    out = {}
    for b in (1, 3, 4, 16):
        txt = subprocess.run([os.path.join(REFDIR, "TEST_similarities"), "-b", str(b)], capture_output=True, text=True,
                             check=True).stdout
        out[str(b)] = {k: float(v) for k, v in re.findall(r"(Hamming|Jaccard): ([-0-9.e]+)", txt)}
    out["row_A"] = [1, 2, 5, 10, 12, 20]
    out["row_B"] = [0, 2, 4, 10, 16]
    with open(os.path.join(HERE, "similarities.json"), "w") as f:
        json.dump(out, f, indent=1)
    print("similarities", out)


def run_matrix_blocking(rowptr, cols, tau, cb, rb):
    """Runs the reference PROGRAM on an edge list; returns (grouping from .g, permutation recovered
    from the reordered edge list)."""
    n = len(rowptr) - 1
    with tempfile.TemporaryDirectory() as d:
        el = os.path.join(d, "m.el")
        rows = np.repeat(np.arange(n), np.diff(rowptr))
        np.savetxt(el, np.stack([rows, cols], 1), fmt="%d")
        subprocess.run([os.path.join(REFDIR, "Matrix_Blocking"), "-f", el, "-a", "5", "-b", str(cb), "-B", str(rb), "-F",
                        "1", "-t", str(tau), "-o", os.path.join(d, "out"), "-v", "0"], check=True, capture_output=True)
        # the .g file is one line: "GROUPING,g0,g1,...," (preprocess/src/general/utilities.cpp:175-240)
        toks = open(os.path.join(d, "out.g")).read().strip().split(",")
        assert toks[0] == "GROUPING"
        g = np.array([int(t) for t in toks[1:] if t.strip() != ""], dtype=np.int64)
        reordered = np.loadtxt(os.path.join(d, "m_reordered.el"), dtype=np.int64, ndmin=2)
    return g, reordered


def random_pattern(n, ncols, kmax, seed, clustered=False):
    rng = np.random.default_rng(seed)
    rows, cols = [], []
    for i in range(n):
        if clustered:
            base = (i // 24) * 40 % max(1, ncols - 64)
            c = base + rng.integers(0, 64, rng.integers(1, kmax + 1))
        else:
            c = rng.integers(0, ncols, rng.integers(0, kmax + 1))
        c = np.unique(np.minimum(c, ncols - 1))
        if i == n - 1:
            c = np.unique(np.append(c, ncols - 1))
        rows += [i] * len(c)
        cols += list(c)
    rowptr = np.zeros(n + 1, np.int64)
    rowptr[1:] = np.cumsum(np.bincount(np.array(rows, dtype=np.int64), minlength=n))
    return rowptr, np.array(cols, dtype=np.int64)


def reorder_fixtures():
    R = oracle.ref()
    cases = {
        "random_small": (*random_pattern(96, 96, 5, 1), 0.5, 16, 16),
        "random_wide": (*random_pattern(200, 640, 12, 2), 0.5, 16, 16),
        "clustered": (*random_pattern(240, 400, 20, 3, clustered=True), 0.5, 16, 16),
        "clustered_tau08": (*random_pattern(160, 300, 10, 4, clustered=True), 0.8, 16, 16),
        "blocks3": (*random_pattern(60, 60, 6, 5), 0.6, 3, 3),
    }
    for name, sc in (("band", 0.125), ("uniform", 0.015625), ("powerlaw", 0.0078125), ("clustered_cfg", 0.003),
                     ("llm", 0.0625)):
        p = gen.make_config(name.replace("_cfg", ""), scale=sc)
        cases["cfg_" + name] = (p.rowptr.astype(np.int64), p.colidx.astype(np.int64), 0.5, 16, 16)
    for name, (rowptr, cols, tau, cb, rb) in cases.items():
        n = len(rowptr) - 1
        g_prog, reordered = run_matrix_blocking(rowptr, cols, tau, cb, rb)
        G = np.zeros(n, np.int64)
        P = np.zeros(n, np.int64)
        with tempfile.TemporaryDirectory() as d:
            el = os.path.join(d, "m.el")
            np.savetxt(el, np.stack([np.repeat(np.arange(n), np.diff(rowptr)), cols], 1), fmt="%d")
            got = R.ref_group_and_permute(el.encode(), tau, cb, rb, 1, n, G, P)
        assert got == n and np.array_equal(G, g_prog), name
        G_raw = np.zeros(n, np.int64)  # the clustering's own grouping (no -F 1) and its permutation
        P_raw = np.zeros(n, np.int64)
        with tempfile.TemporaryDirectory() as d:
            el = os.path.join(d, "m.el")
            np.savetxt(el, np.stack([np.repeat(np.arange(n), np.diff(rowptr)), cols], 1), fmt="%d")
            assert R.ref_group_and_permute(el.encode(), tau, cb, rb, 0, n, G_raw, P_raw) == n
        # the program's reordered edge list must be the CSR with rows taken in order P
        lens = np.diff(rowptr)[P]
        exp_rows = np.repeat(np.arange(n), lens)
        exp_cols = np.concatenate([cols[rowptr[r]:rowptr[r + 1]] for r in P]) if len(cols) else cols
        assert np.array_equal(reordered[:, 0], exp_rows) and np.array_equal(reordered[:, 1], exp_cols), name
        np.savez_compressed(os.path.join(HERE, f"reorder_{name}.npz"), rowptr=rowptr, cols=cols.astype(np.int32),
                            tau=np.float32(tau), col_block=cb, row_block=rb, grouping=G.astype(np.int32),
                            perm=P.astype(np.int32), raw_grouping=G_raw.astype(np.int32), raw_perm=P_raw.astype(np.int32))
        print("reorder", name, n, "rows; identity perm:", bool(np.array_equal(P, np.arange(n))))


def multiply_fixtures():
    R = oracle.ref()
    for name, sc, N in (("band", 0.03125, 24), ("uniform", 0.00390625, 40), ("llm", 0.03125, 16)):
        p = gen.make_config(name, scale=sc)
        # the blocked arrays come from the reference's own blocking code (VBR::fill_from_CSR_inplace), not from the oracle
        brp, bci, bv = oracle.ref_bcsr_via_vbr(p.M, p.K, p.rowptr, p.colidx, p.vals)
        rng = np.random.default_rng(7)
        B_nk = rng.standard_normal((N, p.K)).astype(np.float16)
        nb = len(bci)
        # reference VBR: blocks column-major inside, block-column indices, fp32, column-major B and C
        mab = np.ascontiguousarray(bv.reshape(nb, 16, 16).transpose(0, 2, 1)).astype(np.float32).reshape(-1)
        jab = (bci // 16).astype(np.int64)
        nzcount = np.diff(brp).astype(np.int64)
        Bf = np.ascontiguousarray(B_nk.astype(np.float32)).reshape(-1)          # [n][k] == column-major K x N
        Cf = np.zeros(p.M * N, np.float32)                                        # column-major M x N
        R.ref_vbr_multiply(p.M, p.K, p.M // 16, 16, nzcount, jab if nb else np.zeros(1, np.int64),
                           mab if nb else np.zeros(1, np.float32), nb, 16, Bf, N, Cf)
        C = Cf.reshape(N, p.M).T.copy()
        np.savez_compressed(os.path.join(HERE, f"multiply_{name}.npz"), M=p.M, K=p.K, N=N, rowptr=p.rowptr,
                            colidx=p.colidx, vals=p.vals, bcsr_rowptr=brp, bcsr_colidx=bci, bcsr_vals=bv, B_nk=B_nk,
                            C_f32=C)
        print("multiply", name, p.M, p.K, N, "nnzb", nb)


def reader_cases():
    """(name, Matrix-Market text) of the reader / blocked-format fixtures: every banner variant the reader accepts,
    shapes that are not multiples of 16, duplicate entries, unsorted columns, explicit zeros, and each benchmark
    configuration at a small scale."""
    rng = np.random.default_rng(31)
    cases = []

    def coo_text(banner, M, K, rows, cols, vals=None):
        lines = [f"%%MatrixMarket matrix coordinate {banner}", "% fixture", f"{M} {K} {len(rows)}"]
        for i in range(len(rows)):
            lines.append(f"{rows[i] + 1} {cols[i] + 1}" + ("" if vals is None else f" {vals[i]}"))
        return "\n".join(lines) + "\n"

    M, K = 253, 251
    keys = np.unique(rng.integers(0, M * K, 3000))
    rng.shuffle(keys)  # file order is kept inside the rows: columns end up unsorted
    cases.append(("general_real_shuffled", coo_text("real general", M, K, keys // K, keys % K,
                                                    [repr(float(v)) for v in rng.standard_normal(keys.size)])))
    n = 100
    keys = np.unique(rng.integers(0, n * n, 600))
    r, c = keys // n, keys % n
    low = r >= c
    cases.append(("symmetric_real", coo_text("real symmetric", n, n, r[low], c[low],
                                             [repr(float(v)) for v in rng.standard_normal(int(low.sum()))])))
    keys = np.unique(rng.integers(0, 70 * 90, 400))
    cases.append(("pattern_general", coo_text("pattern general", 70, 90, keys // 90, keys % 90)))
    keys = rng.integers(0, 40 * 48, 500)  # with repeats: duplicate (row, col) entries, the last one wins in a block
    cases.append(("integer_duplicates", coo_text("integer general", 40, 48, keys // 48, keys % 48,
                                                 [str(int(v)) for v in rng.integers(-9, 10, keys.size)])))
    keys = np.unique(rng.integers(0, 64 * 64, 300))
    vals = rng.standard_normal(keys.size)
    vals[::3] = 0.0  # stored zeros still make their block "nonzero"
    cases.append(("explicit_zeros", coo_text("real general", 64, 64, keys // 64, keys % 64, [repr(float(v)) for v in vals])))
    cases.append(("single_entry_last_corner", coo_text("real general", 33, 17, [32], [16], ["-2.5"])))
    for name, sc in (("band", 0.03), ("uniform", 0.01), ("powerlaw", 0.004), ("clustered", 0.0005), ("llm", 0.012)):
        p = gen.make_config(name, scale=sc)
        rows = np.repeat(np.arange(p.M), np.diff(p.rowptr))
        cases.append((f"cfg_{name}", coo_text("real general", p.M, p.K, rows, p.colidx,
                                              [repr(float(v)) for v in p.vals.astype(np.float32)])))
    return cases


def reader_fixtures():
    """Outputs of the reference's own mmio_allinone + SparseMatrix::csrToBcsr (compiled unmodified into
    oracle/_ref/libsmat_ref_gpu.so; both are host code and run without a GPU) on reader_cases()."""
    for name, text in reader_cases():
        with tempfile.TemporaryDirectory() as d:
            path = os.path.join(d, name + ".mtx")
            with open(path, "w") as f:
                f.write(text)
            # small cases also get the reference's export for the Magicube baseline (SparseMatrix::outputCsr writes
            # ./data/magicube_cop20k_A.mtx relative to the current directory)
            magicube = b""
            export = len(text) < 20000
            cwd = os.getcwd()
            os.makedirs(os.path.join(d, "data"))
            os.chdir(d)
            try:
                M, K, crp, cci, cv, brp, bci, bv = oracle.ref_sparse_matrix(path, host_only=True, export_magicube=export)
                if export:
                    magicube = open(os.path.join(d, "data", "magicube_cop20k_A.mtx"), "rb").read()
                # and the reference's alternative, gap-skipping blocking (csrToBcsrKnapsacking)
                knap = oracle.ref_sparse_matrix(path, host_only=True, knapsack=True)
            finally:
                os.chdir(cwd)
        np.savez_compressed(os.path.join(HERE, f"reader_{name}.npz"), mtx=np.frombuffer(text.encode(), np.uint8), M=M, K=K,
                            magicube=np.frombuffer(magicube, np.uint8), knap_rowptr=knap[5], knap_colidx=knap[6],
                            knap_vals=knap[7],
                            csr_rowptr=crp, csr_colidx=cci, csr_vals=cv, bcsr_rowptr=brp, bcsr_colidx=bci, bcsr_vals=bv)
        print("reader", name, M, K, "nnz", len(cci), "nnzb", len(bci))


def formats_fixtures():
    """Runs the reference's own Python glue (src/reorder.py, imported from the reference tree) and its
    Matrix_Blocking program on a small pattern matrix: text converters, row pass, column pass."""
    import shutil
    import types
    ref_src = os.path.join(os.environ["SMAT_REFERENCE"], "src")  # root of the reference tree
    sys.modules.setdefault("utils", types.ModuleType("utils"))  # plotting helpers, not needed (matplotlib absent)
    sys.path.insert(0, ref_src)
    import reorder as ref_reorder  # the reference module
    out = os.path.join(HERE, "formats")
    os.makedirs(out, exist_ok=True)
    rng = np.random.default_rng(9)
    n = 96
    keys = np.unique(np.concatenate([rng.integers(0, n * n, 500), [(n - 1) * n + n - 1]]))
    rng.shuffle(keys)
    with open(os.path.join(out, "in.mtx"), "w") as f:
        f.write(f"%%MatrixMarket matrix coordinate pattern general\n% fixture\n{n} {n} {len(keys)}\n")
        f.write("\n".join(f"{k // n + 1} {k % n + 1}" for k in keys.tolist()))
    with tempfile.TemporaryDirectory() as d:
        shutil.copy(os.path.join(out, "in.mtx"), os.path.join(d, "m.mtx"))
        os.makedirs(os.path.join(d, "programs", "general"))
        shutil.copy(os.path.join(REFDIR, "Matrix_Blocking"), os.path.join(d, "programs", "general", "Matrix_Blocking"))
        os.makedirs(os.path.join(d, "results"))
        cwd = os.getcwd()
        os.chdir(d)  # Matrix_Blocking writes its default outfile under ./results
        try:
            ref_reorder.mtx2el(os.path.join(d, "m.mtx"), os.path.join(d, "m.el"))
            shutil.copy(os.path.join(d, "m.el"), os.path.join(out, "ref.el"))
            ref_reorder.el2mtx(os.path.join(d, "m.el"), os.path.join(d, "back.mtx"))
            shutil.copy(os.path.join(d, "back.mtx"), os.path.join(out, "ref_back.mtx"))
            ref_reorder.reorder_using_paolo(os.path.join(d, "m.mtx"), d, 16, 16)
            shutil.copy(os.path.join(d, "m_reordered.el"), os.path.join(out, "ref_reordered.el"))
            shutil.copy(os.path.join(d, "m_reordered.mtx"), os.path.join(out, "ref_reordered.mtx"))
            ref_reorder.reorder_cols_using_paolo(os.path.join(d, "m_reordered.el"), d, 16, 16)
            shutil.copy(os.path.join(d, "m_reordered_transposed.el"), os.path.join(out, "ref_reordered_transposed.el"))
            shutil.copy(os.path.join(d, "m_reordered_transposed_reordered.el"),
                        os.path.join(out, "ref_reordered_transposed_reordered.el"))
        finally:
            os.chdir(cwd)
    # the reference's band-matrix generator (src/generate_matrices.py:5-35), imported from the reference tree
    import importlib.util
    spec = importlib.util.spec_from_file_location("ref_generate_matrices", os.path.join(ref_src, "generate_matrices.py"))
    ref_gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref_gen)
    with tempfile.TemporaryDirectory() as d:
        ref_gen.generate_band_mtx_matrix(37, 5, d, "band.mtx")
        shutil.copy(os.path.join(d, "band.mtx"), os.path.join(out, "ref_band_37_5.mtx"))
    print("formats fixtures:", sorted(os.listdir(out)))


def vbr_cases():
    """(name, M, K, rowptr, colidx, vals fp16, grouping, col_block): groupings of unequal groups, negative group
    numbers as the clustering writes them for full groups, empty rows, a last block-column that sticks out of K."""
    cases = []
    for name, M, K, density, n_groups, cb, seed in [("small", 23, 40, 0.2, 6, 4, 1), ("ragged", 64, 100, 0.08, 11, 16, 2),
                                                    ("tall", 96, 48, 0.1, 3, 8, 3), ("singletons", 17, 33, 0.3, 17, 5, 4)]:
        rng = np.random.default_rng(seed)
        mask = rng.random((M, K)) < density
        mask[M // 2] = False  # an empty row
        vals = (rng.standard_normal((M, K)) * mask).astype(np.float16)
        mask = vals != 0
        rowptr = np.zeros(M + 1, np.int32)
        rowptr[1:] = np.cumsum(mask.sum(axis=1))
        g = rng.integers(0, n_groups, M).astype(np.int64) if n_groups < M else rng.permutation(M).astype(np.int64)
        full = rng.random(M) < 0.3
        g = np.where(full & (g != M - 1), g - M, g)  # "full group" marks of the clustering (never -1)
        cases.append((name, M, K, rowptr, np.nonzero(mask)[1].astype(np.int32), vals[mask], g, cb))
    return cases


def vbr_fixtures():
    """Outputs of the unmodified VBR::fill_from_CSR_inplace(cmat, grouping, col_block) for vbr_cases()."""
    for name, M, K, rowptr, colidx, vals, g, cb in vbr_cases():
        v = oracle.ref_vbr_from_grouping(M, K, rowptr, colidx, vals, g, cb)
        np.savez_compressed(os.path.join(HERE, f"vbr_{name}.npz"), M=M, K=K, rowptr=rowptr, colidx=colidx,
                            vals=vals.view(np.uint16), grouping=g, col_block=cb, row_part=v["row_part"], row_perm=v["row_perm"],
                            nzcount=v["nzcount"], jab=v["jab"], mab=v["mab"].astype(np.float16).view(np.uint16))
        print("vbr", name, "block-rows", len(v["nzcount"]), "blocks", len(v["jab"]))


if __name__ == "__main__":
    assert oracle.have_ref(), "build oracle/_ref first: make -C oracle ref REF=<reference tree>"
    similarities()
    reorder_fixtures()
    multiply_fixtures()
    reader_fixtures()
    formats_fixtures()
    vbr_fixtures()
