"""Parity of the CUDA SpMM (through the C ABI) with the CPU oracle and the reference-generated
fixtures.  Tolerance: max relative error 1e-2 (fp16 in, fp32 accumulate, fp16 out), where the error of
an entry is measured against max(|c_ref|, 1e-2 * sum_k |a||b|) so that entries dominated by
cancellation are judged against the magnitude of the terms that were summed."""
import os

import numpy as np
import pytest

import oracle
import smat_b200 as S
from smat_b200 import generators as gen

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _torch():
    import torch
    return torch


def _oracle_c(bv, brp, bci, B_nk, M, N, K, rows=None):
    b0, b1 = (0, M // 16) if rows is None else rows
    C = oracle.bcsr_spmm(bv, brp, bci, B_nk, M, N, K, b0, b1, threads=8)
    Cabs = oracle.bcsr_spmm(np.abs(bv), brp, bci, np.abs(B_nk), M, N, K, b0, b1, threads=8)
    return C, Cabs


def _rel_err(C_gpu, C_ref, C_abs):
    c = C_gpu.astype(np.float32)
    ref16 = C_ref.astype(np.float16).astype(np.float32)
    denom = np.maximum(np.abs(ref16), 1e-2 * C_abs) + 1e-30
    return float(np.max(np.abs(c - ref16) / denom))


def _close(a, b):
    """Equal up to the rounding of differently grouped fp32 partial sums to fp16."""
    a = a.astype(np.float32)
    b = b.astype(np.float32)
    return bool(np.all(np.abs(a - b) <= 2.0 ** -9 * np.maximum(np.abs(a), np.abs(b)) + 1e-3 * max(1e-6, float(np.abs(a).max()))))


def _run(brp, bci, bv, B_nk, M, N, K, variant="call"):
    torch = _torch()
    A = S.SparseMatrix.from_bcsr(M, K, brp, bci, bv)
    B = S.Matrix.from_host(B_nk)
    C = S.Matrix(M, N, fill=float("nan"))
    kernel = {"smem": 1, "tmem": 2, "wide": 3, "tall": 4}.get(variant, 0)  # force one kernel variant, else automatic choice
    S.set_variant(kernel)
    try:
        if variant == "call":
            S.spmm(A, B, C, check=True)
        else:
            plan = S.Plan(A)
            plan.spmm(B, C, check=True)
            plan.close()
    finally:
        S.set_variant(0)
    torch.cuda.synchronize()
    return C.data.cpu().numpy()


def _problem(name, scale, N=None):
    p = gen.make_config(name, scale=scale)
    if N is not None and N != p.N:  # same A, a B with the requested number of columns
        p["B_nk"] = np.random.default_rng(99).standard_normal((N, p.K)).astype(np.float16)
        p["N"] = N
    brp, bci, bv = oracle.csr_to_bcsr(p.M, p.K, p.rowptr, p.colidx, p.vals)
    return p, brp, bci, bv


@pytest.mark.parametrize("variant", ["call", "plan", "smem", "tmem", "wide", "tall"])
@pytest.mark.parametrize("name,scale,N", [("band", 1.0, 64), ("band", 0.1, 8), ("uniform", 0.02, 256),
                                          ("uniform", 0.01, 136), ("powerlaw", 0.01, 128), ("clustered", 0.004, 512),
                                          ("llm", 0.0625, 256), ("llm", 0.04, 24)])
def test_matches_oracle(name, scale, N, variant):
    p, brp, bci, bv = _problem(name, scale, N)
    C = _run(brp, bci, bv, p.B_nk, p.M, N, p.K, variant)
    Cref, Cabs = _oracle_c(bv, brp, bci, p.B_nk, p.M, N, p.K)
    assert not np.isnan(C.astype(np.float32)).any()
    assert _rel_err(C, Cref, Cabs) <= TOL


@pytest.mark.parametrize("name", ["band", "uniform", "llm"])
def test_matches_reference_vbr_multiply_fixture(golden_dir, name):
    """C of the reference's own CPU blocked multiply (VBR::multiply) on the same inputs."""
    z = np.load(os.path.join(golden_dir, f"multiply_{name}.npz"))
    M, K, N = int(z["M"]), int(z["K"]), int(z["N"])
    C = _run(z["bcsr_rowptr"], z["bcsr_colidx"], z["bcsr_vals"], z["B_nk"], M, N, K)
    Cabs = oracle.bcsr_spmm(np.abs(z["bcsr_vals"]), z["bcsr_rowptr"], z["bcsr_colidx"], np.abs(z["B_nk"]), M, N, K)
    assert _rel_err(C, z["C_f32"], Cabs) <= TOL


def test_reordered_matrix_matches_oracle():
    """Config-2 pipeline at reduced size: reorder rows (values carried), block, multiply."""
    p = gen.make_config("uniform", scale=0.03)
    _, perm = S.reorder_rows(p.rowptr, p.colidx)
    rp, ci, v = S.apply_row_permutation(p.rowptr, p.colidx, p.vals, perm)
    brp, bci, bv = oracle.csr_to_bcsr(p.M, p.K, rp, ci, v)
    C = _run(brp, bci, bv, p.B_nk, p.M, p.N, p.K)
    Cref, Cabs = _oracle_c(bv, brp, bci, p.B_nk, p.M, p.N, p.K)
    assert _rel_err(C, Cref, Cabs) <= TOL
    # a row reorder only permutes the rows of C
    brp0, bci0, bv0 = oracle.csr_to_bcsr(p.M, p.K, p.rowptr, p.colidx, p.vals)
    C0 = _run(brp0, bci0, bv0, p.B_nk, p.M, p.N, p.K)
    # (up to the rounding of differently grouped fp32 partial sums: an item of the last round may be cut at other steps)
    assert _close(C, C0[perm])


def test_edge_cases():
    rng = np.random.default_rng(0)
    # empty matrix: C is zero-filled
    M, K, N = 64, 48, 16
    C = _run(np.zeros(M // 16 + 1, np.int32), np.zeros(0, np.int32), np.zeros(0, np.float16),
             rng.standard_normal((N, K)).astype(np.float16), M, N, K)
    assert np.all(C == 0)
    # one block in the last block-row / last block-column; other block-rows empty -> zeros
    brp = np.array([0, 0, 0, 0, 1], np.int32)
    bci = np.array([32], np.int32)
    bv = rng.standard_normal(256).astype(np.float16)
    B = rng.standard_normal((N, K)).astype(np.float16)
    C = _run(brp, bci, bv, B, M, N, K)
    Cref, Cabs = _oracle_c(bv, brp, bci, B, M, N, K)
    assert np.all(C[:48] == 0) and _rel_err(C, Cref, Cabs) <= TOL
    # a single block-row (M = 16) with every block present, N = 8
    M, K, N = 16, 160, 8
    brp = np.array([0, 10], np.int32)
    bci = (np.arange(10) * 16).astype(np.int32)
    bv = rng.standard_normal(2560).astype(np.float16)
    B = rng.standard_normal((N, K)).astype(np.float16)
    C = _run(brp, bci, bv, B, M, N, K)
    Cref, Cabs = _oracle_c(bv, brp, bci, B, M, N, K)
    assert _rel_err(C, Cref, Cabs) <= TOL


def test_ragged_rows_and_long_block_row():
    """Block-rows with 0, 1 and hundreds of blocks side by side (load imbalance, as in a power-law matrix)."""
    rng = np.random.default_rng(4)
    Mb, Kb, N = 40, 600, 72
    counts = rng.integers(0, 4, Mb)
    counts[7] = 600
    counts[8] = 0
    counts[21] = 311
    brp = np.zeros(Mb + 1, np.int32)
    brp[1:] = np.cumsum(counts)
    bci = np.concatenate([np.sort(rng.choice(Kb, c, replace=False)) for c in counts]).astype(np.int32) * 16
    bv = rng.standard_normal(brp[-1] * 256).astype(np.float16)
    B = rng.standard_normal((N, Kb * 16)).astype(np.float16)
    for variant in ("call", "smem", "tmem", "wide", "tall"):
        C = _run(brp, bci, bv, B, Mb * 16, N, Kb * 16, variant)
        Cref, Cabs = _oracle_c(bv, brp, bci, B, Mb * 16, N, Kb * 16)
        assert _rel_err(C, Cref, Cabs) <= TOL


@pytest.mark.parametrize("variant", ["call", "smem", "tmem", "wide", "tall"])
@pytest.mark.parametrize("Mb,Kb,N,fill", [(3, 4096, 128, 0.5), (16, 2048, 264, 0.3), (40, 1024, 512, 0.15), (1, 9000, 8, 1.0)])
def test_items_cut_across_ctas(Mb, Kb, N, fill, variant):
    """Few block-rows, many block-columns: far fewer work items than SMs, so every item is computed in parts by
    many CTAs and assembled from fp32 partial tiles (including a three-row group and a lone block-row)."""
    rng = np.random.default_rng(Mb * 1000 + N)
    counts = np.maximum(1, rng.binomial(Kb, fill, Mb))
    brp = np.zeros(Mb + 1, np.int32)
    brp[1:] = np.cumsum(counts)
    bci = np.concatenate([np.sort(rng.choice(Kb, c, replace=False)) for c in counts]).astype(np.int32) * 16
    bv = (rng.standard_normal(brp[-1] * 256) * 0.1).astype(np.float16)
    B = rng.standard_normal((N, Kb * 16)).astype(np.float16)
    C = _run(brp, bci, bv, B, Mb * 16, N, Kb * 16, variant)
    Cref, Cabs = _oracle_c(bv, brp, bci, B, Mb * 16, N, Kb * 16)
    assert _rel_err(C, Cref, Cabs) <= TOL
    again = _run(brp, bci, bv, B, Mb * 16, N, Kb * 16, variant)
    assert np.array_equal(C.view(np.uint16), again.view(np.uint16))  # same cuts, same order of addition


@pytest.mark.parametrize("variant", ["plan", "smem", "tmem", "wide"])
def test_balanced_schedule_for_skewed_matrices(variant):
    """One group of block-rows holds a third of all steps (as the power-law configuration does after the reorder):
    such plans deal out equal ranges of the flattened (item, step) sequence, so range boundaries fall inside work
    items almost everywhere and C is assembled from partial tiles; two groups are empty (their rows must be zeroed)."""
    rng = np.random.default_rng(11)
    Mb, Kb, N = 1024, 2048, 264
    counts = rng.integers(1, 4, Mb)
    counts[160:176] = rng.integers(900, 1100, 16)  # the heavy group
    counts[80:112] = 0                             # two empty groups
    brp = np.zeros(Mb + 1, np.int32)
    brp[1:] = np.cumsum(counts)
    bci = np.concatenate([np.sort(rng.choice(Kb, c, replace=False)) for c in counts]).astype(np.int32) * 16
    bv = (rng.standard_normal(brp[-1] * 256) * 0.1).astype(np.float16)
    B = rng.standard_normal((N, Kb * 16)).astype(np.float16)
    C = _run(brp, bci, bv, B, Mb * 16, N, Kb * 16, variant)
    Cref, Cabs = _oracle_c(bv, brp, bci, B, Mb * 16, N, Kb * 16)
    assert np.all(C[80 * 16:112 * 16] == 0)
    assert _rel_err(C, Cref, Cabs) <= TOL
    again = _run(brp, bci, bv, B, Mb * 16, N, Kb * 16, variant)
    assert np.array_equal(C.view(np.uint16), again.view(np.uint16))


def test_listed_schedule_for_skewed_matrices():
    """Many groups, twenty of them eight times heavier than the rest: the plan deals whole groups out to the CTAs
    heaviest first (a fixed list per CTA) instead of round-robin; some groups are empty."""
    rng = np.random.default_rng(12)
    Mb, Kb, N = 16384, 1024, 72
    counts = rng.integers(1, 4, Mb)
    for g in rng.choice(Mb // 16, 20, replace=False):
        counts[g * 16:(g + 1) * 16] = rng.integers(90, 110, 16)
    counts[4000 * 1:4000 + 64] = 0
    brp = np.zeros(Mb + 1, np.int32)
    brp[1:] = np.cumsum(counts)
    bci = np.concatenate([np.sort(rng.choice(Kb, c, replace=False)) for c in counts]).astype(np.int32) * 16
    bv = (rng.standard_normal(brp[-1] * 256) * 0.1).astype(np.float16)
    B = rng.standard_normal((N, Kb * 16)).astype(np.float16)
    C = _run(brp, bci, bv, B, Mb * 16, N, Kb * 16, "plan")
    Cref, Cabs = _oracle_c(bv, brp, bci, B, Mb * 16, N, Kb * 16)
    assert np.all(C[4000 * 16:4064 * 16] == 0)
    assert _rel_err(C, Cref, Cabs) <= TOL
    # whole items only: bit-identical to the round-robin launch of the call entry point
    C2 = _run(brp, bci, bv, B, Mb * 16, N, Kb * 16, "smem")
    assert np.array_equal(C.view(np.uint16), C2.view(np.uint16))


def test_block_row_range_entry_point():
    torch = _torch()
    p, brp, bci, bv = _problem("powerlaw", 0.01, 64)
    A = S.SparseMatrix.from_bcsr(p.M, p.K, brp, bci, bv)
    B = S.Matrix.from_host(p.B_nk)
    full = S.Matrix(p.M, 64)
    S.spmm(A, B, full, check=True)
    bounds = S.partition_block_rows(brp, 4)
    for g in range(4):
        b0, b1 = int(bounds[g]), int(bounds[g + 1])
        shard = torch.full(((b1 - b0) * 16, 64), float("nan"), dtype=torch.float16, device="cuda")
        S.spmm_rows(A, B, shard, b0, b1, check=True)
        # a shard cuts its work items at other places than the full launch, so fp32 partial sums may be grouped
        # differently before the one rounding to fp16: equal up to that rounding, not bit for bit
        assert _close(shard.cpu().numpy(), full.data[b0 * 16:b1 * 16].cpu().numpy())


@pytest.mark.parametrize("kernel", ["auto", "tall"])
@pytest.mark.parametrize("ranges", ["", "3"])
@pytest.mark.parametrize("N", [64, 264, 1024])
def test_host_buffer_entry_point(N, ranges, kernel, monkeypatch):
    """smat_plan_spmm_host: B and C in pinned host memory, copies pipelined in column chunks (1, 3 and 4 chunks
    here, the 264-column case with a ragged last chunk), called twice to cover the reuse of its staging; the last
    chunk multiplied and copied out in one range of block-rows (the automatic choice at this size) and in three."""
    torch = _torch()
    if ranges:
        monkeypatch.setenv("SMAT_HOST_RANGES", ranges)
    p, brp, bci, bv = _problem("uniform", 0.03, N)
    A = S.SparseMatrix.from_bcsr(p.M, p.K, brp, bci, bv)
    S.set_variant(4 if kernel == "tall" else 0)  # a tall plan (24-row work items) takes the same chunks and row ranges
    try:
        plan = S.Plan(A, n_hint=N)
    finally:
        S.set_variant(0)
    assert plan.info()["tall"] == (kernel == "tall")
    B_host = torch.from_numpy(p.B_nk.view(np.int16)).pin_memory()
    C_host = torch.full((p.M, N), -1, dtype=torch.int16).pin_memory()
    Cref, Cabs = _oracle_c(bv, brp, bci, p.B_nk, p.M, N, p.K)
    for _ in range(2):
        C_host.fill_(-1)
        plan.spmm_host(B_host, C_host)
        torch.cuda.synchronize()
        S.api._check(S.lib().smat_device_status(None))
        assert _rel_err(C_host.numpy().view(np.float16), Cref, Cabs) <= TOL
    plan.close()


def test_deterministic():
    p, brp, bci, bv = _problem("llm", 0.0625, 256)
    a = _run(brp, bci, bv, p.B_nk, p.M, 256, p.K)
    b = _run(brp, bci, bv, p.B_nk, p.M, 256, p.K)
    assert np.array_equal(a.view(np.uint16), b.view(np.uint16))


def test_tester_harness_reports_throughput():
    p, brp, bci, bv = _problem("band", 1.0, 64)
    A = S.SparseMatrix.from_bcsr(p.M, p.K, brp, bci, bv)
    t = S.Tester(A, 64, warmup_iterations=1, profiling_iterations=3)
    ms, tflops = t.evaluateSparse2()
    assert ms > 0 and tflops > 0
    # B is all ones in the reference harness (matrix.h:38): every C entry is a row sum of A
    want = np.zeros(p.M, np.float32)
    np.add.at(want, np.repeat(np.arange(p.M), np.diff(p.rowptr)), p.vals.astype(np.float32))
    got = t.C.data[:, 0].float().cpu().numpy()
    assert np.max(np.abs(got - want)) <= 1e-2 * np.maximum(np.abs(want), 1).max()


@pytest.mark.parametrize("name", ["llm", "clustered", "uniform", "powerlaw"])
def test_full_size_sampled_block_rows(name):
    """The benchmark's matrices at full size, prepared the way bench.py prepares them (similarity reorder from the
    permutation cache where the configuration asks for one, device-side blocking, a plan): sampled block-rows of the
    GPU result against the oracle -- the first, the last, the one with the most blocks, one of the group with the most
    blocks, and random ones -- plus the size-independent property that block-rows without blocks are exactly zero.
    These sizes select code paths the small cases do not: 256-column work items over several rounds (uniform), the
    listed schedule with thousands of steps per CTA (power-law), steps of 32 blocks (clustered)."""
    from smat_b200 import formats
    torch = _torch()
    p = gen.make_config(name)
    rp, ci, v = p.rowptr, p.colidx, p.vals
    if p.reorder:
        seed = {"uniform": 1, "powerlaw": 2}[name]
        perm, _, _ = formats.cached_permutation(formats.cache_key(name, seed, 1.0, 0.5, 16), rp, ci)
        rp, ci, v = S.apply_row_permutation(rp, ci, v, perm)
    A = S.SparseMatrix.from_csr(p.M, p.K, rp, ci, v)
    B = S.Matrix.from_host(p.B_nk)
    C = S.Matrix(p.M, p.N, fill=float("nan"))
    plan = S.Plan(A, n_hint=p.N)
    plan.spmm(B, C, check=True)
    plan.close()
    brp, bci, bv = A.host_arrays()
    Mb = p.M // 16
    rng = np.random.default_rng(0)
    counts = np.diff(brp)
    heaviest = int(np.argmax(counts))
    per_group = np.add.reduceat(counts, np.arange(0, Mb, 16))
    in_heaviest_group = int(np.argmax(per_group)) * 16 + 7
    picks = sorted(set([0, Mb - 1, heaviest, min(in_heaviest_group, Mb - 1)] + rng.integers(0, Mb, 6).tolist()))
    for br in picks:
        Cref, Cabs = _oracle_c(bv, brp, bci, p.B_nk, p.M, p.N, p.K, rows=(br, br + 1))
        got = C.data[br * 16:br * 16 + 16].cpu().numpy()
        assert _rel_err(got, Cref, Cabs) <= TOL, br
    empty = np.nonzero(counts == 0)[0]
    for br in empty[:4]:
        assert torch.all(C.data[br * 16:br * 16 + 16] == 0)
    assert not torch.isnan(C.data).any()


def test_tall_plan_dense_and_odd_shapes():
    """The tall kernel (24-row work items, panels read from tensor memory) on shapes that exercise its plan: quads
    with more blocks than a step holds (dense block-rows: steps are cut and the panel is fetched again), a group
    height that does not divide the matrix, an odd number of steps per CTA, N below and beyond one tile."""
    rng = np.random.default_rng(21)
    for Mb, Kb, N, fill in [(50, 96, 200, 1.0), (24, 333, 136, 0.6), (7, 5, 8, 1.0), (100, 64, 520, 0.2)]:
        mask = rng.random((Mb, Kb)) < fill
        mask[:, 0] |= ~mask.any(axis=1)
        counts = mask.sum(axis=1)
        brp = np.zeros(Mb + 1, np.int32)
        brp[1:] = np.cumsum(counts)
        bci = (np.nonzero(mask)[1] * 16).astype(np.int32)
        bv = (rng.standard_normal(brp[-1] * 256) * 0.25).astype(np.float16)
        B = rng.standard_normal((N, Kb * 16)).astype(np.float16)
        C = _run(brp, bci, bv, B, Mb * 16, N, Kb * 16, "tall")
        Cref, Cabs = _oracle_c(bv, brp, bci, B, Mb * 16, N, Kb * 16)
        assert _rel_err(C, Cref, Cabs) <= TOL
        again = _run(brp, bci, bv, B, Mb * 16, N, Kb * 16, "tall")
        assert np.array_equal(C.view(np.uint16), again.view(np.uint16))


def test_plan_chooses_tall_kernel_for_block_sparse_layer():
    """Plan creation counts the steps of both walk orders and takes the 24-row one where its estimate wins: a
    block-sparse layer with a fifth of its blocks kept and enough work to fill the device does, the same matrix with a
    forced 16-row kernel does not; both give the oracle's result.  smat_plan_info reports the choice."""
    torch = _torch()
    rng = np.random.default_rng(33)
    Mb, Kb, N = 192, 512, 2048
    mask = rng.random((Mb, Kb)) < 0.2
    brp = np.zeros(Mb + 1, np.int32)
    brp[1:] = np.cumsum(mask.sum(axis=1))
    bci = (np.nonzero(mask)[1] * 16).astype(np.int32)
    bv = (rng.standard_normal(brp[-1] * 256) * 0.25).astype(np.float16)
    B_nk = rng.standard_normal((N, Kb * 16)).astype(np.float16)
    Cref, Cabs = _oracle_c(bv, brp, bci, B_nk, Mb * 16, N, Kb * 16)
    A = S.SparseMatrix.from_bcsr(Mb * 16, Kb * 16, brp, bci, bv)
    B = S.Matrix.from_host(B_nk)
    for variant, want_tall in ((0, True), (1, False)):
        S.set_variant(variant)
        try:
            plan = S.Plan(A, n_hint=N)
        finally:
            S.set_variant(0)
        info = plan.info()
        assert info["tall"] == want_tall, info
        assert (16 <= info["rows_per_item"] <= 24) if want_tall else (info["rows_per_item"] <= 16)
        assert info["steps"] > 0 and info["kernel"] == ("spmm_bcsr_tall_kernel" if want_tall else "spmm_bcsr_tc_kernel")
        C = S.Matrix(Mb * 16, N, fill=float("nan"))
        plan.spmm(B, C, check=True)
        torch.cuda.synchronize()
        assert _rel_err(C.data.cpu().numpy(), Cref, Cabs) <= TOL
        plan.close()


def test_bounded_wait_timeout_is_reported():
    """The error path of the kernels' bounded waits, driven from the host: a one-thread kernel waits on a barrier that
    nothing completes, gives up after ~0.2 ms and sets the device status word; smat_device_status reports
    SMAT_ERR_DEVICE_WAIT once, clears the word, and the context keeps working."""
    torch = _torch()
    L = S.lib()
    assert L.smat_device_status(None) == 0
    assert L.smat_selftest_wait_timeout(torch.cuda.current_stream().cuda_stream) == 0
    rc = L.smat_device_status(torch.cuda.current_stream().cuda_stream)
    assert rc == -3 and b"site code 90" in L.smat_last_error_string()
    assert L.smat_device_status(None) == 0
    p, brp, bci, bv = _problem("band", 0.1, 8)
    C = _run(brp, bci, bv, p.B_nk, p.M, 8, p.K)
    Cref, Cabs = _oracle_c(bv, brp, bci, p.B_nk, p.M, 8, p.K)
    assert _rel_err(C, Cref, Cabs) <= TOL


def test_inconsistent_row_pointers_are_reported_not_written_past():
    """nonzeroBlocks smaller than what the row pointers claim: the plan buffers are sized from nonzeroBlocks, so the
    plan kernels refuse the range (empty plan, status word) and smat_device_status returns SMAT_ERR_RANGE."""
    torch = _torch()
    p, brp, bci, bv = _problem("band", 0.1, 8)
    A = S.SparseMatrix.from_bcsr(p.M, p.K, brp, bci, bv)
    B = S.Matrix.from_host(p.B_nk)
    C = S.Matrix(p.M, 8, fill=0.0)
    L = S.lib()
    stream = torch.cuda.current_stream().cuda_stream
    for entry in ("plain", "static"):
        lie = A.nnzb - 5  # fewer blocks than bcsrRowPtr[M / 16]
        if entry == "plain":
            rc = L.smat_spmm_bcsr_f16(A.getBcsrValues(), A.getBcsrRowPtr(), A.getBcsrColIdx(), B.data.data_ptr(), C.data.data_ptr(),
                                      p.M, 8, p.K, lie, None, None, stream)
        else:
            rc = L.smat_spmm_bcsr_f16_static(A.getBcsrValues(), A.getBcsrRowPtr(), A.getBcsrColIdx(), B.data.data_ptr(),
                                             C.data.data_ptr(), p.M, 8, p.K, lie, stream)
        assert rc == 0
        rc = L.smat_device_status(stream)
        assert rc == -6 and b"bcsrRowPtr" in L.smat_last_error_string(), entry
        assert L.smat_device_status(stream) == 0


@pytest.mark.parametrize("name,scale", [("uniform", 0.03), ("powerlaw", 0.01)])
def test_row_and_column_reorder_keep_the_product(name, scale):
    """The reference's full preprocessing -- similarity reorder of the rows, then of the columns through the transpose
    (src/reorder.py:107-182) -- with values carried and the rows of B permuted to match:
    spmm(P A Q^T, Q B) must equal P spmm(A, B)."""
    p = gen.make_config(name, scale=scale)
    _, perm = S.reorder_rows(p.rowptr, p.colidx)
    rp, ci, v = S.apply_row_permutation(p.rowptr, p.colidx, p.vals, perm)
    _, cperm = S.reorder_cols(rp, ci, p.K)
    rp2, ci2, v2 = S.apply_col_permutation(rp, ci, v, cperm)
    B2 = S.permute_rows_of_B(p.B_nk, cperm)
    brp0, bci0, bv0 = oracle.csr_to_bcsr(p.M, p.K, p.rowptr, p.colidx, p.vals)
    brp2, bci2, bv2 = oracle.csr_to_bcsr(p.M, p.K, rp2, ci2, v2)
    C0 = _run(brp0, bci0, bv0, p.B_nk, p.M, p.N, p.K)
    C2 = _run(brp2, bci2, bv2, B2, p.M, p.N, p.K)
    Cref, Cabs = _oracle_c(bv2, brp2, bci2, B2, p.M, p.N, p.K)
    assert _rel_err(C2, Cref, Cabs) <= TOL
    # against the unpermuted product: the same sums in another order of addition
    d = np.abs(C2.astype(np.float32) - C0[perm].astype(np.float32))
    Cabs0 = oracle.bcsr_spmm(np.abs(bv0), brp0, bci0, np.abs(p.B_nk), p.M, p.N, p.K, 0, p.M // 16, threads=8)[perm]
    assert float(np.max(d / (np.maximum(np.abs(C0[perm].astype(np.float32)), 1e-2 * Cabs0) + 1e-30))) <= TOL
    assert len(bci2) <= len(bci0)  # the point of the exercise: fewer nonzero blocks
