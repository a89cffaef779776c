#!/usr/bin/env python
"""Benchmark of the block-sparse SpMM hot path:  C = A_blocked x B  on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config NAME] [--impl ours|reference]

One "step" is one multiplication of the whole matrix by a B that is resident in HBM.  Default workload: the
block-sparse weight layer ("llm": 8192 x 28672, 20 % of the 16x16 blocks kept, 4096 activation columns) -- the
workload both stated targets are defined on (fraction of the roofline at >= 20 % block fill; scaling over 1/2/4/8 GPUs).
Prints ONE JSON line.

  value      effective TFLOP/s = 2*16*16*N*nnzb / t with A (blocked + plan), B and C resident in HBM; t = median over
             --repeats timed regions of --steps launches each, maximum over ranks
  e2e        same metric through the library's host-buffer call: each step copies B host->device from pinned memory,
             multiplies, and copies C device->host (N > 1: every rank uploads 1/N of B, the slices are exchanged over
             NVLink with one NCCL all-gather)
  roofline   algorithmic bytes (or FLOPs) per launch / measured launch time, against the measured peak
  all_configs   (1 GPU) the same measurement, one region, for the other four configurations
  gpu_baselines (1 GPU) the reference's own kernels compiled unmodified for sm_100a, and cuSPARSE CSR SpMM, on the same
                GPU and matrix
  cpu_baseline  the reference's own CPU blocked multiply (VBR::multiply) on a bounded sample
  parity_max_rel_err  sampled block-rows of every measured C against the CPU oracle (the oracle is the checker only)
With --impl reference the reference's CPU blocked multiply is the thing timed (all host cores, each on its own
block-row range).  For N > 1 (torchrun) block-rows are partitioned by block count, B is replicated, C stays sharded, and
there is no collective in the timed region of `value`.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "SpMM effective TFLOP/s (nonzero-block FLOPs)"

# DRAM bytes (read + write) per launch of the SpMM kernel from an ncu capture of the same workload
# (see profiles/): filled per workload, None where no capture exists.
NCU_TRAFFIC_BYTES = {  # (config, scale, GPUs, kernel) -> bytes per launch
    # uniform: 117.86 MB (113.68 read + 4.17 written, mean of two launches) measured at scale 0.25 (nnzb 204859) with the 16-row
    # kernel, scaled by nnzb to the full-size matrix (3548444 blocks): every block is read once per launch and dominates the traffic
    ("uniform", 0.25, 1, "spmm_bcsr_tc_kernel"): int(117.86e6),
    # block-sparse layer, full size: dram__bytes_read.sum + dram__bytes_write.sum of the SpMM kernel, mean of three launches,
    # captured at full size (the two counters take one pass).  B (235 MB) does not fit L2 and is streamed from HBM once per
    # round of work items
    ("llm", 1.0, 1, "spmm_bcsr_tc_kernel"): 1102730000,   # 16-row kernel, 256-column items: 3.5 rounds
    ("llm", 1.0, 1, "spmm_bcsr_tall_kernel"): 1421549000,  # 24-row kernel (the default plan): 4.8 rounds
}
SEEDS = {"band": 0, "uniform": 1, "powerlaw": 2, "clustered": 3, "llm": 4}
ALL_CONFIGS = ["band", "uniform", "powerlaw", "clustered", "llm"]


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": float(p["hbm_gbs"]), "tflops": float(p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU every 200 ms while active."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self._stop, self._t = index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                f = [x.strip() for x in out.strip().split(",")]
                if len(f) >= 6:
                    self.samples.append(f)
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        mhz = [float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in self.samples for n, v in zip(names, s[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(mhz) if mhz else None,
                "sm_max_mhz": float(self.samples[0][1]) if self.samples[0][1].replace(".", "").isdigit() else None,
                "reasons": reasons, "samples": len(self.samples)}


def build_problem(name, scale, log):
    """Seeded synthetic matrix -> (problem, host CSR after the optional row reorder, reorder seconds)."""
    import smat_b200 as S
    from smat_b200 import generators as gen
    t = time.time()
    if name == "clustered_literal":  # the off-cluster density read literally: 0.001 % of n^2 positions
        p = gen.make_config("clustered", scale=scale, literal_offcluster=True)
    else:
        p = gen.make_config(name, scale=scale)
    log(f"generated {p.desc} in {time.time() - t:.1f}s")
    return p


def reorder_if_needed(p, log, perm=None, name=None, scale=1.0):
    """Row reorder of the configurations that ask for one.  The permutation comes from the on-disk cache when the file
    for (configuration, seed, scale, tau, block) exists and fits the matrix, else it is computed and stored."""
    import smat_b200 as S
    from smat_b200 import formats
    if not p.reorder:
        return p.rowptr, p.colidx, p.vals, 0.0, None
    secs, hit = 0.0, False
    if perm is None:
        key = formats.cache_key(name or p.name, SEEDS.get(name or p.name, -1), scale, 0.5, 16)
        perm, secs, hit = formats.cached_permutation(key, p.rowptr, p.colidx, tau=0.5, col_block=16, row_block=16, threads=0, log=log)
    rp, ci, v = S.apply_row_permutation(p.rowptr, p.colidx, p.vals, perm)
    log(f"row reorder (tau 0.5, 16x16, Keeper): " + ("from the cache" if hit else f"{secs:.1f}s"))
    return rp, ci, v, secs, perm


def algorithmic_bytes(bcsr_rowptr, bcsr_colidx, M, N):
    nnzb = int(bcsr_rowptr[-1])
    Mb = M // 16
    distinct_cols = int(np.unique(bcsr_colidx).size)
    return 512 * nnzb + 4 * nnzb + 4 * (Mb + 1) + 32 * N * distinct_cols + 2 * M * N


def cpu_reference_multiply(bvals, brp, bci, B_nk, M, K, N, brow_ranges, threads):
    """Runs the reference's VBR::multiply (oracle/_ref) -- or the oracle port when the reference
    library is absent -- on the given block-row ranges, one range per thread.  Returns (seconds, kind,
    number of blocks multiplied)."""
    import oracle
    R = oracle.ref() if oracle.have_ref() else None
    Bf = np.ascontiguousarray(B_nk.astype(np.float32)).reshape(-1)  # [n][k] == column-major K x N
    jobs = []
    for (b0, b1) in brow_ranges:
        p0, p1 = int(brp[b0]), int(brp[b1])
        nb = p1 - p0
        if R is not None:
            blocks = bvals[p0 * 256:p1 * 256].reshape(nb, 16, 16)
            mab = np.ascontiguousarray(blocks.transpose(0, 2, 1)).astype(np.float32).reshape(-1)  # column-major blocks
            jab = (bci[p0:p1] // 16).astype(np.int64)
            nzc = np.diff(brp[b0:b1 + 1]).astype(np.int64)
            Cf = np.zeros((b1 - b0) * 16 * N, np.float32)
            jobs.append((b0, b1, nb, mab if nb else np.zeros(1, np.float32), jab if nb else np.zeros(1, np.int64), nzc, Cf))
        else:
            jobs.append((b0, b1, nb))
    done = []

    def work(job):
        if R is not None:
            b0, b1, nb, mab, jab, nzc, Cf = job
            R.ref_vbr_multiply((b1 - b0) * 16, K, b1 - b0, 16, nzc, jab, mab, nb, 16, Bf, N, Cf)
        else:
            b0, b1, nb = job
            oracle.bcsr_spmm(bvals, brp, bci, B_nk, M, N, K, b0, b1, threads=1)
        done.append(job[2])

    t = time.time()
    ths = [threading.Thread(target=work, args=(j,)) for j in jobs[:threads]]
    for th in ths:
        th.start()
    for th in ths:
        th.join()
    return time.time() - t, ("reference" if R is not None else "port"), sum(done)


def gpu_baselines(A, B, p, N, log):
    """Informational: the reference's kernels (unmodified, compiled for sm_100a) and cuSPARSE CSR SpMM on
    the same GPU and matrix.  mmaCBT is timing-only (its B slab copy is the intended tile only for K = 16)."""
    import torch
    import oracle
    G = oracle.ref_gpu()
    if G is None:
        return {"unavailable": "oracle/_ref/libsmat_ref_gpu.so not built"}
    Mb, Kb = p.M // 16, p.K // 16
    flops = 2.0 * 256.0 * N * A.nnzb
    res = {}
    if Mb * Kb <= 600_000_000:
        rows = torch.repeat_interleave(torch.arange(Mb, device="cuda"), (A.bcsrRowPtr[1:] - A.bcsrRowPtr[:-1]).long())
        rel = torch.full((Mb * Kb,), -1, dtype=torch.int32, device="cuda")  # relativeBlockIndexMapping, matrix.h:425-431
        rel[rows * Kb + (A.bcsrColIdx[: A.nnzb] // 16).long()] = torch.arange(A.nnzb, dtype=torch.int32, device="cuda")
        Cref = torch.empty((p.M, N), dtype=torch.float16, device="cuda")
        for which, name in ((0, "ref_mmaCBT"), (1, "ref_mmaBT")):
            ms = G.ref_gpu_launch(which, A.getBcsrValues(), A.getBcsrRowPtr(), A.getBcsrColIdx(), B.data.data_ptr(),
                                  Cref.data_ptr(), p.M, N, p.K, A.nnzb, rel.data_ptr(), rel.data_ptr(), 1, 3)
            res[name] = {"ms": round(float(ms), 4), "tflops": round(flops / (ms * 1e-3) * 1e-12, 2) if ms > 0 else None}
            log(f"{name} on this GPU: {ms:.3f} ms")
        del rel, Cref
    else:
        res["ref_mmaCBT"] = {"unavailable": "dense Mb*Kb map beyond 2.4 GB"}
    Cc = torch.empty((p.M, N), dtype=torch.float16, device="cuda")
    ms = G.cusparse_csr_spmm_f16(A.csrRowPtr.data_ptr(), A.csrColIdx.data_ptr(), A.csrVal.data_ptr(), A.nnz,
                                 B.data.data_ptr(), Cc.data_ptr(), p.M, N, p.K, 1, 5)
    res["cusparse_csr"] = {"ms": round(float(ms), 4), "tflops": round(flops / (ms * 1e-3) * 1e-12, 2) if ms > 0 else None,
                           "note": "fp16 in, fp32 compute, ALG_DEFAULT; throughput quoted in the same nonzero-block FLOPs"}
    log(f"cuSPARSE CSR SpMM on this GPU: {ms:.3f} ms")
    return res


def sample_ranges(brp, Mb, target_blocks, parts):
    """`parts` disjoint contiguous block-row ranges from the start of the matrix, about target_blocks each."""
    out, b0 = [], 0
    for _ in range(parts):
        b1 = b0
        while b1 < Mb and brp[b1] - brp[b0] < target_blocks:
            b1 += 1
        if b1 == b0:
            break
        out.append((b0, b1))
        b0 = b1
        if b0 >= Mb:
            break
    return out


def parity_check(C_rows, b0, brp_h, bci_h, bv_h, B_nk, M, N, K, n_samples=4):
    """Outside every timed region: `n_samples` block-rows of this rank's C (the heaviest one among them) against the CPU
    oracle, with the error measure of the test-suite: |c - ref| / max(|ref|, 1e-2 * sum |a||b|).  C_rows maps a
    block-row of the shard to its 16 x N fp16 rows (numpy)."""
    import oracle
    b1 = b0 + C_rows.n_brows
    if b1 <= b0:
        return 0.0
    counts = np.diff(brp_h[b0:b1 + 1])
    picks = sorted({b0 + int(np.argmax(counts)), b0, b1 - 1, b0 + (b1 - b0) // 2, b0 + (b1 - b0) // 3}, key=lambda x: x)[:max(1, n_samples + 1)]
    worst = 0.0
    for br in picks:
        ref = oracle.bcsr_spmm(bv_h, brp_h, bci_h, B_nk, M, N, K, br, br + 1)
        mag = oracle.bcsr_spmm(np.abs(bv_h), brp_h, bci_h, np.abs(B_nk), M, N, K, br, br + 1)
        ref16 = ref.astype(np.float16).astype(np.float32)
        got = C_rows(br - b0).astype(np.float32)
        worst = max(worst, float(np.max(np.abs(got - ref16) / (np.maximum(np.abs(ref16), 1e-2 * mag) + 1e-30))))
    return worst


class _Rows:
    """Block-rows of a C held as a torch tensor (device or pinned host) for parity_check."""

    def __init__(self, C):
        self.C, self.n_brows = C, C.shape[0] // 16

    def __call__(self, i):
        return self.C[i * 16:(i + 1) * 16].cpu().numpy().view(np.float16)


def roofline_of(peaks, bytes_alg, flops, kernel_ms, traffic, kernel):
    t_hbm = bytes_alg / (peaks["hbm_gbs"] * 1e9)
    t_tensor = flops / (peaks["tflops"] * 1e12)
    secs = kernel_ms * 1e-3
    if t_hbm >= t_tensor:
        ach = bytes_alg / secs / 1e9
        roof = {"bound": "hbm", "achieved": round(ach, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(ach / peaks["hbm_gbs"], 4), "traffic": traffic}
    else:
        ach = flops / secs / 1e12
        roof = {"bound": "tensor", "achieved": round(ach, 1), "peak": peaks["tflops"], "unit": "TFLOP/s",
                "frac": round(ach / peaks["tflops"], 4), "traffic": traffic}
    roof.update({"peak_source": peaks["source"], "algorithmic_bytes": int(bytes_alg), "flops": flops,
                 "t_hbm_ms": round(t_hbm * 1e3, 4), "t_tensor_ms": round(t_tensor * 1e3, 4),
                 "kernel": kernel, "kernel_ms": round(kernel_ms, 4)})
    return roof


def prepare(name, scale, rank, world, dist, log, keep_csr=False):
    """Generates a configuration, reorders it if it asks for that, builds the blocked matrix on the device, the block-row
    range of this rank and its plan.  Returns a dict of everything the measurements need."""
    import torch
    import smat_b200 as S
    p = build_problem(name, scale, log)
    perm = None
    if p.reorder and world > 1:  # rank 0 obtains the permutation; the others receive it
        t = torch.empty(p.M, dtype=torch.int64, device="cuda")
        if rank == 0:
            _, _, _, _, perm0 = reorder_if_needed(p, log, None, name, scale)
            t.copy_(torch.from_numpy(np.asarray(perm0, dtype=np.int64)))
        dist.broadcast(t, 0)
        perm = t.cpu().numpy()
    rp, ci, v, reorder_s, perm = reorder_if_needed(p, log, perm, name, scale)
    t0 = time.time()
    A = S.SparseMatrix.from_csr(p.M, p.K, rp, ci, v, keep_csr=keep_csr)
    build_s = time.time() - t0
    brp_h, bci_h, bv_h = A.host_arrays()
    bounds = S.partition_block_rows(brp_h, world)
    b0, b1 = int(bounds[rank]), int(bounds[rank + 1])
    t0 = time.time()
    plan = S.Plan(A, b0, b1, n_hint=p.N)
    torch.cuda.synchronize()
    plan_s = time.time() - t0
    log(f"{name}: M={p.M} K={p.K} N={p.N} nnzb={A.nnzb} (device BCSR build {build_s:.2f}s, plan {plan_s:.2f}s); "
        f"rank {rank}: block-rows [{b0},{b1}) = {int(brp_h[b1] - brp_h[b0])} blocks")
    B = S.Matrix.from_host(p.B_nk)
    Cd = torch.empty(((b1 - b0) * 16, p.N), dtype=torch.float16, device="cuda")
    return {"p": p, "A": A, "plan": plan, "B": B, "Cd": Cd, "b0": b0, "b1": b1, "bounds": bounds, "host": (brp_h, bci_h, bv_h),
            "nnz": len(ci), "setup_s": {"reorder": round(reorder_s, 2), "bcsr_build": round(build_s, 3), "plan": round(plan_s, 3)}}


def time_regions(ctx, steps, warmup, repeats, barrier, sampler=None):
    """`warmup` untimed launches, then `repeats` regions of `steps` launches, each between two CUDA events on the launch
    stream with a barrier + synchronize on both sides.  Returns the per-step milliseconds of every region (this rank)."""
    import torch
    import smat_b200 as S
    plan, B, Cd = ctx["plan"], ctx["B"], ctx["Cd"]
    for _ in range(warmup):
        plan.spmm(B, Cd)
    S.api._check(S.lib().smat_device_status(None))
    out = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(repeats):
        barrier()
        e0.record()
        for _ in range(steps):
            plan.spmm(B, Cd)
        e1.record()
        barrier()
        out.append(e0.elapsed_time(e1) / steps)
    S.api._check(S.lib().smat_device_status(None))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of --steps launches; the median is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="llm", choices=ALL_CONFIGS)
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--cpu-sample-seconds", type=float, default=15.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gpu-baselines", action="store_true",
                    help="skip the reference's own kernels (compiled for sm_100a) and cuSPARSE CSR SpMM on this GPU")
    ap.add_argument("--variant", type=int, default=0, choices=[0, 1, 2, 3, 4],
                    help="kernel variant for every plan of this run (smat_spmm_set_variant; 0 = chosen per matrix)")
    ap.add_argument("--no-all-configs", action="store_true", help="skip the one-region measurement of the other configurations")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    def log(msg):
        if rank == 0:
            print(f"[bench] {msg}", file=sys.stderr, flush=True)

    if args.impl == "reference":
        return run_reference_arm(args, rank, world, log)

    import torch
    import smat_b200 as S

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    S.set_variant(args.variant)
    want_gpu_baselines = world == 1 and not args.no_gpu_baselines
    ctx = prepare(args.config, args.scale, rank, world, dist, log, keep_csr=want_gpu_baselines)
    p, A, plan, B, Cd, b0, b1 = ctx["p"], ctx["A"], ctx["plan"], ctx["B"], ctx["Cd"], ctx["b0"], ctx["b1"]
    brp_h, bci_h, bv_h = ctx["host"]
    N, Mb = p.N, p.M // 16
    my_blocks = int(brp_h[b1] - brp_h[b0])
    flops_total = 2.0 * 256.0 * N * A.nnzb

    # ---------------- resident timing ----------------
    launches0 = S.launch_count()
    with ClockSampler(local_rank) as clocks:
        regions = time_regions(ctx, args.steps, args.warmup, args.repeats, barrier)
        launches = S.launch_count() - launches0
        # keep sampling under load for at least ~1.5 s so that the clock record is meaningful
        t_end = time.time() + max(0.0, 1.5 - sum(regions) * args.steps / 1e3)
        while time.time() < t_end:
            plan.spmm(B, Cd)
        torch.cuda.synchronize()
    ms_step_local = statistics.median(regions)
    ms_step = max_over_ranks(ms_step_local)
    value = flops_total / (ms_step * 1e-3) * 1e-12
    parity = parity_check(_Rows(Cd), b0, brp_h, bci_h, bv_h, p.B_nk, p.M, N, p.K)

    # ---------------- end to end: host B in, host C out, every step ----------------
    B_host = torch.from_numpy(p.B_nk.view(np.int16)).pin_memory()
    C_host = torch.empty(((b1 - b0) * 16, N), dtype=torch.int16).pin_memory()

    def e2e_step():
        if dist is None:
            # smat_plan_spmm_host: B copied in and C copied out in column chunks, pipelined with the multiplication
            plan.spmm_host(B_host, C_host)
        else:
            # every rank uploads its 1/N of B; the slices are exchanged on the device (NCCL all-gather over NVLink)
            plan.spmm_host_sharded(B_host, C_host)

    for _ in range(2):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    e2e_value = flops_total / (e2e_ms * 1e-3) * 1e-12
    parity = max(parity, parity_check(_Rows(C_host.view(torch.float16)), b0, brp_h, bci_h, bv_h, p.B_nk, p.M, N, p.K))
    parity = max_over_ranks(parity)
    h2d = int(N * p.K * 2) if dist is None else int((S.b_slice_of_rank(N, world, rank)[1] - S.b_slice_of_rank(N, world, rank)[0]) * p.K * 2)
    del B_host, C_host

    # ---------------- optional exchange step, reported beside the SpMM: all-gather of the C shards ----------------
    gather = None
    if dist is not None:
        C_full = torch.empty((p.M, N), dtype=torch.float16, device="cuda")
        for _ in range(2):
            S.all_gather_rows(Cd, ctx["bounds"], out=C_full)
        barrier()
        g_steps = 5
        e0.record()
        for _ in range(g_steps):
            S.all_gather_rows(Cd, ctx["bounds"], out=C_full)
        e1.record()
        barrier()
        gather = {"ms": round(max_over_ranks(e0.elapsed_time(e1) / g_steps), 4),
                  "bytes_received_per_rank": int(p.M * N * 2 - (b1 - b0) * 16 * N * 2),
                  "note": "padded NCCL all_gather of the C shards + copy into place; not part of value or e2e"}
        del C_full

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---------------- roofline of the SpMM kernel (rank 0's launch) ----------------
    peaks = load_peaks()
    bytes_alg = algorithmic_bytes(brp_h[b0:b1 + 1] - brp_h[b0], bci_h[brp_h[b0]:brp_h[b1]], (b1 - b0) * 16, N)
    kinfo = plan.info()
    roof = roofline_of(peaks, bytes_alg, 2.0 * 256.0 * N * my_blocks, ms_step_local,
                       NCU_TRAFFIC_BYTES.get((args.config, args.scale, world, kinfo["kernel"])), kinfo["kernel"])
    roof["rows_per_item"] = kinfo["rows_per_item"]

    # ---------------- CPU baseline: the reference's blocked multiply on a bounded sample ----------------
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        # calibrate on a small range, then size the sample for the requested seconds
        cal = sample_ranges(brp_h, Mb, max(64, A.nnzb // 2000), 1)
        secs, kind, nb = cpu_reference_multiply(bv_h, brp_h, bci_h, p.B_nk, p.M, p.K, N, cal, 1)
        rate = nb / max(secs, 1e-6)
        want = int(min(A.nnzb, max(nb, rate * args.cpu_sample_seconds)))
        rng = sample_ranges(brp_h, Mb, want, 1)
        secs, kind, nb = cpu_reference_multiply(bv_h, brp_h, bci_h, p.B_nk, p.M, p.K, N, rng, 1)
        cpu = {"value": round(2.0 * 256.0 * N * nb / secs * 1e-12, 6), "unit": "TFLOP/s", "cores": 1, "kind": kind,
               "sample": f"block-rows [{rng[0][0]},{rng[0][1]}) = {nb} of {A.nnzb} blocks ({100.0 * nb / A.nnzb:.2f}%), "
                         f"{secs:.1f}s, VBR::multiply fp32 single thread"}

    other = gpu_baselines(A, B, p, N, log) if want_gpu_baselines else None

    def l2_label(nnzb, K, n_cols, rows):
        resident = nnzb * 512 + n_cols * K * 2 + rows * n_cols * 2  # A blocks + B + C touched by every step
        return ("inputs larger than L2 (A blocks, B and C of a step: %.0f MB; every step streams them from HBM)" % (resident / 1e6)
                if resident > 126e6 else "inputs fit L2 (%.0f MB); no flush between steps" % (resident / 1e6))

    out = {
        "metric": METRIC, "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_step, 5), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": f"{args.config}: {p.desc}; 16x16 blocking" + ("; similarity row reorder" if p.reorder else ""),
                   "M": p.M, "K": p.K, "N": N, "nnzb": A.nnzb, "block_fill": round(ctx["nnz"] / (A.nnzb * 256.0), 5),
                   "parallelism": f"block-rows split by block count over {world} GPU(s), B replicated, C sharded",
                   "l2": l2_label(my_blocks, p.K, N, (b1 - b0) * 16),
                   "kernel_variant": args.variant,
                   "timing": f"median of {args.repeats} regions of {args.steps} launches (CUDA events on the launch stream), max over ranks",
                   "setup_s": ctx["setup_s"]},
        "regions_ms_per_step": [round(x, 5) for x in regions],
        "e2e": {"value": round(e2e_value, 2), "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": int((b1 - b0) * 16 * N * 2), "ms_per_step": round(e2e_ms, 4), "steps": args.steps,
                "note": ("smat_plan_spmm_host per step: B host->device (pinned) and C device->host in column chunks pipelined with the "
                         "multiplication; A (blocked) resident") if world == 1 else
                        ("per step and rank: 1/N of B host->device (pinned), NCCL all-gather of the slices over NVLink, multiply, "
                         "C shard device->host; h2d/d2h bytes are rank 0's")},
        "gpu_launches": int(launches),
        "parity_max_rel_err": float(f"{parity:.3e}"),
        "clocks": clocks.summary(),
        "roofline": roof,
        "cpu_baseline": cpu,
    }
    if other is not None:
        out["gpu_baselines"] = other
    if gather is not None:
        out["c_allgather"] = gather

    # ---------------- the other configurations, one region each (1 GPU) ----------------
    if world == 1 and not args.no_all_configs:
        rows = [{"config": args.config, "ms": round(ms_step, 5), "tflops": round(value, 2), "bound": roof["bound"], "frac": roof["frac"],
                 "nnzb": A.nnzb, "parity_max_rel_err": float(f"{parity:.3e}")}]
        plan.close()
        del ctx, plan, A, B, Cd
        torch.cuda.empty_cache()
        for name in [n for n in ALL_CONFIGS + ["clustered_literal"] if n != args.config]:
            try:
                c2 = prepare(name, args.scale, 0, 1, None, log)
                reg = time_regions(c2, max(args.steps, 20), 3, 1, barrier)
                p2, h2 = c2["p"], c2["host"]
                ms2 = reg[0]
                r2 = roofline_of(peaks, algorithmic_bytes(h2[0], h2[1], p2.M, p2.N), 2.0 * 256.0 * p2.N * c2["A"].nnzb, ms2, None,
                                 c2["plan"].info()["kernel"])
                par2 = parity_check(_Rows(c2["Cd"]), 0, h2[0], h2[1], h2[2], p2.B_nk, p2.M, p2.N, p2.K)
                rows.append({"config": name, "ms": round(ms2, 5), "tflops": round(2.0 * 256.0 * p2.N * c2["A"].nnzb / (ms2 * 1e-3) * 1e-12, 2),
                             "bound": r2["bound"], "frac": r2["frac"], "kernel": r2["kernel"], "nnzb": c2["A"].nnzb,
                             "block_fill": round(c2["nnz"] / (c2["A"].nnzb * 256.0), 5), "parity_max_rel_err": float(f"{par2:.3e}"),
                             "setup_s": c2["setup_s"]})
                c2["plan"].close()
                del c2
                torch.cuda.empty_cache()
            except Exception as e:  # one configuration failing must not lose the headline line
                rows.append({"config": name, "error": f"{type(e).__name__}: {e}"[:200]})
        out["all_configs"] = rows
    print(json.dumps(out), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_reference_arm(args, rank, world, log):
    """The reference's CPU blocked multiply (oracle/_ref when built, else the oracle port) on the same
    workload, all host cores, each step a bounded sample."""
    if rank != 0:
        return
    import oracle
    import smat_b200 as S
    p = build_problem(args.config, args.scale, log)
    rp, ci, v, reorder_s, _ = reorder_if_needed(p, log, None, args.config, args.scale)
    brp, bci, bv = oracle.csr_to_bcsr(p.M, p.K, rp, ci, v)
    nnzb, Mb, N = len(bci), p.M // 16, p.N
    cores = os.cpu_count() or 1
    # size one step at roughly 2 s of work per core
    cal = sample_ranges(brp, Mb, max(64, nnzb // 4000), 1)
    secs, kind, nb = cpu_reference_multiply(bv, brp, bci, p.B_nk, p.M, p.K, N, cal, 1)
    per_core = int(max(nb, nb / max(secs, 1e-6) * 2.0))
    ranges = sample_ranges(brp, Mb, per_core, cores)
    for _ in range(args.warmup):
        cpu_reference_multiply(bv, brp, bci, p.B_nk, p.M, p.K, N, ranges, cores)
    t_tot, blocks = 0.0, 0
    for _ in range(args.steps):
        secs, kind, nb = cpu_reference_multiply(bv, brp, bci, p.B_nk, p.M, p.K, N, ranges, cores)
        t_tot += secs
        blocks += nb
    value = 2.0 * 256.0 * N * blocks / t_tot * 1e-12
    step_blocks = blocks // max(args.steps, 1)
    sample = (f"{len(ranges)} block-row ranges, {step_blocks} of {nnzb} blocks per step "
              f"({100.0 * step_blocks / nnzb:.2f}%), VBR::multiply fp32, one range per thread")
    out = {
        "impl": "reference", "metric": METRIC, "value": round(value, 6), "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(t_tot / max(args.steps, 1) * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32 (CPU)", "data": "synthetic",
        "config": {"workload": f"{args.config}: {p.desc}; 16x16 blocking" + ("; similarity row reorder" if p.reorder else ""),
                   "M": p.M, "K": p.K, "N": N, "nnzb": nnzb},
        "cpu_baseline": {"value": round(value, 6), "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": round(value, 6), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
