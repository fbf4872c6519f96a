"""Benchmark of the GCN layer path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (default): the largest partitioned configuration -- a 3-layer GCN
(100 -> 256 -> 256 -> 47) training step (forward, NLL loss on all nodes,
backward, Adam) on a seeded R-MAT graph with 2,449,029 nodes and 61,859,140
undirected edges (+ self-loops, symmetric normalisation, int32 CSR), X ~ N(0,1).
At N GPUs the graph is row-partitioned (strong scaling: the same graph).

One JSON line on stdout from rank 0.  `value` is the epoch (= one step) time
with inputs resident in HBM; `e2e` times the same step through the public API
from pinned host buffers (features + labels copied in, loss read back) every
step; `roofline` is measured live on the CSR aggregation kernel with CUDA
events; `cpu_baseline` is the reference's own CPU code on a bounded sample.

`--impl reference` times the reference's CPU implementation (its gcn.cpp built
for CPU, driven by its autograd wrapper) on host cores, on a bounded sample of
the same workload, scaled to the full size.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "gcn_train_epoch_ms"
DIMS = [100, 256, 256, 47]


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shrink", type=int, default=1,
                    help="divide nodes and edges by this factor (profiling captures and quick checks only)")
    ap.add_argument("--precision", default="fp32", choices=["fp32", "fp32_simt", "tf32x3", "tf32", "bf16"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-aux", action="store_true", help="skip the auxiliary single-GPU measurements")
    ap.add_argument("--cpu-sample-div", type=int, default=32)
    ap.add_argument("--partition", default="auto", choices=["auto", "features", "rows", "hybrid"],
                    help="multi-GPU scheme: adjacency rows (all-gather of the aggregated matrix), feature columns "
                         "(two transposes around the aggregation), or hybrid (rows for narrow and constant "
                         "matrices, feature slabs for the hidden width); auto = rows at 2 GPUs, hybrid from 4")
    ap.add_argument("--wide-from", type=int, default=128,
                    help="hybrid scheme: matrices at least this wide are aggregated by feature slabs, narrower ones "
                         "through the row partition")
    ap.add_argument("--exchange", default="auto", choices=["auto", "collective"],
                    help="auto: blocks move by peer copies through symmetric memory; collective: NCCL collectives")
    ap.add_argument("--no-parity", action="store_true",
                    help="skip the untimed CPU float64 check of the benchmarked graph's layers (profiler captures)")
    ap.add_argument("--exchange-probe", action="store_true",
                    help="time the multi-GPU block exchanges alone (peer memory against NCCL) instead of the step")
    ap.add_argument("--profile-warmup", action="store_true",
                    help="honour --warmup below 3 (profiler captures only; such a run is not a benchmark)")
    return ap.parse_args()


def workload(shrink: int):
    synth = _load_synth()
    cfg = dict(synth.CONFIGS["rmat_products"])
    if shrink > 1:
        cfg["nodes"] //= shrink
        cfg["edges"] //= shrink
        cfg["scale"] = max(8, (cfg["nodes"] - 1).bit_length())
    return cfg


# ---------------------------------------------------------------- clocks
class ClockSampler:
    """nvidia-smi sampled every 200 ms while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------- SpMM timer
class SpmmTimer:
    """CUDA-event pairs around every CSR aggregation enqueued while active
    (events are recorded on the stream the kernels run on)."""

    def __init__(self):
        self.records = []
        self.active = False

    def wrap(self, cls):
        timer = self
        orig = cls.matmul

        def timed(self_adj, H, **kw):
            if not timer.active:
                return orig(self_adj, H, **kw)
            a = torch.cuda.Event(enable_timing=True)
            b = torch.cuda.Event(enable_timing=True)
            a.record()
            out = orig(self_adj, H, **kw)
            b.record()
            M, K = self_adj.shape
            F = H.size(1)
            # algorithmic (compulsory) bytes: rowptr + col + val + H read once + Y written once
            nbytes = 4 * (M + 1) + 8 * self_adj.nnz + 4 * K * F + 4 * M * F
            timer.records.append((a, b, nbytes, F, self_adj.nnz))
            return out

        cls.matmul = timed
        orig_blocks = cls.matmul_into_blocks

        def timed_blocks(self_adj, H, *a, **kw):  # the aggregation whose stores go to the owners' buffers
            if not timer.active:
                return orig_blocks(self_adj, H, *a, **kw)
            e_a = torch.cuda.Event(enable_timing=True)
            e_b = torch.cuda.Event(enable_timing=True)
            e_a.record()
            out = orig_blocks(self_adj, H, *a, **kw)
            e_b.record()
            M, K = self_adj.shape
            F = H.size(1)
            timer.records.append((e_a, e_b, 4 * (M + 1) + 8 * self_adj.nnz + 4 * K * F + 4 * M * F, F, self_adj.nnz))
            return out

        cls.matmul_into_blocks = timed_blocks

    def summary(self):
        tot_ms, tot_b, gather_b = 0.0, 0, 0
        per_f = {}
        for a, b, nbytes, F, nnz in self.records:
            ms = a.elapsed_time(b)
            tot_ms += ms
            tot_b += nbytes
            gather_b += nbytes + 4 * nnz * F
            d = per_f.setdefault(F, [0.0, 0, 0])
            d[0] += ms
            d[1] += nbytes
            d[2] += 1
        return tot_ms, tot_b, gather_b, per_f, len(self.records)


def gather_ceiling(dev, n_rows_h: int, F: int = 256):
    """Rate at which the memory system delivers gathered rows of an n_rows_h x F fp32 matrix to the SMs, measured
    with gc_gather_sum_f32 (the aggregation's access pattern and nothing else) on three index lists: rows drawn
    from a 64 MB region (every gather an L2 hit), from the whole matrix (every gather from DRAM) and a 73 % / 27 %
    mix (the L2 hit rate ncu reports for the aggregation on this graph).  TB/s of gathered bytes."""
    from graphcuda_b200 import _lib
    L = _lib.lib()
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    H = torch.randn(n_rows_h, F, generator=g, device=dev)
    n_out, deg = 1 << 19, 64
    Y = torch.empty(n_out, F, device=dev)
    hot = min((64 << 20) // (F * 4), n_rows_h)
    cold = torch.randint(0, n_rows_h, (n_out * deg,), generator=g, device=dev, dtype=torch.int32)
    warm = torch.randint(0, hot, (n_out * deg,), generator=g, device=dev, dtype=torch.int32)
    mix = torch.where(torch.rand(n_out * deg, generator=g, device=dev) < 0.73, warm, cold)
    res = {}
    for name, idx in (("l2_resident", warm), ("l2_hit_73pct", mix), ("dram", cold)):
        def run():
            st = L.gc_gather_sum_f32(H.data_ptr(), F, n_rows_h, F, idx.data_ptr(), n_out, deg, Y.data_ptr(), F, 4,
                                     torch.cuda.current_stream(dev).cuda_stream)
            if st != 0:
                raise RuntimeError(L.gc_last_error().decode())
        ms = _time_ms(run, warm=2, iters=5)
        res[name + "_TBs"] = n_out * deg * F * 4 / (ms * 1e-3) / 1e12
    return res


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


# ---------------------------------------------------------------- CPU baseline (reference code)
def _load_synth():
    """The seeded generators, loaded by file path: importing the package would load the CUDA library, and the
    reference arm must run without any of this repository's kernels in the process."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("_gc_synth", os.path.join(ROOT, "graphcuda_b200", "synth.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _cpu_reference_sample(cfg, sample_div: int, steps: int, warmup: int, budget_s: float):
    """ms per training step of the reference's CPU path (its gcn.cpp compiled for CPU when present, else the
    restatement of it) on an R-MAT sample 1/sample_div the size of the workload (same generator, same average
    degree, same 3-layer model).  Stops early when budget_s is used up; returns (ms, steps actually timed, kind)."""
    synth = _load_synth()
    from oracle import gcn_oracle as O
    from oracle import ref_loader
    kind = "port"
    ops = None
    if ref_loader.ref_ext_available():
        try:
            ops = ref_loader.load_ref_ext()
            kind = "reference"
        except Exception:
            ops = None
    n = cfg["nodes"] // sample_div
    m = cfg["edges"] // sample_div
    scale = max(8, (n - 1).bit_length())
    e = synth.rmat_edges(scale, n, m, cfg["seed"])
    A = O.normalized_adjacency_coo(synth.symmetrize(e), n)
    X = synth.normal_features(n, DIMS[0], seed=11)
    y = synth.uniform_labels(n, DIMS[-1], seed=12)
    torch.manual_seed(0)
    model = O.GCN(DIMS, ops=ops)
    opt = torch.optim.Adam(model.parameters(), lr=0.01)

    def step():
        opt.zero_grad(set_to_none=True)
        loss = torch.nn.functional.nll_loss(model(X, A), y)
        loss.backward()
        opt.step()
        return loss.item()

    t_begin = time.perf_counter()
    for i in range(warmup):
        step()
        if i >= 0 and time.perf_counter() - t_begin > budget_s / 3:
            break
    done = 0
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
        done += 1
        if time.perf_counter() - t_begin > budget_s:
            break
    ms = (time.perf_counter() - t0) * 1e3 / max(done, 1)
    return ms, done, kind, n, m


def cpu_reference_epoch_ms(cfg, sample_div: int, steps: int, warmup: int, check_div: int = 0,
                           budget_s: float = 150.0):
    """The reference's CPU path timed on a bounded sample and scaled to the full workload.

    The main sample (1/sample_div) runs the requested steps; a second, larger sample (1/check_div, two steps)
    measures how the time grows with the size (exponent p: time ~ size^p).  `value` is the time of the LARGEST
    sample measured, scaled linearly to the full size: on these hosts the growth is super-linear (p > 1: caches),
    so the linear figure is a lower bound of the reference's time -- the comparison errs in the reference's
    favour -- and the power-law figure is reported beside it.  Returns a dict."""
    # all the host threads this process may use (a launcher may have exported OMP_NUM_THREADS=1 for its workers)
    avail = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(max(1, avail))
    ms_a, done_a, kind, n_a, m_a = _cpu_reference_sample(cfg, sample_div, steps, warmup, budget_s)
    p = 1.0
    second = None
    if check_div and check_div < sample_div:
        ms_b, done_b, _, n_b, m_b = _cpu_reference_sample(cfg, check_div, 2, 1, budget_s)
        import math
        p = math.log(ms_b / ms_a) / math.log(sample_div / check_div)
        second = {"div": check_div, "nodes": n_b, "undirected_edges": m_b, "ms_per_step": ms_b, "steps": done_b}
        full = ms_b * check_div
        power_law = ms_b * (check_div ** p)
    else:
        full = ms_a * sample_div
        power_law = None
    sample = (f"R-MAT sample 1/{sample_div} of the workload ({n_a} nodes, {m_a} undirected edges, same degree, "
              f"same 3-layer model, fwd+loss+bwd+Adam): {ms_a:.1f} ms per step over {done_a} timed steps")
    if second:
        sample += (f"; second sample 1/{check_div} ({second['nodes']} nodes): {second['ms_per_step']:.1f} ms per step "
                   f"=> time ~ size^{p:.3f} (1.000 = linear); value = the 1/{check_div} time x {check_div} "
                   f"(linear: a lower bound when the exponent exceeds 1; with the measured exponent: "
                   f"{power_law:.0f} ms)")
    else:
        sample += f"; value = that time x {sample_div} (work is linear in nodes and edges)"
    return {"value": full, "unit": "ms", "cores": torch.get_num_threads(), "kind": kind, "sample": sample,
            "extrapolated": True, "measured": {"div": sample_div, "ms_per_step": ms_a, "steps": done_a},
            "second_point": second, "growth_exponent": p, "power_law_estimate_ms": power_law}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = workload(args.shrink)
    # the sample is sized so that one step is a few seconds of CPU work; the requested step counts are honoured
    # as far as they fit a bounded run (the line says how many steps were timed)
    cb = cpu_reference_epoch_ms(cfg, args.cpu_sample_div, max(1, args.steps), max(1, args.warmup),
                                check_div=max(1, args.cpu_sample_div // 4), budget_s=150.0)
    ms = cb["value"]
    done = cb["measured"]["steps"]
    line = {
        "impl": "reference", "metric": METRIC, "value": ms, "unit": "ms", "n_gpus": args.gpus, "steps": done,
        "warmup": max(1, args.warmup), "ms_per_step": ms, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": config_dict(cfg, args, 1),
        "value_is": "extrapolated from bounded samples of the workload (see cpu_baseline.sample); "
                    "the measured per-step times are in cpu_baseline.measured / second_point",
        "steps_requested": args.steps, "steps_capped": done < args.steps,
        "cpu_baseline": cb,
        "e2e": {"value": ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "shared_objects_of_this_repo_loaded": _repo_shared_objects(),
    }
    print(json.dumps(line), flush=True)


def _repo_shared_objects():
    """Shared objects under this repository mapped into this process (the reference arm must show the
    reference's CPU module only, never the CUDA library of the package)."""
    found = set()
    try:
        for ln in open("/proc/self/maps"):
            path = ln.split()[-1]
            if path.startswith(ROOT) and ".so" in path:
                found.add(os.path.relpath(path, ROOT))
    except OSError:
        pass
    return sorted(found)


def config_dict(cfg, args, world):
    return {
        "workload": "rmat_products: 3-layer GCN 100-256-256-47 train step, R-MAT a=.57 b=.19 c=.19 d=.05",
        "nodes": cfg["nodes"], "undirected_edges": cfg["edges"], "nnz": 2 * cfg["edges"] + cfg["nodes"],
        "dims": DIMS, "optimizer": "Adam lr=0.01", "loss": "nll over all nodes",
        "parallelism": (f"{args.partition}-sharded x{world}" if world > 1 else "single GPU"),
        "precision": args.precision, "l2": "inputs larger than L2 (no flush needed)",
        "shrink": args.shrink,
    }


# ---------------------------------------------------------------- per-phase device times (one extra, untimed step)
class PhaseProfile:
    """CUDA-event pairs around every aggregation kernel call, GEMM call and exchange of ONE training step, with
    each exchange waited for where it is issued (no overlap), so the phases add up: what a step spends in the
    aggregation, the dense products, moving blocks between GPUs, and everything else."""

    def __init__(self):
        self.ev = {"spmm_ms": [], "gemm_ms": [], "exchange_ms": []}
        self.undo = []

    def _wrap(self, obj, name, phase, sync_work=False):
        orig = getattr(obj, name)
        prof = self

        def timed(*a, **kw):
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            out = orig(*a, **kw)
            if sync_work and isinstance(out, tuple) and out[1] is not None:
                out[1].wait()  # the gather is complete before the clock stops (and before anything overlaps it)
            e1.record()
            prof.ev[phase].append((e0, e1))
            return out

        setattr(obj, name, timed)
        self.undo.append((obj, name, orig))

    def install(self):
        from graphcuda_b200 import partition as P
        self._wrap(P.CudaBackend, "spmm", "spmm_ms")
        self._wrap(P.CudaBackend, "spmm_into_blocks", "spmm_ms")  # the aggregation that stores into the owners
        self._wrap(P.CudaBackend, "gemm", "gemm_ms")
        self._wrap(P.PartitionedGraph, "all_gather_rows_async", "exchange_ms", sync_work=True)
        self._wrap(P.FeatureShardedGraph, "rows_to_columns", "exchange_ms")
        self._wrap(P.FeatureShardedGraph, "columns_to_rows", "exchange_ms")
        self._wrap(P.PartitionedGraph, "all_reduce_sum", "exchange_ms")
        self._wrap(P.FeatureShardedGraph, "all_reduce_sum", "exchange_ms")

    def remove(self):
        for obj, name, orig in reversed(self.undo):
            setattr(obj, name, orig)
        self.undo = []

    def result(self, step_ms):
        out = {k: sum(a.elapsed_time(b) for a, b in v) for k, v in self.ev.items()}
        out["calls"] = {k: len(v) for k, v in self.ev.items()}
        out["step_ms_serialised"] = step_ms
        out["other_ms"] = step_ms - out["spmm_ms"] - out["gemm_ms"] - out["exchange_ms"]
        big = max(("spmm_ms", "gemm_ms", "exchange_ms", "other_ms"), key=lambda k: out[k])
        out["limiter"] = big[:-3]
        return out


# ---------------------------------------------------------------- parity (outside every timed region)
PARITY_TOL = 1e-4


def _cpu_rows_times_matrix(rows, rowptr, col, val, H):
    """sum_j A[r, j] H[j, :] in float64 for the listed rows of a CSR matrix held on the CPU."""
    out = torch.zeros(len(rows), H.size(1), dtype=torch.float64)
    for i, r in enumerate(rows.tolist()):
        s, e = int(rowptr[r]), int(rowptr[r + 1])
        if e > s:
            out[i] = val[s:e].double() @ H[col[s:e].long()].double()
    return out


def _rel_errs(out, ref):
    out = out.double()
    d = (out - ref)
    return float(d.norm() / max(float(ref.norm()), 1e-300)), float(d.abs().max() / max(float(ref.abs().max()), 1e-300))


def parity_block(make_model, X, y, graph, X_gathered, csr_host, n, world, rank, dev, gather_rows):
    """Compares the training path on the benchmarked graph with the reference's layer formulas evaluated on the
    CPU in float64 (src/graphcuda/cpp/gcn.cpp:10-15 forward, :34 weight gradient), layer by layer on the
    layer's own input as the GPU produced it:
      * forward: relu((A h_{l-1}) W_l) on ~1000 sampled rows (the highest- and lowest-degree rows, the rest
        drawn at random over ALL ranks' rows);
      * backward: the whole dW_1 = (A X)^T G_1 (a sum over every node, all-reduced over the ranks).
    gather_rows(t) returns the full matrix (all ranks' row blocks) on every rank.  Runs once, untimed.

    The check runs on freshly initialised weights (the seed the benchmark starts from), not on the weights the
    timed steps leave behind: with uniform random labels Adam drives this model to all-zero hidden activations
    within a few steps (the loss settles at exactly ln 47), and a comparison of zeros with zeros would prove
    nothing.  The logits of 64 fixed nodes from the same forward are returned as a probe that lines run on
    different numbers of GPUs can be compared on."""
    import graphcuda_b200 as gc
    model = make_model()
    if world == 1:
        out, hs = model(X, graph, log_softmax=False, return_hidden=True)
    else:
        out, hs = model(X, graph, X_gathered=X_gathered, log_softmax=False, return_hidden=True)
    for h in hs[1:]:
        h.retain_grad()
    loss = gc.log_softmax_nll_loss(out, y, scale=1.0 / n)
    loss.backward()
    weights = [p_.detach() for p_ in model.parameters()]
    full = [gather_rows(h.detach()) for h in hs]
    G1 = gather_rows((hs[1].grad * (hs[1].detach() > 0)).contiguous())  # gated gradient of layer 1 (idempotent)
    dW1 = list(model.parameters())[0].grad.detach().clone()
    probe_rows = torch.linspace(0, n - 1, 64).long()
    probe = full[-1][probe_rows.to(dev)].double()
    logits_probe = {"rows": "64 nodes, torch.linspace(0, n-1, 64); weights as initialised from seed 0",
                    "sum": float(probe.sum().item()), "abs_sum": float(probe.abs().sum().item()),
                    "l2": float(probe.norm().item()),
                    "first_row": [float(f"{float(v):.6e}") for v in probe[0].tolist()[:8]]}
    res = None
    if rank == 0:
        rowptr, col, val = csr_host
        deg = (rowptr[1:] - rowptr[:-1])
        order = torch.argsort(deg, descending=True, stable=True)
        g = torch.Generator().manual_seed(123)
        rows = torch.cat([order[:16], order[-16:], torch.randint(0, n, (992,), generator=g)]).unique()
        layers = {}
        worst = 0.0
        for l, W in enumerate(weights):
            Hprev = full[l].cpu()
            ref = _cpu_rows_times_matrix(rows, rowptr, col, val, Hprev) @ W.double().cpu()
            if l < len(weights) - 1:
                ref = ref * (ref > 0)
            fro, mx = _rel_errs(full[l + 1][rows.to(dev)].cpu(), ref)
            layers[f"layer{l + 1}_forward"] = {"rel_fro": fro, "rel_max": mx, "rows": int(rows.numel())}
            worst = max(worst, fro, mx)
            del Hprev
        # dW of the first layer over every node: (A X)^T G in float32 blocks summed in float64
        A = torch.sparse_csr_tensor(rowptr.long(), col.long(), val, size=(n, n))
        AX = A @ full[0].cpu()
        Gc = G1.cpu()
        acc = torch.zeros(AX.size(1), Gc.size(1), dtype=torch.float64)
        for s0 in range(0, n, 1 << 16):
            acc += (AX[s0:s0 + (1 << 16)].t() @ Gc[s0:s0 + (1 << 16)]).double()
        fro, mx = _rel_errs(dW1.cpu(), acc)
        layers["layer1_weight_gradient"] = {"rel_fro": fro, "rel_max": mx, "rows": n}
        worst = max(worst, fro, mx)
        res = {"ok": bool(worst < PARITY_TOL), "tolerance": PARITY_TOL, "max_rel_err": worst, "checks": layers,
               "reference": "CPU float64 evaluation of relu((A h) W) and (A X)^T G on the GPU's own layer inputs, "
                            "sampled rows over all ranks (forward) / all rows (weight gradient)",
               "weights": "freshly initialised (seed 0)", "loss_first_step": float(loss.item()),
               "hidden_abs_mean": [float(f.abs().mean().item()) for f in full[1:]]}
    else:
        float(loss.item())
    return res, logits_probe


# ---------------------------------------------------------------- our arm
def run_ours(args):
    import torch.distributed as dist

    import graphcuda_b200 as gc
    from graphcuda_b200 import _lib, adjacency, ops, synth
    from graphcuda_b200.models import GCN
    from graphcuda_b200.partition import DistGCN, FeatureShardedGraph, HybridGraph, PartitionedGraph

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.partition == "auto":
        args.partition = "hybrid" if world >= 4 else "rows"  # measured: 21.8 / 22.4 ms at 2, 15.9 / 14.9 at 4, 14.6 / 10.1 at 8
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = _lib.lib()
    cfg = workload(args.shrink)
    n = cfg["nodes"]

    # ---- inputs (seeded, generated on the device; identical on every rank) ----
    t0 = time.time()
    edges = synth.rmat_edges(cfg["scale"], n, cfg["edges"], cfg["seed"], device=dev)
    adj = gc.normalized_adjacency(synth.symmetrize(edges), n, symmetric=True)
    del edges
    csr_host = None
    if rank == 0 and not args.no_parity:  # the checker's copy of the graph (host memory)
        csr_host = (adj.rowptr.cpu().long(), adj.col.cpu(), adj.val.cpu())
    part = None
    if world == 1:
        X = synth.normal_features(n, DIMS[0], seed=11, device=dev)
        y = synth.uniform_labels(n, DIMS[-1], seed=12, device=dev)
        torch.manual_seed(0)
        model = GCN(DIMS, precision=args.precision).to(dev)
        rows = n
    else:
        if args.partition == "rows":
            part = PartitionedGraph(adj.rowptr, adj.col, adj.val, n, rank=rank, world=world, exchange=args.exchange)
        elif args.partition == "hybrid":
            part = HybridGraph(adj.rowptr, adj.col, adj.val, adj, n, rank=rank, world=world, exchange=args.exchange,
                               wide_from=args.wide_from)
        else:
            part = FeatureShardedGraph(adj, n, rank=rank, world=world, exchange=args.exchange)
        lo, hi = part.lo, part.hi
        Xf = synth.normal_features(n, DIMS[0], seed=11, device=dev)
        yf = synth.uniform_labels(n, DIMS[-1], seed=12, device=dev)
        X = Xf[lo:hi].contiguous()
        y = yf[lo:hi].contiguous()
        del Xf, yf
        if args.partition == "rows":
            del adj
        torch.manual_seed(0)
        model = DistGCN(DIMS, precision=args.precision).to(dev)
        rows = hi - lo
        adj = None
    torch.cuda.synchronize()
    setup_s = time.time() - t0
    opt = gc.FusedAdam(model.parameters(), lr=0.01)  # torch.optim.Adam's update, one launch for all weights

    X_gathered = None
    if world > 1:
        X_gathered = part.prepare_constant(X)

    def step(Xd, yd, Xg):
        opt.zero_grad(set_to_none=True)
        # log_softmax + NLL over all nodes, fused (mean over the n nodes of the whole graph)
        if world == 1:
            loss = gc.log_softmax_nll_loss(model(Xd, adj, log_softmax=False), yd, scale=1.0 / n)
        else:
            loss = gc.log_softmax_nll_loss(model(Xd, part, X_gathered=Xg, log_softmax=False), yd, scale=1.0 / n)
        loss.backward()
        opt.step()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    timer = SpmmTimer()
    timer.wrap(adjacency.CSRAdjacency)

    # ---- warm-up ----
    n_warm = args.warmup if args.profile_warmup else max(args.warmup, 3)
    for _ in range(n_warm):
        step(X, y, X_gathered)
    barrier()
    ops.check_gemm_flag(dev)

    # ---- timed region: inputs resident in HBM ----
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = L.gc_launch_count()
    timer.active = True
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    t_host = time.perf_counter()
    for _ in range(args.steps):
        loss = step(X, y, X_gathered)
    enqueue_ms = (time.perf_counter() - t_host) * 1e3 / max(args.steps, 1)  # host time to issue a step (no sync)
    e1.record()
    barrier()
    timer.active = False
    launches = L.gc_launch_count() - launches0
    ms_step = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    clocks = sampler.stop() if rank == 0 else None
    final_loss = float(loss.item())

    # ---- parity, untimed: the layers of THIS graph against the reference's formulas on the CPU, and a probe of
    # the logits of 64 fixed nodes (spread over all ranks' rows) that lines run at different N can be compared on
    def gather_rows(t):
        if world == 1:
            return t
        B = part.part.block
        src = torch.zeros((B, t.size(1)), dtype=t.dtype, device=dev)
        src[:t.size(0)].copy_(t)
        full = torch.empty((B * world, t.size(1)), dtype=t.dtype, device=dev)
        dist.all_gather_into_tensor(full, src)
        return part.part.unpad(full)

    phases = None
    if world > 1:  # rank 0's phases of one extra step, exchanges not overlapped
        prof = PhaseProfile()
        prof.install()
        try:
            barrier()
            e0.record()
            step(X, y, X_gathered)
            e1.record()
            barrier()
            phases = prof.result(e0.elapsed_time(e1))
        finally:
            prof.remove()
    parity = logits_probe = None
    if not args.no_parity:
        def fresh_model():
            torch.manual_seed(0)
            m = GCN(DIMS, precision=args.precision) if world == 1 else DistGCN(DIMS, precision=args.precision)
            return m.to(dev)

        parity, logits_probe = parity_block(fresh_model, X, y, adj if world == 1 else part, X_gathered, csr_host, n,
                                            world, rank, dev, gather_rows)
        barrier()

    # ---- end to end: pinned host inputs copied in, loss read back, every step ----
    Xh = X.cpu().pin_memory()
    yh = y.cpu().pin_memory()
    feed = gc.PinnedFeed(dev, like=[X, y])

    def e2e_run(k: int, overlap: bool) -> None:
        """k steps, each with its own host->device copy of the inputs and a device->host read of the loss.
        overlap: the copy of step i + 1 is issued before step i computes (input prefetch, as a data loader does);
        otherwise copy and compute alternate.  The first copy is never hidden."""
        feed.submit([Xh, yh])
        for i in range(k):
            Xd, yd = feed.take()
            if overlap and i + 1 < k:
                feed.submit([Xh, yh])
            Xg = part.prepare_constant(Xd, keep=False) if world > 1 else None  # fresh inputs every step
            loss = step(Xd, yd, Xg)
            feed.release()
            float(loss.item())  # the device-to-host read of the result
            if not overlap and i + 1 < k:
                feed.submit([Xh, yh])

    e2e_times = {}
    for overlap in (False, True):
        e2e_run(2, overlap)
        barrier()
        e0.record()
        e2e_run(args.steps, overlap)
        e1.record()
        barrier()
        e2e_times[overlap] = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    e2e_ms = e2e_times[True]
    h2d = Xh.numel() * 4 + yh.numel() * 8
    if world > 1:
        t = torch.tensor([h2d], dtype=torch.float64, device=dev)
        dist.all_reduce(t)
        h2d = int(t.item())

    # ---- roofline of the CSR aggregation (rank 0's launches) ----
    sp_ms, sp_bytes, sp_gather_bytes, per_f, n_spmm = timer.summary()
    peak, peak_src = measured_peaks()
    achieved = sp_bytes / (sp_ms * 1e-3) / 1e9 if sp_ms > 0 else 0.0
    roofline = {
        "kernel": "spmm_pieces_kernel (+ spmm_finalize_kernel)",
        "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
        "peak_source": peak_src,
        "bytes": "compulsory: 4(M+1) + 8 nnz + 4 K F + 4 M F per launch",
        "launches_timed": n_spmm, "avg_launch_ms": sp_ms / n_spmm if n_spmm else None,
        "gather_model_gbs": sp_gather_bytes / (sp_ms * 1e-3) / 1e9 if sp_ms > 0 else 0.0,
        "per_feature_width": {str(F): {"ms": d[0] / d[2], "gbs": d[1] / (d[0] * 1e-3) / 1e9, "launches": d[2]}
                              for F, d in sorted(per_f.items())},
        "share_of_step": sp_ms / args.steps / ms_step if ms_step > 0 else None,
        # dram__bytes_read.sum + dram__bytes_write.sum of the F = 256 launch (pieces + finalize kernels) from an ncu
        # capture on the half-size graph, scaled by the non-zeros: an offline figure, not a measurement of this
        # run; the compulsory bytes of that launch are 6.04e9
        "traffic": 21.7e9 if (args.shrink == 1 and world == 1) else None,
        "traffic_source": "profiled offline with ncu (dram__bytes_read.sum + dram__bytes_write.sum, F = 256 launch, "
                          "pieces + finalize kernels) on the half-size graph, x2 for the non-zeros; the kernel "
                          "source has not changed since that capture",
        "traffic_note": "bytes per F=256 launch at full size on 1 GPU; compulsory 6.04e9",
    }

    if world == 1 and per_f.get(256):
        # what the memory system can deliver for this access pattern, beside what the aggregation gets
        try:
            gc_ = gather_ceiling(dev, n, 256)
            d256 = per_f[256]
            gathered = adj.nnz * 256 * 4 / (d256[0] / d256[2] * 1e-3) / 1e12
            gc_["aggregation_F256_gathered_TBs"] = gathered
            gc_["aggregation_vs_l2_resident_ceiling"] = gathered / gc_["l2_resident_TBs"]
            gc_["note"] = ("gathered bytes = nnz x F x 4; the aggregation's figure includes its L1 hits, the ceiling "
                           "rows are uniform random (no L1 reuse)")
            roofline["gather_ceiling"] = gc_
        except Exception as ex:
            roofline["gather_ceiling"] = {"error": repr(ex)[:200]}

    line = {
        "metric": METRIC, "value": ms_step, "unit": "ms", "n_gpus": world, "steps": args.steps,
        "warmup": n_warm, "ms_per_step": ms_step, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config_dict(cfg, args, world),
        "roofline": roofline,
        "e2e": {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * world,
                "how": "public API (GCN + log_softmax_nll_loss + FusedAdam) fed by PinnedFeed: every step copies its "
                       "features and labels from pinned host memory and reads the loss back; the copy of step i+1 is "
                       "in flight while step i computes, the first copy of the timed region is exposed",
                "value_without_prefetch": e2e_times[False]},
        "gpu_launches": int(launches), "clocks": clocks, "final_loss": final_loss, "setup_s": setup_s,
        "host_enqueue_ms_per_step": enqueue_ms,
        "partition": (args.partition if world > 1 else "none"),
        "exchange": (("peer copies through symmetric memory" if part.symm is not None else "NCCL collectives")
                     if world > 1 else "none"),
        "parity": parity, "logits_probe": logits_probe, "phases": phases,
        "spmm_gbs": achieved, "spmm_pct_hbm_peak": 100.0 * achieved / peak,
    }

    if rank == 0 and world == 1 and not args.no_aux:
        try:
            line["aux"] = aux_measurements(dev, args)
            # the F = 256 aggregation of the headline graph gathering a bf16 copy of H (reduced-precision tier)
            from graphcuda_b200 import ops as _ops2
            Hf = synth.normal_features(n, 256, seed=256, device=dev)
            H16 = _ops2.to_bf16(Hf)
            line["aux"]["rmat_products_spmm_F256_ms"] = {"fp32_H": _time_ms(lambda: adj.matmul(Hf), warm=2, iters=5),
                                                         "bf16_H": _time_ms(lambda: adj.matmul(H16), warm=2, iters=5)}
            del Hf, H16
            # the same training step in the opt-in reduced-precision tiers (1e-2 relative): not the headline
            for tier in ("tf32", "bf16"):
                torch.manual_seed(0)
                m2 = GCN(DIMS, precision=tier).to(dev)
                o2 = gc.FusedAdam(m2.parameters(), lr=0.01)

                def tier_step():
                    o2.zero_grad(set_to_none=True)
                    l2 = gc.log_softmax_nll_loss(m2(X, adj, log_softmax=False), y, scale=1.0 / n)
                    l2.backward()
                    o2.step()

                line["aux"][f"rmat_products_train_step_ms_{tier}_tier"] = _time_ms(tier_step, warm=2, iters=5)
                del m2, o2
            torch.cuda.empty_cache()
            line["aux"]["reference_cuda_same_box"] = reference_cuda_same_box(dev, adj)
            # the script's test(): no-grad forward of the same model + fused argmax / accuracy counts
            line["aux"]["rmat_products_eval_forward_argmax_ms"] = _time_ms(lambda: model.evaluate(X, adj, y), warm=2,
                                                                          iters=5)
        except Exception as ex:  # auxiliary numbers never take the headline down
            line["aux"] = {"error": repr(ex)}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_reference_epoch_ms(cfg, args.cpu_sample_div, 2, 1,
                                                      check_div=max(1, args.cpu_sample_div // 4), budget_s=90.0)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _time_ms(fn, warm=3, iters=10):
    for _ in range(warm):
        fn()
    a = torch.cuda.Event(enable_timing=True)
    b = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def aux_measurements(dev, args):
    """Secondary single-GPU numbers: the Cora-shaped 2-layer training epoch, the
    arxiv-shaped CSR aggregation and the feature-transform GEMM."""
    import graphcuda_b200 as gc
    from graphcuda_b200 import synth
    from graphcuda_b200.models import GCN
    out = {}
    peak, _ = measured_peaks()

    # 2-layer GCN, N=2708, 1433 -> 16 -> 7, Adam lr=0.01 (train step only, like the reference's timer)
    c = synth.CONFIGS["cora_like"]
    e = synth.preferential_attachment_edges(c["nodes"], c["edges"], c["seed"]).to(dev)
    adj = gc.normalized_adjacency(synth.symmetrize(e), c["nodes"], symmetric=True)
    X = synth.bow_features(c["nodes"], c["features"], 0.0127, seed=1, device=dev)
    y = synth.uniform_labels(c["nodes"], c["classes"], seed=2, device=dev)
    train = synth.planetoid_split(c["nodes"])[0].to(dev)
    torch.manual_seed(0)
    model = GCN([c["features"], c["hidden"], c["classes"]]).to(dev)
    opt = gc.FusedAdam(model.parameters(), lr=0.01)

    def cora_step():
        opt.zero_grad(set_to_none=True)
        loss = gc.log_softmax_nll_loss(model(X, adj, log_softmax=False), y, train, scale=1.0 / 140)
        loss.backward()
        opt.step()

    out["cora_like_2layer_train_epoch_ms"] = _time_ms(cora_step, warm=5, iters=20)
    # the same step recorded once as a CUDA graph and replayed (launch-bound workload)
    torch.manual_seed(0)
    model_g = GCN([c["features"], c["hidden"], c["classes"]]).to(dev)
    opt_g = gc.FusedAdam(model_g.parameters(), lr=0.01)
    graphed = gc.GraphedTrainStep(model_g, adj, X, y, opt_g, row_mask=train)
    out["cora_like_2layer_train_epoch_ms_cuda_graph"] = _time_ms(graphed.step, warm=5, iters=50)

    # arxiv-shaped CSR aggregation, F = 128 / 256 (fused bias + ReLU)
    c = synth.CONFIGS["rmat_arxiv"]
    e = synth.rmat_edges(c["scale"], c["nodes"], c["edges"], c["seed"], device=dev)
    adj = gc.normalized_adjacency(synth.symmetrize(e), c["nodes"], symmetric=True)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for F in (128, 256):
        H = synth.normal_features(c["nodes"], F, seed=F, device=dev)
        b = synth.normal_features(1, F, seed=F + 1, device=dev)[0]
        nbytes = 4 * (c["nodes"] + 1) + 8 * adj.nnz + 8 * c["nodes"] * F + 4 * F
        ms_warm = _time_ms(lambda: adj.matmul(H, bias=b, relu=True))
        # cold: L2 flushed (a 256 MiB write) before every launch, kernel timed alone
        ts = []
        for _ in range(5):
            flush.zero_()
            a_ = torch.cuda.Event(enable_timing=True)
            b_ = torch.cuda.Event(enable_timing=True)
            a_.record()
            adj.matmul(H, bias=b, relu=True)
            b_.record()
            torch.cuda.synchronize()
            ts.append(a_.elapsed_time(b_))
        ms_cold = statistics.median(ts)
        from graphcuda_b200 import ops as _ops
        H16 = _ops.to_bf16(H)
        ms16 = _time_ms(lambda: adj.matmul(H16, bias=b, relu=True))
        out[f"arxiv_like_spmm_F{F}_bf16_gathers_ms"] = ms16
        out[f"arxiv_like_spmm_F{F}"] = {
            "ms_l2_warm": ms_warm, "ms_l2_flushed": ms_cold, "alg_bytes": nbytes,
            "gbs_l2_flushed": nbytes / (ms_cold * 1e-3) / 1e9, "frac_hbm_l2_flushed": nbytes / (ms_cold * 1e-3) / 1e9 / peak,
            "gbs_l2_warm": nbytes / (ms_warm * 1e-3) / 1e9,
        }
    # same-box library context: cuSPARSE through torch.sparse.mm on the same matrix (what the reference's
    # spmm_cusparse wrapper calls, src/graphcuda/cuda/spmm_cusparse.cu:105-116, there in COO form)
    try:
        A_csr = torch.sparse_csr_tensor(adj.rowptr.long(), adj.col.long(), adj.val, size=adj.shape)
        Hc = synth.normal_features(c["nodes"], 256, seed=256, device=dev)
        out["arxiv_like_spmm_F256_cusparse_via_torch_ms"] = _time_ms(lambda: torch.sparse.mm(A_csr, Hc))
        del A_csr, Hc
    except Exception as ex:
        out["arxiv_like_spmm_F256_cusparse_via_torch_ms"] = repr(ex)
    # feature transform 169,343 x 128 x 256 on the tensor cores (split-TF32) vs CUDA cores
    Xa = synth.normal_features(c["nodes"], 128, seed=3, device=dev)
    W = synth.reference_init(128, 256, seed=4, device=dev)
    flops = 2.0 * c["nodes"] * 128 * 256
    gbytes = 4.0 * (c["nodes"] * 128 + 128 * 256 + c["nodes"] * 256)
    for prec in ("tf32x3", "tf32", "bf16", "fp32_simt"):
        ms = _time_ms(lambda: gc.gemm(Xa, W, precision=prec))
        out[f"arxiv_like_gemm_{prec}"] = {"ms": ms, "tflops": flops / (ms * 1e-3) / 1e12,
                                          "gbs": gbytes / (ms * 1e-3) / 1e9, "frac_hbm": gbytes / (ms * 1e-3) / 1e9 / peak}
    del Xa, adj, e

    # GEMM operator sweep (matmul1..4 / gemm_cublas all run this engine): uniform(-1, 1) operands
    sweep = {}
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    for (M, N, K) in ((2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192), (1 << 20, 64, 128),
                      (1 << 20, 256, 256)):
        A = torch.rand(M, K, generator=g, device=dev) * 2 - 1
        B = torch.rand(K, N, generator=g, device=dev) * 2 - 1
        fl = 2.0 * M * N * K
        by = 4.0 * (M * K + K * N + M * N)
        row = {}
        for prec in ("tf32x3", "tf32", "bf16"):
            ms = _time_ms(lambda: gc.gemm(A, B, precision=prec), warm=2, iters=5)
            row[prec] = {"ms": ms, "useful_tflops": fl / (ms * 1e-3) / 1e12, "gbs": by / (ms * 1e-3) / 1e9}
        row["bf16"]["includes"] = "the conversion of both fp32 operands to bf16 inside the call"
        # same-box library context: cuBLAS SGEMM through torch.matmul (fp32, TF32 off), what the reference's
        # gemm_cublas wrapper calls (src/graphcuda/cuda/gemm_cublas.cu:37-48)
        torch.backends.cuda.matmul.allow_tf32 = False
        ms = _time_ms(lambda: torch.matmul(A, B), warm=2, iters=5)
        row["cublas_sgemm_via_torch"] = {"ms": ms, "useful_tflops": fl / (ms * 1e-3) / 1e12}
        sweep[f"{M}x{N}x{K}"] = row
        del A, B
    out["gemm_sweep"] = sweep

    # dense-adjacency fused aggregation: N = 32,768, G(n, p = 0.01) + self-loops, normalised, dense fp32 (4.3 GB);
    # Y = relu(A_hat (X W) + b), 512 -> 256
    n4 = 32768
    e4 = synth.erdos_renyi_edges(n4, 0.01, seed=3, device=dev)
    a4 = gc.normalized_adjacency(synth.symmetrize(e4), n4, symmetric=True)
    dense = torch.zeros(n4, n4, device=dev)
    rows4 = torch.repeat_interleave(torch.arange(n4, device=dev), (a4.rowptr[1:] - a4.rowptr[:-1]).long())
    dense[rows4, a4.col.long()] = a4.val
    X4 = synth.normal_features(n4, 512, seed=5, device=dev)
    W4 = synth.reference_init(512, 256, seed=6, device=dev)
    b4 = synth.normal_features(1, 256, seed=7, device=dev)[0] * 0.1
    dadj = gc.DenseAdjacency(dense, symmetric=True)
    fl4 = 2.0 * n4 * 512 * 256 + 2.0 * n4 * n4 * 256
    row = {}
    peaks_tc = {}
    try:
        d_ = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        peaks_tc = {"bf16": float(d_["bf16_tflops"])}
    except Exception:
        pass
    for prec in ("tf32x3", "tf32", "bf16"):
        def fused():
            H = gc.gemm(X4, W4, precision=prec)
            return dadj.matmul(H, bias=b4, relu=True, precision=prec)
        ms = _time_ms(fused, warm=2, iters=5)
        row[prec] = {"ms": ms, "useful_tflops": fl4 / (ms * 1e-3) / 1e12,
                     "adj_gbs": (2.0 if prec == "bf16" else 4.0) * n4 * n4 / (ms * 1e-3) / 1e9}
        if prec == "bf16":
            row[prec]["note"] = "the adjacency's bf16 copy (2.1 GB) is made once and reused; H is converted per call"
            if "bf16" in peaks_tc:
                row[prec]["frac_of_measured_bf16_peak"] = row[prec]["useful_tflops"] / peaks_tc["bf16"]
    # the same layer through the CSR path
    ms = _time_ms(lambda: a4.matmul(gc.gemm(X4, W4), bias=b4, relu=True), warm=2, iters=5)
    row["csr"] = {"ms": ms}
    out["dense_adj_32768_512_256"] = row
    return out


def reference_cuda_same_box(dev, full_graph=None):
    """The reference's own CUDA extension (built unmodified for sm_100 by baseline/build_ref_cuda.py) timed on
    this GPU beside this library on the same inputs: its library wrappers only -- spmm_cusparse (cuSPARSE COO
    SpMM with a cudaMalloc / cudaFree per call, src/graphcuda/cuda/spmm_cusparse.cu:57-119), gemm_cublas
    (gemm_cublas.cu:37-48) and the layer gcn_conv_forward / gcn_conv_backward (gcn.cu:5-52).  Its hand-written
    matmul3 / matmul4 are not launched (they access out of bounds off 128-multiples: matmul3.cu:215-232,
    matmul4.cu:185-201)."""
    import graphcuda_b200 as gc
    from graphcuda_b200 import synth
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import build_ref_cuda
        ext = build_ref_cuda.load()
    except Exception as ex:
        return {"unavailable": f"reference CUDA extension not loadable here: {ex!r}"[:300]}
    out = {"built_from": "src/graphcuda/cuda/*.cu, unmodified, -gencode arch=compute_100,code=sm_100"}

    def layer_case(name, adj, X, W):
        A = adj.to_sparse_coo()
        n, fout = X.size(0), W.size(1)
        dY = synth.normal_features(n, fout, seed=9, device=dev)
        r = {}
        Y, mask = ext.gcn_conv_forward(X, A, W, True)
        ours = gc.GCNConv(W.size(0), fout).to(dev)
        with torch.no_grad():
            ours.weights.copy_(W)
        Xg = X.clone().requires_grad_()
        Yo = ours(Xg, adj)
        r["forward_rel_diff_vs_reference"] = float((Yo - Y).norm() / Y.norm())
        r["reference_spmm_cusparse_ms"] = _time_ms(lambda: ext.spmm_cusparse(A, X), warm=2, iters=5)
        r["ours_spmm_ms"] = _time_ms(lambda: adj.matmul(X), warm=2, iters=5)
        AX = adj.matmul(X)
        r["reference_gemm_cublas_ms"] = _time_ms(lambda: ext.gemm_cublas(AX, W), warm=2, iters=5)
        r["ours_gemm_ms"] = _time_ms(lambda: gc.gemm(AX, W), warm=2, iters=5)

        def ref_layer():
            Y_, m_ = ext.gcn_conv_forward(X, A, W, True)
            ext.gcn_conv_backward(dY, X, A, W, True, m_)

        def our_layer():
            Xg.grad = None
            ours.weights.grad = None
            ours(Xg, adj).backward(dY)

        r["reference_layer_fwd_bwd_ms"] = _time_ms(ref_layer, warm=2, iters=5)
        r["ours_layer_fwd_bwd_ms"] = _time_ms(our_layer, warm=2, iters=5)
        out[name] = r

    try:
        c = synth.CONFIGS["cora_like"]
        e = synth.preferential_attachment_edges(c["nodes"], c["edges"], c["seed"]).to(dev)
        adj = gc.normalized_adjacency(synth.symmetrize(e), c["nodes"], symmetric=True)
        layer_case("cora_like_1433_16", adj, synth.bow_features(c["nodes"], c["features"], 0.0127, seed=1, device=dev),
                   synth.reference_init(c["features"], c["hidden"], seed=4, device=dev))
        c = synth.CONFIGS["rmat_arxiv"]
        e = synth.rmat_edges(c["scale"], c["nodes"], c["edges"], c["seed"], device=dev)
        adj = gc.normalized_adjacency(synth.symmetrize(e), c["nodes"], symmetric=True)
        layer_case("arxiv_like_128_256", adj, synth.normal_features(c["nodes"], 128, seed=3, device=dev),
                   synth.reference_init(128, 256, seed=4, device=dev))
        del adj, e
        if full_graph is not None:
            n = full_graph.shape[0]
            layer_case("products_like_100_256", full_graph, synth.normal_features(n, 100, seed=11, device=dev),
                       synth.reference_init(100, 256, seed=4, device=dev))
    except Exception as ex:
        out["error"] = repr(ex)[:300]
    return out


def run_exchange_probe(args):
    """`--exchange-probe` (under torchrun, N >= 2): times the block exchanges of the partitioned layers by themselves,
    on matrices of the workload's size -- the all-gather of row blocks pulled through symmetric memory against NCCL's
    all_gather_into_tensor, and the rows -> columns transpose as one scatter kernel into the peers' buffers against
    NCCL's all_to_all_single with its pack copy.  One JSON line from rank 0 (max over ranks)."""
    import torch.distributed as dist

    from graphcuda_b200.partition import FeatureShardedGraph, PartitionedGraph
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        raise SystemExit("--exchange-probe needs at least two ranks (torchrun)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    n = workload(args.shrink)["nodes"]
    empty = (torch.zeros(n + 1, dtype=torch.int32, device=dev), torch.empty(0, dtype=torch.int32, device=dev),
             torch.empty(0, dtype=torch.float32, device=dev))
    out = {"probe": "exchange", "n_gpus": world, "nodes": n}

    def timed(fn, iters=5):
        for _ in range(2):
            fn()
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda.synchronize()
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / iters], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for exch in ("auto", "collective"):
        rows_g = PartitionedGraph(*empty, n, rank=rank, world=world, exchange=exch)
        cols_g = FeatureShardedGraph(None, n, rank=rank, world=world, device=dev, exchange=exch)
        name = "peer_memory" if rows_g.symm is not None else "nccl"
        if exch == "auto" and rows_g.symm is None:
            out["peer_memory"] = "symmetric memory unavailable"
            continue
        for F in (256, 48):
            H = torch.randn(rows_g.rows, F, device=dev)

            def gather():
                _, work = rows_g.all_gather_rows_async(H, tag="p")
                if work is not None:
                    work.wait()

            ms = timed(gather)
            recv = (world - 1) * rows_g.part.block * F * 4
            out[f"{name}_all_gather_F{F}"] = {"ms": ms, "GBs_in_per_rank": recv / ms / 1e6}
            ms = timed(lambda: cols_g.rows_to_columns(H, tag="p"))
            sent = (world - 1) * rows_g.part.block * cols_g.slab_width(F) * 4
            out[f"{name}_rows_to_columns_F{F}"] = {"ms": ms, "GBs_out_per_rank": sent / ms / 1e6}
        del rows_g, cols_g
    if rank == 0:
        print(json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def main():
    args = parse()
    if args.exchange_probe:
        return run_exchange_probe(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
