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
    ap.add_argument("--precision", default="fp32", choices=["fp32", "fp32_simt", "tf32x3", "tf32"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-aux", action="store_true", help="skip the auxiliary single-GPU measurements")
    ap.add_argument("--cpu-sample-div", type=int, default=32)
    ap.add_argument("--partition", default="auto", choices=["auto", "features", "rows"],
                    help="multi-GPU scheme: aggregation sharded over feature columns (all-to-all) or adjacency rows "
                         "(all-gather); auto = rows up to 4 GPUs, features from 8 (measured cross-over)")
    ap.add_argument("--profile-warmup", action="store_true",
                    help="honour --warmup below 3 (profiler captures only; such a run is not a benchmark)")
    return ap.parse_args()


def workload(shrink: int):
    from graphcuda_b200 import synth
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
def cpu_reference_epoch_ms(cfg, sample_div: int, steps: int, warmup: int):
    """The reference's own CPU path (its gcn.cpp compiled for CPU when present,
    else the oracle restatement of it) on an R-MAT sample 1/sample_div the size,
    time scaled by sample_div (work is linear in nodes and edges)."""
    from graphcuda_b200 import synth
    from oracle import gcn_oracle as O
    from oracle import ref_loader
    # all the host threads this process may use (a launcher may have exported OMP_NUM_THREADS=1 for its workers)
    avail = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(max(1, avail))
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

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    ms = (time.perf_counter() - t0) * 1e3 / max(steps, 1)
    sample = (f"R-MAT sample 1/{sample_div} of the workload ({n} nodes, {m} undirected edges, same degree, "
              f"same 3-layer model, fwd+loss+bwd+Adam), {steps} timed steps after {warmup} warm-up, "
              f"time x{sample_div}")
    return ms * sample_div, kind, torch.get_num_threads(), sample


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = workload(args.shrink)
    # a bounded run: the sample is sized so that one step is a few seconds of CPU work
    steps = max(1, min(args.steps, 5))
    warm = max(1, min(args.warmup, 2))
    ms, kind, cores, sample = cpu_reference_epoch_ms(cfg, args.cpu_sample_div, steps, warm)
    line = {
        "impl": "reference", "metric": METRIC, "value": ms, "unit": "ms", "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": config_dict(cfg, args, 1),
        "cpu_baseline": {"value": ms, "unit": "ms", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def config_dict(cfg, args, world):
    return {
        "workload": "rmat_products: 3-layer GCN 100-256-256-47 train step, R-MAT a=.57 b=.19 c=.19 d=.05",
        "nodes": cfg["nodes"], "undirected_edges": cfg["edges"], "nnz": 2 * cfg["edges"] + cfg["nodes"],
        "dims": DIMS, "optimizer": "Adam lr=0.01", "loss": "nll over all nodes",
        "parallelism": (f"{args.partition}-sharded x{world}" if world > 1 else "single GPU"),
        "precision": args.precision, "l2": "inputs larger than L2 (no flush needed)",
        "shrink": args.shrink,
    }


# ---------------------------------------------------------------- our arm
def run_ours(args):
    import torch.distributed as dist

    import graphcuda_b200 as gc
    from graphcuda_b200 import _lib, adjacency, ops, synth
    from graphcuda_b200.models import GCN
    from graphcuda_b200.partition import DistGCN, FeatureShardedGraph, PartitionedGraph, RowPartition

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.partition == "auto":
        args.partition = "features" if world >= 8 else "rows"
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
    X_full_host = None
    part = None
    if world == 1:
        X = synth.normal_features(n, DIMS[0], seed=11, device=dev)
        y = synth.uniform_labels(n, DIMS[-1], seed=12, device=dev)
        torch.manual_seed(0)
        model = GCN(DIMS, precision=args.precision).to(dev)
        rows = n
    else:
        if args.partition == "rows":
            part = PartitionedGraph(adj.rowptr, adj.col, adj.val, n, rank=rank, world=world)
        else:
            part = FeatureShardedGraph(adj, n, rank=rank, world=world)
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
    for _ in range(args.steps):
        loss = step(X, y, X_gathered)
    e1.record()
    barrier()
    timer.active = False
    launches = L.gc_launch_count() - launches0
    ms_step = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    clocks = sampler.stop() if rank == 0 else None
    final_loss = float(loss.item())

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
            Xg = part.prepare_constant(Xd) if world > 1 else None
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
        # dram__bytes_read.sum + dram__bytes_write.sum of the F = 256 launch (pieces + finalize kernels), captured
        # with ncu on the half-size graph and scaled by the non-zeros (profiles/spmm_pieces_kernel_rmat_products.md);
        # the compulsory bytes of that launch are 6.04e9
        "traffic": 21.7e9 if (args.shrink == 1 and world == 1) else None,
        "traffic_note": "bytes per F=256 launch at full size on 1 GPU; compulsory 6.04e9",
    }

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
        "spmm_gbs": achieved, "spmm_pct_hbm_peak": 100.0 * achieved / peak,
    }

    if rank == 0 and world == 1 and not args.no_aux:
        try:
            line["aux"] = aux_measurements(dev, args)
            # the script's test(): no-grad forward of the same model + fused argmax / accuracy counts
            line["aux"]["rmat_products_eval_forward_argmax_ms"] = _time_ms(lambda: model.evaluate(X, adj, y), warm=2,
                                                                          iters=5)
        except Exception as ex:  # auxiliary numbers never take the headline down
            line["aux"] = {"error": repr(ex)}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        ms, kind, cores, sample = cpu_reference_epoch_ms(cfg, args.cpu_sample_div, 2, 1)
        line["cpu_baseline"] = {"value": ms, "unit": "ms", "cores": cores, "kind": kind, "sample": sample}
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
    for prec in ("tf32x3", "tf32", "fp32_simt"):
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
        for prec in ("tf32x3", "tf32"):
            ms = _time_ms(lambda: gc.gemm(A, B, precision=prec), warm=2, iters=5)
            row[prec] = {"ms": ms, "useful_tflops": fl / (ms * 1e-3) / 1e12, "gbs": by / (ms * 1e-3) / 1e9}
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
    for prec in ("tf32x3", "tf32"):
        def fused():
            H = gc.gemm(X4, W4, precision=prec)
            return dadj.matmul(H, bias=b4, relu=True, precision=prec)
        ms = _time_ms(fused, warm=2, iters=5)
        row[prec] = {"ms": ms, "useful_tflops": fl4 / (ms * 1e-3) / 1e12,
                     "adj_gbs": 4.0 * n4 * n4 / (ms * 1e-3) / 1e9}
    # the same layer through the CSR path
    ms = _time_ms(lambda: a4.matmul(gc.gemm(X4, W4), bias=b4, relu=True), warm=2, iters=5)
    row["csr"] = {"ms": ms}
    out["dense_adj_32768_512_256"] = row
    return out


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
