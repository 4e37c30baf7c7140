#!/usr/bin/env python
"""Benchmark of the fused GNN sparse-kernel path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload C1..C5] [--impl reference]

One "step" is one training epoch of the workload's model on its synthetic graph:
forward, loss, backward and Adam update over the whole graph (the reference's epoch,
script/train/train_gatconv_our.py:184-200).  Prints ONE JSON line (rank 0).

Default workload: C5, the 3-layer GAT (4x128, 4x128, 1x47) on the R-MAT graph with
2,449,029 nodes and ~124 M directed edges — the configuration the 1/2/4/8-GPU metric
is quoted on; it fits one GPU, so the same workload is timed at every N (strong
scaling: destination-row blocks over the ranks, exchange of the referenced rows).

The line's extra records (single GPU, default workload):
  roofline       the HBM-bound entry point with the largest time inside the timed region:
                 `achieved` = measured DRAM bytes per launch (profiles/traffic.json, one ncu
                 capture) / CUDA-event time, `frac` = achieved / measured copy bandwidth;
                 the figure from algorithmic bytes (every gathered row counted once per
                 edge, no cache reuse) is kept beside it as `*_algorithmic`;
  models         the other four configurations, run after the timed workload in the same
                 process: eager epoch, epoch replayed as a CUDA graph, sum of kernel time,
                 dominant entry point and what bounds it;
  cpu_baseline   the reference's CPU formulation on a bounded sample, at two sample sizes,
                 extrapolated by edge count (flagged as such);
  gpu_reference  the reference's own CUDA operators (compiled unmodified into oracle/_ref)
                 timed per operator next to this library's on the same inputs.
With N > 1: `per_rank` (rows, edges, halo rows, rows sent, entry-point and push time of every
rank), the NVLink bytes and GB/s of the `gnn_halo_push[width]` entries, and the DRAM capture of
the whole graph scaled to the rank's block by algorithmic bytes.  `--timeline PATH` writes one
timed step of rank 0 as a list of library calls (start and duration on the device's clock).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402
import torch.nn.functional as F  # noqa: E402


def mean_cross_entropy(logits, labels):
    """F.cross_entropy(reduction="mean") written as log_softmax + gather: the framework's fused
    NLL reduction takes 2.6 ms for 2.4 M rows, this form 0.3 ms, same value."""
    return -F.log_softmax(logits, dim=1).gather(1, labels.view(-1, 1)).mean()

METRIC = "fwd_bwd_epoch_ms"
UNIT = "ms/epoch"

# (nodes, edges incl. self-loops) the generators produce for seed 0 at full size; the CPU legs
# extrapolate to these without building the full graph
FULL_SIZES = {"C1": (2708, 13264), "C2": (232965, 113696831), "C3": (32768, 655360),
              "C4": (19717, 108365), "C5": (2449029, 126053365)}
# gathered operand fits in the 126 MB L2: those epochs are launch / L2 bound, not HBM bound
L2_RESIDENT = {"C1", "C3", "C4"}

WORKLOADS = {
    "C1": dict(kind="gat", desc="GAT 2-layer, 2,708 nodes / 10,556+2,708 edges, in 1433, 8x8 -> 1x7",
               n=2708, edges=10556, in_dim=1433, hidden=[8], heads=[8], classes=7),
    "C2": dict(kind="gat", desc="GAT 2-layer, Chung-Lu power-law 232,965 nodes / ~114.6M edges, in 602, 4x64 -> 1x41",
               n=232965, mean_deg=492, max_deg=21600, in_dim=602, hidden=[64], heads=[4], classes=41),
    "C3": dict(kind="edgeconv", desc="DGCNN 4 EdgeConv layers (64,64,128,256), 32 clouds x 1024 points, kNN k=20, 40 classes",
               batch=32, points=1024, k=20, dims=[64, 64, 128, 256], classes=40),
    "C4": dict(kind="gmm", desc="MoNet 2 GMMConv layers, 19,717 nodes / 88,648+19,717 edges, in 500, K=3, D=2, hidden 16, 3 classes",
               n=19717, edges=88648, in_dim=500, hidden=16, classes=3, kernels=3, dim=2),
    "C5": dict(kind="gat", desc="GAT 3-layer, R-MAT 2,449,029 nodes / ~124M directed edges, in 100, 4x128 -> 4x128 -> 1x47",
               n=2449029, rmat_pairs=83_400_000, in_dim=100, hidden=[128, 128], heads=[4, 4], classes=47),
}


# ----------------------------------------------------------------------------------------
# helpers
# ----------------------------------------------------------------------------------------

def env_int(name, default):
    return int(os.environ.get(name, default))


class ClockSampler:
    """nvidia-smi clock / throttle-reason sampling during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.path = gpu_index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
                except ValueError:
                    continue
                for nm, v in zip(names, f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(nm)
        finally:
            try:
                os.unlink(self.path)
            except OSError:
                pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "power_w_max": max(power), "samples": len(sm)}


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def algorithmic_bytes(name: str, n: int, e: int, H: int, Fw: int, D: int = 0) -> float:
    """Bytes one call of an entry point must move when every gathered row is read once
    per edge and every per-node array once (no cache reuse)."""
    HF = H * Fw
    if name == "gnn_gat_fwd":
        return 4.0 * e * (1 + H + HF) + 4.0 * n * (1 + 3 * H + HF)
    if name == "gnn_gat_bwd_row":
        return 4.0 * e * (1 + H + HF) + 4.0 * n * (1 + HF + 3 * H)
    if name == "gnn_gat_bwd_col":
        return 4.0 * e * (1 + 3 * H + HF) + 4.0 * n * (1 + HF + 3 * H)
    if name == "gnn_gat_bwd_col_edges":  # the column pass plus the E x H store of the edge gradients
        return 4.0 * e * (1 + 4 * H + HF) + 4.0 * n * (1 + HF + 3 * H)
    if name == "gnn_gat_bwd_pack":
        return 4.0 * n * (2 * HF + 7 * H)
    if name == "gnn_gat_bwd_pack_elu":  # also writes the pre-activation gradient
        return 4.0 * n * (3 * HF + 7 * H)
    if name == "gnn_gat_bwd_row_sum":
        return 4.0 * e * (1 + H) + 4.0 * n * (1 + H)
    if name == "gnn_edgeconv_fwd":
        return 4.0 * e * (1 + Fw) + 12.0 * n * Fw
    if name == "gnn_edgeconv_bwd":
        return 16.0 * n * Fw
    if name == "gnn_gmm_fwd":
        return 4.0 * e * (1 + D + HF) + 4.0 * n * (1 + HF)
    if name == "gnn_mhsddmm":
        return 4.0 * e * (1 + HF + H) + 4.0 * n * (1 + HF)
    if name == "gnn_gat_scores_fwd":
        return 4.0 * n * (HF + 2 * H)
    if name == "gnn_gat_scores_bwd":
        return 4.0 * n * (3 * HF + 2 * H)
    return 0.0


class BytesLedger:
    """Wraps _capi.call so that every timed entry-point call is stored with the
    algorithmic bytes of its arguments, keyed by entry point and shape ("name[HxF]")."""

    def __init__(self):
        from ae_mlsys_gnn_b200 import _capi

        self.capi = _capi
        self.timer = _capi.CallTimer(with_events=True)
        self.bytes: list[float] = []
        self.keys: list[str] = []
        self.link_bytes: dict[str, float] = {}  # bytes stored into other GPUs' memory, per push key
        self._orig = _capi.call

    def __enter__(self):
        capi, ledger = self.capi, self
        capi.install_timer(self.timer)
        orig = self._orig

        def call(name, *args):
            b, shape = ledger._bytes_of(name, args)
            key = f"{name}[{shape}]" if shape else name
            ledger.bytes.append(b)
            ledger.keys.append(key)
            if name == "gnn_halo_push":  # (x, row_floats, send_idx, send_off[world+1], dst, world, ...)
                ledger.link_bytes[key] = ledger.link_bytes.get(key, 0.0) + 4.0 * args[1] * args[3][args[5]]
            orig(name, *args)

        capi.call = call  # operator modules look the function up as capi.call at call time
        return self

    def __exit__(self, *exc):
        self.capi.call = self._orig
        self.capi.install_timer(None)

    @staticmethod
    def _bytes_of(name, a):
        if name in ("gnn_gat_fwd", "gnn_gat_fwd_part", "gnn_gat_fwd_act"):
            return algorithmic_bytes("gnn_gat_fwd", a[2], a[3], a[7], a[8]), f"{a[7]}x{a[8]}"
        if name == "gnn_gat_bwd_row":
            return algorithmic_bytes(name, a[2], a[3], a[10], a[11]), f"{a[10]}x{a[11]}"
        if name in ("gnn_gat_bwd_col", "gnn_gat_bwd_col_part"):
            return algorithmic_bytes("gnn_gat_bwd_col", a[2], a[3], a[8], a[9]), f"{a[8]}x{a[9]}"
        if name == "gnn_gat_bwd_col_edges":
            return (algorithmic_bytes(name if a[13] else "gnn_gat_bwd_col", a[2], a[3], a[8], a[9]),
                    f"{a[8]}x{a[9]}")
        if name in ("gnn_gat_bwd_pack", "gnn_gat_bwd_pack_elu"):
            return algorithmic_bytes(name, a[0], 0, a[6], a[7]), f"{a[6]}x{a[7]}"
        if name == "gnn_gat_bwd_row_sum":
            return algorithmic_bytes(name, a[2], a[3], a[5], 1), f"{a[5]}"
        if name == "gnn_edgeconv_fwd":
            return algorithmic_bytes(name, a[4], a[4] * a[0], 1, a[5]), f"k{a[0]}x{a[5]}"
        if name == "gnn_edgeconv_bwd":
            return algorithmic_bytes(name, a[2], 0, 1, a[4]), f"{a[4]}"
        if name == "gnn_gmm_fwd":
            return algorithmic_bytes(name, a[2], a[3], a[9], a[11], a[10]), f"{a[9]}x{a[11]}"
        if name == "gnn_mhsddmm":
            return algorithmic_bytes(name, a[2], a[3], a[6], a[7]), f"{a[6]}x{a[7]}"
        if name == "gnn_gat_scores_fwd":
            return algorithmic_bytes(name, a[3], 0, a[4], a[5]), f"{a[4]}x{a[5]}"
        if name == "gnn_gat_scores_bwd":
            return algorithmic_bytes(name, a[5], 0, a[6], a[7]), f"{a[6]}x{a[7]}"
        if name in ("gnn_gemm_tf32x3", "gnn_gemm_tf32x3_scores"):
            return 0.0, f"{a[4]}x{a[5]}x{a[6]}"
        if name == "gnn_gemm_tf32x3_tn":
            return 0.0, f"{a[3]}x{a[4]}x{a[5]}"
        if name == "gnn_halo_push":
            return 0.0, f"{a[1]}"
        return 0.0, ""

    def summary(self):
        per = {}
        for (name, s, t), b, key in zip(self.timer.records, self.bytes, self.keys):
            d = per.setdefault(key, {"ms": 0.0, "bytes": 0.0, "calls": 0})
            d["ms"] += s.elapsed_time(t)
            d["bytes"] += b
            d["calls"] += 1
        return per


def count_launches(counts: dict, csr2csc_launches: int) -> int:
    from ae_mlsys_gnn_b200._capi import KERNELS_PER_CALL

    total = 0
    for name, c in counts.items():
        k = KERNELS_PER_CALL.get(name)
        total += c * (csr2csc_launches if k is None else k)
    return total


def csr2csc_launch_count(n_cols: int, nnz: int) -> int:
    bits = 1
    while bits < 31 and (1 << bits) < n_cols:
        bits += 1
    passes = (bits + 7) // 8
    tiles = max(1, (nnz + 4095) // 4096)
    scan = 3 if (256 * tiles + 4095) // 4096 > 1 else 1
    return passes * (2 + scan) + 3


# ----------------------------------------------------------------------------------------
# workload construction (device-side, seeded; nothing here is timed)
# ----------------------------------------------------------------------------------------

def build_inputs(wl: dict, device, seed: int, scale: float = 1.0):
    """Returns a dict with the graph / inputs / labels of a workload on `device`.
    ``scale`` < 1 builds the same generator at 1/scale fewer nodes and edges (used for
    the bounded CPU sample)."""
    from ae_mlsys_gnn_b200 import graphs as G

    kind = wl["kind"]
    if kind == "edgeconv":
        batch = max(1, int(round(wl["batch"] * scale)))
        pts = G.unit_ball_points(batch, wl["points"], seed, device)
        src = G.knn_sources(pts, wl["k"])
        labels = G.uniform_labels(batch, wl["classes"], seed + 2, device)
        return dict(points=pts, src=src, labels=labels, n=batch * wl["points"], nnz=int(src.numel()))
    n = max(64, int(round(wl["n"] * scale)))
    if "rmat_pairs" in wl:
        g = G.rmat_graph(n, int(wl["rmat_pairs"] * scale), seed=seed, device=device)
    elif "mean_deg" in wl:
        # a scaled-down sample keeps the degree law but cannot keep the degrees themselves
        mean = min(wl["mean_deg"], n / 32)
        g = G.chung_lu_graph(n, mean, min(n / 2, mean * wl["max_deg"] / wl["mean_deg"]), seed=seed,
                             device=device)
    else:
        g = G.uniform_graph(n, int(wl["edges"] * scale), seed=seed, device=device)
    if wl["name"] == "C1":
        x = G.bag_of_words(n, wl["in_dim"], 0.0127, seed + 1, device)
    elif kind == "gmm":
        x = G.sparse_l1_features(n, wl["in_dim"], 0.1, seed + 1, device)
    else:
        x = G.normal_features(n, wl["in_dim"], seed + 1, device)
    labels = G.uniform_labels(n, wl["classes"], seed + 2, device)
    out = dict(graph=g, x=x, labels=labels, n=n, nnz=g.nnz)
    if kind == "gmm":
        out["pseudo"] = G.degree_pseudo(g)
    return out


def make_model(wl: dict, cpu: bool = False):
    if cpu:
        from oracle import cpu_models as M
        if wl["kind"] == "gat":
            return M.CpuGAT(wl["in_dim"], wl["hidden"], wl["heads"], wl["classes"], 1)
        if wl["kind"] == "edgeconv":
            return M.CpuDGCNN(wl["k"], wl["dims"], wl["classes"])
        return M.CpuMoNet(wl["in_dim"], wl["hidden"], wl["classes"], 2, wl["dim"], wl["kernels"])
    from ae_mlsys_gnn_b200 import models as M
    if wl["kind"] == "gat":
        return M.GAT(wl["in_dim"], wl["hidden"], wl["heads"], wl["classes"], 1)
    if wl["kind"] == "edgeconv":
        return M.DGCNN(wl["k"], wl["dims"], wl["classes"])
    return M.MoNet(wl["in_dim"], wl["hidden"], wl["classes"], 2, wl["dim"], wl["kernels"])


# ----------------------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle's DGL-style CPU models on a bounded sample
# ----------------------------------------------------------------------------------------

def cpu_sample_scale(wl: dict) -> float:
    return {"C1": 1.0, "C2": 1.0 / 32, "C3": 1.0 / 8, "C4": 1.0, "C5": 1.0 / 256}[wl["name"]]


def _time_cpu_epochs(wl: dict, scale: float, steps: int, warmup: int, seed: int):
    """(ms per epoch, nodes, edges) of the CPU model on the generator at `scale`."""
    d = build_inputs(wl, "cpu", seed, scale)
    torch.manual_seed(seed)
    model = make_model(wl, cpu=True)
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)

    def step():
        if wl["kind"] == "gat":
            out = model(d["graph"].row_ptr, d["graph"].col_ind, d["x"])
        elif wl["kind"] == "edgeconv":
            out = model(d["points"], d["src"])
        else:
            out = model(d["graph"].row_ptr, d["graph"].col_ind, d["x"], d["pseudo"])
        loss = F.cross_entropy(out, d["labels"])
        opt.zero_grad()
        loss.backward()
        opt.step()
        return loss.item()

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    return (time.perf_counter() - t0) * 1e3 / max(1, steps), d["n"], d["nnz"]


def run_cpu_epochs(wl: dict, steps: int, warmup: int, seed: int):
    """Times the CPU model on a bounded sample of the workload and extrapolates to the full
    workload by edge count.  A second, four times larger sample (two epochs) is timed as well
    so that the linearity the extrapolation assumes can be read off the record.  Returns the
    `cpu_baseline` record."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    scale = cpu_sample_scale(wl)
    full_nnz = FULL_SIZES[wl["name"]][1]
    ms, n, nnz = _time_cpu_epochs(wl, scale, steps, warmup, seed)
    rec = {"unit": UNIT, "cores": cores, "kind": "port", "extrapolated": scale < 1.0,
           "sample_ms": ms, "sample_nodes": n, "sample_edges": nnz, "factor": full_nnz / nnz if scale < 1.0 else 1.0}
    value = ms * rec["factor"]
    text = (f"{wl['name']} generator at scale {scale:g}: {n} nodes / {nnz} edges, full model "
            f"fwd+loss+bwd+Adam in PyTorch-CPU fp32 (DGL-style index_select/index_add restatement), "
            f"{ms:.1f} ms per epoch measured")
    if scale < 1.0:
        ms4, n4, nnz4 = _time_cpu_epochs(wl, min(1.0, 4 * scale), 2, 1, seed)
        rec.update(sample4x_ms=ms4, sample4x_edges=nnz4, sample4x_extrapolated_ms=ms4 * full_nnz / nnz4)
        text += (f", x{rec['factor']:.1f} (edge ratio to the full {full_nnz} edges); a sample of {nnz4} edges "
                 f"took {ms4:.1f} ms, which extrapolates to {ms4 * full_nnz / nnz4:.0f} ms")
    rec["value"] = value
    rec["sample"] = text
    return rec


def config_of(wl: dict, world: int, exchange: str | None = None) -> dict:
    """The `config` record, identical in the library's arm and in the reference arm."""
    n, nnz = FULL_SIZES[wl["name"]]
    exchange = exchange or os.environ.get("GNN_B200_EXCHANGE", "peer")
    return {"workload": f"{wl['name']}: {wl['desc']}", "nodes": n, "edges": nnz,
            "parallelism": (f"row-block x{world}, {exchange} exchange" if world > 1 else "single GPU"),
            "l2": ("flushed between steps (256 MB write)" if wl["name"] in L2_RESIDENT
                   else "inputs exceed L2 (126 MB)"),
            "seed": 0}


def reference_arm(args, wl):
    rank = env_int("RANK", 0)
    if rank != 0:
        return
    rec = run_cpu_epochs(wl, args.steps, args.warmup, args.seed)
    ms = rec["value"]
    line = {
        "impl": "reference", "metric": METRIC, "value": ms, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_of(wl, args.gpus), "extrapolated": rec["extrapolated"],
        "cpu_baseline": rec,
        "e2e": {"value": ms, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------
# the reference's own CUDA operators, timed next to this library's on the same inputs
# ----------------------------------------------------------------------------------------

def _median_ms(fn, iters=5, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for a, b in ev:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    t = sorted(a.elapsed_time(b) for a, b in ev)
    return t[len(t) // 2]


def gpu_reference_leg(dev, seed: int):
    """Per-operator times of the reference's CUDA kernels (oracle/_ref, built unmodified from
    the reference sources) and of this library on the same inputs.  Shapes are those where
    reading the reference kernels shows no out-of-bounds access (F a multiple of 32; below
    2^24 edges for its float-typed csr2csc permutation): R-MAT 400,000 nodes / ~15.6 M edges
    with 4x128, 4x64 and 1x64 features; EdgeConv 64 clouds x 1,024 points, k = 20, 64 wide.
    The 47-wide output layer is left out (fused_gat_SM.cu:279 reads past the row).  For
    F > 64 and degrees above 32 the reference forward shares a staging buffer between warps
    without a block barrier: its values are not checked here, only its time is taken."""
    try:
        from oracle import build_ref
    except Exception as e:  # the checker is not shipped
        return {"unavailable": f"oracle package missing: {e}"}
    need = ("fused_gat_SM", "fused_edgeconv", "csrtocsc")
    if not all(build_ref.available(m) for m in need):
        return {"unavailable": "oracle/_ref modules not built (python -m oracle.build_ref)"}
    from ae_mlsys_gnn_b200 import graphs as G
    from ae_mlsys_gnn_b200.operators import fused_gat as GAT
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc
    from ae_mlsys_gnn_b200.operators.fused_edgeconv import edgeconv_forward

    gat, ec, tr = (build_ref.load_module(m) for m in need)
    out = {"graph": "R-MAT 400,000 nodes", "ops": {}}
    g = G.rmat_graph(400_000, int(400_000 * 50 * 0.45), seed=seed, device=dev)
    out["graph"] += f" / {g.nnz} edges"
    rp, ci = g.row_ptr, g.col_ind
    cp, ri, pm = csr2csc(rp, ci)
    pos = GAT.invert_permutation(pm)
    gen = torch.Generator(device=dev).manual_seed(seed)

    def rec(name, ref_fn, own_fn):
        r, o = _median_ms(ref_fn), _median_ms(own_fn)
        out["ops"][name] = {"reference_ms": r, "b200_ms": o, "speedup": r / o if o > 0 else None}

    if g.nnz < (1 << 24):
        vals = torch.arange(g.nnz, dtype=torch.float32, device=dev)
        rec("csr2csc", lambda: tr.csr2csc(rp, ci, vals), lambda: csr2csc(rp, ci))
    for H, Fw in ((4, 128), (4, 64), (1, 64)):
        ar = torch.randn(g.n, H, device=dev, generator=gen)
        ac = torch.randn(g.n, H, device=dev, generator=gen)
        x = torch.randn(g.n, H, Fw, device=dev, generator=gen)
        go = torch.randn(g.n, H, Fw, device=dev, generator=gen)
        o, m, s = GAT.gat_forward(ar, ac, rp, ci, 0.2, x)
        rec(f"gat_forward[{H}x{Fw}]", lambda: gat.gat_forward(ar, ac, rp, ci, 0.2, x),
            lambda: GAT.gat_forward(ar, ac, rp, ci, 0.2, x))
        rec(f"gat_backward[{H}x{Fw}]", lambda: gat.gat_backward(0.2, rp, ci, cp, ri, m, s, x, ar, ac, go),
            lambda: GAT.gat_backward_with_output(0.2, rp, ci, cp, ri, pos, m, s, x, ar, ac, o, go))
        out["ops"][f"gat_backward[{H}x{Fw}]"]["b200_two_pass_ms"] = _median_ms(
            lambda: GAT.gat_backward(0.2, rp, ci, cp, ri, m, s, x, ar, ac, go))
    n, k, Fw = 64 * 1024, 20, 64
    src = torch.randint(0, n, (n * k,), device=dev, dtype=torch.int32, generator=gen)
    hs = torch.randn(n, Fw, device=dev, generator=gen)
    hd = torch.randn(n, Fw, device=dev, generator=gen)
    rec(f"edgeconv_forward[64x1024,k{k},{Fw}]", lambda: ec.edgeconv_forward(k, src, hs, hd),
        lambda: edgeconv_forward(k, src, hs, hd))
    return out


# ----------------------------------------------------------------------------------------
# one workload on the GPU(s)
# ----------------------------------------------------------------------------------------

def traffic_from_profile(key: str, workload: str, launch_bytes: float | None = None):
    """DRAM bytes per launch measured once with ncu on the whole graph (profiles/traffic.json), or
    None.  ``launch_bytes``: algorithmic bytes of the launch in question; when the capture records the
    algorithmic bytes of the captured launch and they differ (a rank's block of a partitioned run),
    the measured traffic is scaled by their ratio, i.e. the captured DRAM-to-algorithmic ratio is
    assumed to carry over."""
    try:
        t = json.load(open(os.path.join(ROOT, "profiles", "traffic.json"))).get(workload, {})
        dram = t.get(key)
        full = t.get("_algorithmic_bytes", {}).get(key)
        if dram and launch_bytes and full and abs(launch_bytes - full) > 0.02 * full:
            return dram * launch_bytes / full
        return dram
    except Exception:
        return None


def release_device_memory():
    from ae_mlsys_gnn_b200 import _capi
    from ae_mlsys_gnn_b200.operators import fused_gat

    _capi._workspaces.clear()
    fused_gat._CSR_POS.clear()
    fused_gat._CSC_PERM.clear()
    torch.cuda.empty_cache()


class Workload:
    """Inputs, model, optimizer and the step function of one configuration."""

    def __init__(self, wl, dev, seed, world=1, rank=0, capturable=False):
        from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc

        self.wl, self.dev, self.world, self.rank = wl, dev, world, rank
        self.exchange = None
        d = self.d = build_inputs(wl, dev, seed)
        if (d["n"], d["nnz"]) != FULL_SIZES[wl["name"]] and seed == 0:
            raise SystemExit(f"{wl['name']}: generator produced {d['n']} nodes / {d['nnz']} edges, "
                             f"FULL_SIZES says {FULL_SIZES[wl['name']]}")
        self.n, self.nnz = d["n"], d["nnz"]
        torch.manual_seed(seed)
        self.part = None
        self.setup_ms = {}
        kind = wl["kind"]
        if kind in ("gat", "gmm"):
            g = d["graph"]
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            csr2csc(g.row_ptr, g.col_ind)  # first call sizes the workspace
            a.record()
            self.col_ptr, self.row_ind, self.permute = csr2csc(g.row_ptr, g.col_ind)
            b.record()
            torch.cuda.synchronize()
            self.setup_ms["csr2csc"] = a.elapsed_time(b)
            if rank == 0:
                self.setup_ms["coo_to_csr"] = self._time_graph_build(g, seed)
        if kind == "gat" and world > 1:
            self._partition()
        else:
            self.model = make_model(wl).to(dev)
        self.opt = torch.optim.Adam(self.model.parameters(), lr=1e-3, capturable=capturable)
        torch.cuda.empty_cache()

    @staticmethod
    def _time_graph_build(g, seed):
        """Device time of building this CSR from its shuffled edge list (sort by (dst, src), dedup,
        self-loops): the step the reference's scripts do on the host.  The result is compared
        with the graph in use, bit for bit."""
        from ae_mlsys_gnn_b200.operators.graph_build import coo_to_csr

        dev = g.row_ptr.device
        rp = g.row_ptr.long()
        dst = torch.repeat_interleave(torch.arange(g.n, device=dev, dtype=torch.int32), rp[1:] - rp[:-1])
        perm = torch.randperm(g.nnz, device=dev, generator=torch.Generator(device=dev).manual_seed(seed))
        dst, src = dst[perm].contiguous(), g.col_ind[perm].contiguous()
        del perm, rp
        coo_to_csr(dst[:1024], src[:1024], g.n, True)  # loads the kernels
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        rp2, ci2 = coo_to_csr(dst, src, g.n, True)
        b.record()
        torch.cuda.synchronize()
        if not (torch.equal(rp2, g.row_ptr) and torch.equal(ci2, g.col_ind)):
            raise SystemExit("graph construction on the device does not reproduce the workload's CSR")
        return a.elapsed_time(b)

    def _partition(self):
        wl, d, dev = self.wl, self.d, self.dev
        g = d["graph"]
        scheme = os.environ.get("GNN_B200_EXCHANGE", "peer")
        if scheme == "gather":
            from ae_mlsys_gnn_b200.partition import PartitionedGAT, build_partition

            self.exchange = scheme
            self.part = build_partition(g.row_ptr, g.col_ind, self.col_ptr, self.row_ind, self.rank, self.world)
            self.model = PartitionedGAT(wl["in_dim"], wl["hidden"], wl["heads"], wl["classes"], 1).to(dev)
        else:
            from ae_mlsys_gnn_b200.halo import HaloGAT, build_halo_partition

            if scheme == "peer":  # stores into the peers' memory need working IPC mappings on this node
                from ae_mlsys_gnn_b200 import peer

                if not peer.probe(dev):
                    scheme = "nccl"
            self.exchange = scheme
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            self.part = build_halo_partition(g.row_ptr, g.col_ind, self.col_ptr, self.row_ind, self.rank,
                                             self.world)
            torch.cuda.synchronize()
            self.setup_ms["halo_partition"] = (time.perf_counter() - t0) * 1e3
            self.model = HaloGAT(wl["in_dim"], wl["hidden"], wl["heads"], wl["classes"], 1,
                                 exchange=scheme).to(dev)
        d["x_l"] = self.part.pad_rows(self.part.local_slice(d["x"]))
        d["y_l"] = self.part.local_slice(d["labels"]).contiguous()
        del d["x"]
        self.col_ptr = self.row_ind = self.permute = None
        d["graph"] = None

    def step(self):
        wl, d, model, opt = self.wl, self.d, self.model, self.opt
        if self.part is not None:
            out = model(self.part, d["x_l"])
            loss = model.loss(self.part, out, d["y_l"])
            opt.zero_grad(set_to_none=True)
            loss.backward()
            model.all_reduce_grads(self.world)
        else:
            if wl["kind"] == "gat":
                g = d["graph"]
                out = model(g.row_ptr, g.col_ind, self.col_ptr, self.row_ind, d["x"])
            elif wl["kind"] == "edgeconv":
                out = model(d["points"], d["src"])
            else:
                g = d["graph"]
                out = model(g.row_ptr, g.col_ind, self.col_ptr, self.row_ind, self.permute, d["x"], d["pseudo"])
            loss = mean_cross_entropy(out, d["labels"])
            opt.zero_grad(set_to_none=True)
            loss.backward()
        opt.step()
        return loss


def barrier(world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def timed_epochs(w: Workload, steps: int, warmup: int, sampler=None, timeline_path=None):
    """Warm-up, then `steps` epochs bracketed by barrier + synchronize, one CUDA-event pair per
    step; small workloads get an L2 flush (256 MB write) between steps, outside the pairs.
    Returns (ms per step as the max over ranks, per-entry-point summary, launch counts, clocks)."""
    from ae_mlsys_gnn_b200.operators import dense

    dev, world = w.dev, w.world
    flush = w.wl["name"] in L2_RESIDENT
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if flush else None
    for _ in range(warmup):
        w.step()
    barrier(world)
    if sampler is not None:
        sampler.start()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    with BytesLedger() as ledger:
        barrier(world)
        for a, b in ev:
            if flush:
                flush_buf.fill_(1)
            a.record()
            w.step()
            b.record()
        barrier(world)
    clocks = sampler.stop() if sampler is not None else None
    dense.check_status(dev)  # a GEMM whose bounded wait expired must not pass as a result
    total_ms = torch.tensor([sum(a.elapsed_time(b) for a, b in ev)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
    per = ledger.summary()
    if timeline_path:  # the last timed step as a list of library calls on the device's clock
        a0, b0 = ev[-1]
        span = a0.elapsed_time(b0)
        calls = []
        for (name, s, t), key in zip(ledger.timer.records, ledger.keys):
            at = a0.elapsed_time(s)
            if 0.0 <= at <= span:
                calls.append({"key": key, "t_ms": round(at, 4), "ms": round(s.elapsed_time(t), 4)})
        with open(timeline_path, "w") as f:
            json.dump({"step_ms": span, "calls": calls}, f)
    for key, nbytes in ledger.link_bytes.items():  # NVLink side of the exchange kernels
        if key in per and per[key]["ms"] > 0:
            per[key]["link_bytes"] = nbytes
    return total_ms.item() / steps, per, dict(ledger.timer.counts), clocks


def graphed_epoch_ms(w: Workload, steps: int):
    """The same epoch captured once as a CUDA graph and replayed (single GPU)."""
    from ae_mlsys_gnn_b200.graphed import GraphedStep

    gs = GraphedStep(w.step, warmup=3, device=w.dev)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=w.dev) if w.wl["name"] in L2_RESIDENT else None
    for _ in range(3):
        gs.replay()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in ev:
        if flush_buf is not None:
            flush_buf.fill_(1)
        a.record()
        gs.replay()
        b.record()
    torch.cuda.synchronize()
    return sum(a.elapsed_time(b) for a, b in ev) / steps


def roofline_of(per: dict, steps: int, workload: str):
    """Roofline record of the HBM-bound entry point with the largest time."""
    peak, peak_kind = measured_peak_gbs()
    hbm = {k: v for k, v in per.items() if v["bytes"] > 0}  # the GEMM entries carry no byte count
    if not hbm:
        return None
    key = max(hbm, key=lambda k: hbm[k]["ms"])
    p = per[key]
    launch_ms = p["ms"] / p["calls"]
    alg = p["bytes"] / p["calls"]
    alg_gbs = alg / (launch_ms * 1e-3) / 1e9 if launch_ms > 0 else 0.0
    traffic = traffic_from_profile(key, workload, alg)
    scaled = traffic is not None and traffic != traffic_from_profile(key, workload)
    roof = {"bound": "hbm", "kernel": key, "peak": peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s",
            "launch_ms": launch_ms, "traffic": traffic, "bytes_per_launch_algorithmic": alg,
            "achieved_algorithmic": alg_gbs, "frac_algorithmic": alg_gbs / peak}
    if traffic:
        roof["achieved"] = traffic / (launch_ms * 1e-3) / 1e9
        roof["basis"] = "measured DRAM bytes per launch (ncu, profiles/traffic.json) / CUDA-event time"
        if scaled:
            roof["basis"] += ("; the capture is of the whole graph on one GPU, scaled to this rank's block by"
                              " algorithmic bytes")
    else:  # no capture of this kernel and shape: only the algorithmic figure exists
        roof["achieved"] = alg_gbs
        roof["basis"] = "algorithmic bytes / CUDA-event time (no DRAM capture for this kernel and shape)"
    roof["frac"] = roof["achieved"] / peak
    roof["frac_of_8tbs"] = roof["achieved"] / 8000.0
    entries = {}
    for k, v in per.items():
        e = {"ms_per_step": v["ms"] / steps, "calls_per_step": v["calls"] / steps}
        if v.get("link_bytes"):
            e["nvlink_gb_per_step"] = v["link_bytes"] / steps / 1e9
            e["nvlink_gbs"] = v["link_bytes"] / (v["ms"] * 1e-3) / 1e9
        if v["bytes"] > 0 and v["ms"] > 0:
            e["gbs_algorithmic"] = v["bytes"] / (v["ms"] * 1e-3) / 1e9
            t = traffic_from_profile(k, workload, v["bytes"] / v["calls"])
            if t:
                e["gbs_dram"] = t * v["calls"] / (v["ms"] * 1e-3) / 1e9
        entries[k] = e
    roof["per_entry_point"] = entries
    return roof


def model_record(name: str, dev, seed: int, steps: int):
    """Sub-record of one of the other configurations: eager epoch, graph-replayed epoch, kernel sum."""
    wl = dict(WORKLOADS[name], name=name)
    w = Workload(wl, dev, seed, capturable=True)
    ms, per, counts, _ = timed_epochs(w, steps, 3)
    kernel_ms = sum(v["ms"] for v in per.values()) / steps
    rec = {"workload": wl["desc"], "nodes": w.n, "edges": w.nnz, "epoch_ms": ms,
           "library_entry_points_ms": kernel_ms, "gpu_launches_per_step": count_launches(counts, 0) / steps}
    hbm = {k: v for k, v in per.items() if v["bytes"] > 0}
    if hbm:
        key = max(hbm, key=lambda k: hbm[k]["ms"])
        p = per[key]
        peak, _ = measured_peak_gbs()
        gbs = p["bytes"] / (p["ms"] * 1e-3) / 1e9
        rec["dominant"] = {"entry_point": key, "ms_per_step": p["ms"] / steps,
                           "gbs_algorithmic": gbs, "frac_algorithmic": gbs / peak}
    if name in L2_RESIDENT:
        rec["bound"] = "launch / L2 (gathered operand fits in the 126 MB L2)"
        try:
            rec["epoch_ms_cuda_graph"] = graphed_epoch_ms(w, steps)
        except Exception as e:  # capture refused: report why, keep the eager number
            rec["epoch_ms_cuda_graph"] = None
            rec["cuda_graph_error"] = f"{type(e).__name__}: {e}"[:200]
    else:
        rec["bound"] = "hbm"
    del w
    release_device_memory()
    return rec


# ----------------------------------------------------------------------------------------
# own arm
# ----------------------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="C5", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-models", action="store_true", help="skip the sub-records of the other configurations")
    ap.add_argument("--no-gpu-reference", action="store_true", help="skip timing the reference's CUDA operators")
    ap.add_argument("--timeline", default=None, metavar="PATH",
                    help="rank 0 writes the last timed step as a JSON list of library calls (start, duration)")
    args = ap.parse_args()
    wl = dict(WORKLOADS[args.workload], name=args.workload)
    if args.warmup < 3 and args.impl == "b200":
        args.warmup = 3

    if args.impl == "reference":
        reference_arm(args, wl)
        return

    world = env_int("WORLD_SIZE", 1)
    rank = env_int("RANK", 0)
    local_rank = env_int("LOCAL_RANK", 0)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operators have no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    if world > 1 and wl["kind"] != "gat":
        raise SystemExit("only the GAT workloads are partitioned; EdgeConv / GMMConv run as replicas (N=1)")

    from ae_mlsys_gnn_b200 import _capi
    from ae_mlsys_gnn_b200.operators import dense

    _capi.lib()
    w = Workload(wl, dev, args.seed, world, rank)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms_per_step, per, counts, clocks = timed_epochs(w, args.steps, args.warmup, sampler,
                                                    args.timeline if rank == 0 else None)
    launches = count_launches(counts, 0)

    # ---- end to end: host buffers in, loss out, through the public API -------------------
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(args, w)
        dense.check_status(dev)
    roof = roofline_of(per, args.steps, wl["name"])
    per_rank = None
    if world > 1:  # how even the partition is: every rank's share of rows, halo, sends and kernel time
        part = w.part
        mine = torch.tensor([part.n_local, int(part.row_ptr[-1].item()), part.fwd.n_halo,
                             sum(part.fwd.send_splits), sum(v["ms"] for v in per.values()) / args.steps,
                             sum(v["ms"] for k, v in per.items() if k.startswith("gnn_halo_push")) / args.steps],
                            dtype=torch.float64, device=dev)
        rows = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(rows, mine)
        per_rank = [{"rows": int(r[0]), "edges": int(r[1]), "halo_rows": int(r[2]), "rows_sent": int(r[3]),
                     "entry_points_ms": round(float(r[4]), 3), "halo_push_ms": round(float(r[5]), 3)}
                    for r in rows]
    setup_ms = w.setup_ms
    exchange = w.exchange
    if hasattr(w.model, "close"):
        w.model.close()  # peer-mapped exchange buffers
    fallbacks = dense.fallback_calls()

    single = rank == 0 and world == 1
    models = gpu_ref = cpu = None
    if single and (not args.no_models or not args.no_gpu_reference):
        del w
        release_device_memory()
    if single and not args.no_models and args.workload == "C5":
        models = {}
        for name in ("C1", "C2", "C3", "C4"):
            models[name] = model_record(name, dev, args.seed, min(args.steps, 10))
    if single and not args.no_gpu_reference:
        gpu_ref = gpu_reference_leg(dev, args.seed)
        release_device_memory()
    if single and not args.no_cpu_baseline:
        cpu = run_cpu_epochs(wl, 2, 1, args.seed)

    if rank == 0:
        line = {
            "metric": METRIC, "value": ms_per_step, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_of(wl, world, exchange),
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "setup_ms": setup_ms,
            "cublas_fallback_calls": fallbacks, "roofline": roof, "cpu_baseline": cpu,
            "models": models, "gpu_reference": gpu_ref,
        }
        if per_rank is not None:
            line["per_rank"] = per_rank
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_e2e(args, w: Workload):
    """Same epoch, but every step starts from pinned HOST buffers (graph in CSR, inputs,
    labels), copies them to the device, builds the CSC with the csr2csc kernel
    (single GPU), runs forward/backward/update through the public layers API and reads
    the loss back."""
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc

    wl, d, model, opt, part, dev, world = w.wl, w.d, w.model, w.opt, w.part, w.dev, w.world

    def pin(t):
        return t.detach().cpu().pin_memory()

    kind = wl["kind"]
    if kind == "gat" and part is not None:
        host = {k: pin(v) for k, v in dict(part.index_tensors(), x=d["x_l"], y=d["y_l"]).items()}
    elif kind == "edgeconv":
        host = {k: pin(v) for k, v in dict(points=d["points"], src=d["src"], y=d["labels"]).items()}
    else:
        g = d["graph"]
        host = {k: pin(v) for k, v in dict(row_ptr=g.row_ptr, col_ind=g.col_ind, x=d["x"], y=d["labels"]).items()}
        if kind == "gmm":
            host["pseudo"] = pin(d["pseudo"])
    h2d = sum(v.numel() * v.element_size() for v in host.values())

    side = torch.cuda.Stream(device=dev)

    def upload():
        """Host -> device copies of one step.  Where the step builds the CSC itself, the graph
        arrays go first on the compute stream and the rest (features, labels) on a second
        stream, so that they arrive while the csr2csc kernels run."""
        if not (kind in ("gat", "gmm") and part is None):
            return {k: v.to(dev, non_blocking=True) for k, v in host.items()}
        t = {k: host[k].to(dev, non_blocking=True) for k in ("row_ptr", "col_ind")}
        with torch.cuda.stream(side):
            rest = {k: v.to(dev, non_blocking=True) for k, v in host.items() if k not in t}
        t["_rest"] = rest
        return t

    def arrived(t):
        rest = t.pop("_rest", None)
        if rest is not None:
            cur = torch.cuda.current_stream(dev)
            cur.wait_stream(side)
            for v in rest.values():
                v.record_stream(cur)
            t.update(rest)

    def one():
        t = upload()
        if kind == "gat" and part is not None:
            p2 = part.with_index_tensors(t)
            out = model(p2, t["x"])
            loss = model.loss(p2, out, t["y"])
            opt.zero_grad(set_to_none=True)
            loss.backward()
            model.all_reduce_grads(world)
        elif kind == "gat":
            cp, ri, _ = csr2csc(t["row_ptr"], t["col_ind"])
            arrived(t)
            loss = mean_cross_entropy(model(t["row_ptr"], t["col_ind"], cp, ri, t["x"]), t["y"])
            opt.zero_grad(set_to_none=True)
            loss.backward()
        elif kind == "edgeconv":
            loss = mean_cross_entropy(model(t["points"], t["src"]), t["y"])
            opt.zero_grad(set_to_none=True)
            loss.backward()
        else:
            cp, ri, pm = csr2csc(t["row_ptr"], t["col_ind"])
            arrived(t)
            loss = mean_cross_entropy(model(t["row_ptr"], t["col_ind"], cp, ri, pm, t["x"], t["pseudo"]), t["y"])
            opt.zero_grad(set_to_none=True)
            loss.backward()
        opt.step()
        return loss.item()  # device -> host read of the result

    one()
    barrier(world)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        one()
    b.record()
    barrier(world)
    ms = torch.tensor([a.elapsed_time(b) / args.steps], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return {"value": ms.item(), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4}


if __name__ == "__main__":
    main()
