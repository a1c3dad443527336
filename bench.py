"""Benchmark of the hot path: edges/s of the Clebsch-Gordan tensor-product layer, forward + backward
(l_max = 3, 64 channels, full 64 -> 64 channel mixing per path), on N GPUs of one box.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg5|cfg5q|cfg2|cfg1|cfg3|cfg4|featurize|epilogue]
                    [--feature-mode uv|uu] [--repeats R] [--impl ours|reference|reference_triton] [--no-graph] [--no-cpu-baseline] [--unfused-exchange]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = one pass of the layer over one synthetic graph: spherical harmonics of the edge vectors,
gather of node features by edge source, CG tensor product with shared uvw weights, sum into
destination nodes, and the backward pass for node features, edge vectors and weights.

Workloads (seeded synthetic data, shapes of the benchmark configurations):
  cfg5  random geometric graph, 100k nodes, ~2M edges (degree 20), Morton-ordered node ids.  Used at
        every N (strong scaling): edges are sharded by destination-node range, halo node rows travel
        by NCCL all-to-all.  The working set (410 MB of node features, 2.5 GB of per-node
        intermediates) is far larger than the 126 MB L2, so no explicit flush is needed.
  cfg5q a quarter-size cfg5 (25k nodes, ~500k edges) for profiler captures.
  cfg2  200k edges with uniformly random sources over 10k nodes (single GPU).  Its node table fits in
        L2, so L2 is flushed between steps and every step is timed on its own.  ``--feature-mode uu`` runs the
        same graph with per-path channel-wise weights (23 x 64) instead of the 64 x 64 mixing.
  cfg1 / cfg3 / cfg4  the small configurations (equitorch_b200/utils/workloads.py), one GPU, their own JSON
        lines: per-sample 'uu' product at l_max 2; molecular-style layer with per-edge bfloat16 weights;
        Wigner-rotated SO(2) linear layer at l = 0..6.  L2 is flushed between steps.
  featurize  side measurement, one GPU: radius graph + edge vectors + harmonics + Bessel basis + cutoff of the
        scaling graph's point cloud (100k points, ~2M edges) in two kernel passes.
  epilogue  side measurement, one GPU: Gate -> BatchRMSNorm -> LayerRMSNorm forward + backward on 100k x 16 x 64
        node features (its own JSON line; not the metric of the benchmark).

The timed region runs twice: eagerly with CUDA events around every kernel (the per-kernel table and
``eager_ms_per_step``) and as replays of a CUDA graph of the same step (``value`` / ``ms_per_step``; at small
per-GPU sizes the eager step is bound by the Python launch overhead, ``host_enqueue_ms_per_step``).

Rank 0 prints ONE JSON line.  ``value`` is device-timed with inputs resident in HBM; ``e2e`` moves the
step's inputs from pinned host memory and the result back inside the timed region; ``roofline``
describes the kernel that takes the largest share of the step; ``cpu_baseline`` times the CPU oracle
(a port of the reference's algorithm) on a bounded sample of the same workload.
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

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

IRREPS = "0e+1o+2e+3o"
L_MAX, CHANNELS, DIM, ROWS, PATHS = 3, 64, 16, 99, 23
METRIC = "edges/s, CG tensor product fwd+bwd (lmax=3, C=64)"


# ----------------------------------------------------------------------------------------------
def make_workload(name: str, mode: str = "uv"):
    from equitorch_b200.utils.synthetic import node_features, radius_graph, random_graph
    if name == "cfg5":
        graph, _ = radius_graph(100_000, 2_000_000, seed=0)
        label = "cfg5: random geometric graph, 100k nodes, ~2M edges (avg degree 20), Morton-ordered ids"
    elif name == "cfg5q":   # quarter-size cfg5 for profiler captures (node table 102 MB: still larger than L2)
        graph, _ = radius_graph(25_000, 500_000, seed=0)
        label = "cfg5q: random geometric graph, 25k nodes, ~500k edges (avg degree 20), Morton-ordered ids"
    elif name == "cfg2":
        graph = random_graph(10_000, 200_000, seed=0)
        label = "cfg2: 200k edges, uniform random src over 10k nodes, dst sorted"
    else:
        raise SystemExit(f"unknown workload {name}")
    x = node_features(graph.num_nodes, DIM, CHANNELS, seed=1)
    gen = torch.Generator().manual_seed(2)
    cot = torch.randn(graph.num_nodes, DIM, CHANNELS, generator=gen)
    if mode == "uv":
        weight = (torch.rand(PATHS, CHANNELS, CHANNELS, generator=gen) * 2 - 1) * (3.0 / CHANNELS) ** 0.5
    else:
        weight = (torch.rand(PATHS, CHANNELS, generator=gen) * 2 - 1) * 3.0 ** 0.5
    return graph, x, cot, weight, label


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(hbm_gbs=float(d["hbm_gbs"]), source="measured")
    return dict(hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.thread, self.gpu = [], None, None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return self
        self.thread = threading.Thread(target=lambda: self.rows.extend(self.proc.stdout), daemon=True)
        self.thread.start()
        return self

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=2)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.rows:
            parts = [p.strip() for p in row.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            reasons.update(n for n, v in zip(names, parts[2:6]) if v.lower().startswith("active"))
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------------------------
# CPU arm.  Two timings on the host cores, both on bounded, destination-contiguous samples of the workload:
#   "reference": the reference package itself (installed unmodified under baseline/_ref by build(); its two
#                torch_geometric reductions come from the documented-semantics stand-in of
#                tests/golden/_reference_import.py) - gather, SphericalHarmonics, SO3Linear, index_add, backward -
#                in chunks of 1024 edges, because its CPU path materialises ~1.6 MB of scratch per edge;
#   "port":      the oracle (oracle/, a dense-einsum restatement of the same algorithm) on ~32k edges.
# ----------------------------------------------------------------------------------------------
REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def _prefix(graph, n_edges):
    n_edges = min(n_edges, graph.src.numel())
    last_node = int(graph.dst[n_edges - 1])
    n_edges = int(torch.searchsorted(graph.dst, torch.tensor(last_node), right=True))
    return n_edges, last_node


def cpu_sample_step(graph, x, cot, weight, max_edges: int, mode: str = "uv"):
    """Forward + backward of the oracle on the first destination nodes holding ~max_edges edges."""
    from oracle import tensor_products as otp
    n_edges, last_node = _prefix(graph, max_edges)
    src, dst, vec = graph.src[:n_edges], graph.dst[:n_edges], graph.edge_vec[:n_edges]
    xs = x.clone().requires_grad_(True)
    vs = vec.clone().requires_grad_(True)
    ws = weight.clone().requires_grad_(True)
    t0 = time.perf_counter()
    out = otp.so3_linear_message_passing(xs, vs, src, dst, ws, IRREPS, IRREPS, IRREPS, feature_mode=mode,
                                         num_out_nodes=last_node + 1)
    torch.autograd.grad(out, [xs, vs, ws], cot[: last_node + 1])
    return n_edges, time.perf_counter() - t0


_reference_layer = {}


def reference_available() -> bool:
    return os.path.isdir(os.path.join(REF_DIR, "equitorch"))


def reference_chunk_step(graph, x, cot, weight, first_edge: int, chunk: int = 1024, mode: str = "uv"):
    """One chunk of `chunk` edges through the reference's own modules on the CPU: forward + backward."""
    os.environ["EQUITORCH_REFERENCE_ROOT"] = REF_DIR
    from tests.golden._reference_import import import_reference
    import_reference()
    from equitorch.nn.linears import SO3Linear as RefSO3Linear
    from equitorch.nn.sphericals import SphericalHarmonics as RefSH
    if mode not in _reference_layer:
        _reference_layer[mode] = (RefSO3Linear(IRREPS, IRREPS, IRREPS, CHANNELS, CHANNELS, internal_weights=False,
                                               feature_mode=mode), RefSH(L_MAX))
    layer, sh = _reference_layer[mode]
    e0, e1 = first_edge, min(first_edge + chunk, graph.src.numel())
    src, dst, vec = graph.src[e0:e1], graph.dst[e0:e1], graph.edge_vec[e0:e1]
    d0, d1 = int(dst[0]), int(dst[-1]) + 1
    xs = x.clone().requires_grad_(True)
    vs = vec.clone().requires_grad_(True)
    ws = weight.clone().requires_grad_(True)           # the reference's backward needs a weight that requires grad
    t0 = time.perf_counter()
    msg = layer(xs[src], sh(vs), ws)
    out = torch.zeros(d1 - d0, DIM, CHANNELS).index_add(0, dst - d0, msg)
    torch.autograd.grad(out, [xs, vs, ws], cot[d0:d1])
    return e1 - e0, time.perf_counter() - t0


def cpu_baseline(graph, x, cot, weight, mode="uv", max_edges=32768, repeats=2, chunks=5):
    torch.set_num_threads(os.cpu_count() or 1)
    best, n_edges = None, 0
    for _ in range(repeats + 1):              # first run warms up the allocator and thread pool
        n_edges, dt = cpu_sample_step(graph, x, cot, weight, max_edges, mode)
        best = dt if best is None else min(best, dt)
    port = {"value": n_edges / best, "unit": "edges/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"first {n_edges} edges (by destination) of the workload, fwd+bwd, float32, best of {repeats}"}
    if not reference_available():
        port["reference_unavailable"] = "baseline/_ref is absent (build() installs it where the reference checkout exists)"
        return port
    reference_chunk_step(graph, x, cot, weight, 0, mode=mode)            # warm-up chunk
    done, spent = 0, 0.0
    for k in range(chunks):
        n, dt = reference_chunk_step(graph, x, cot, weight, k * 1024, mode=mode)
        done += n
        spent += dt
    return {"value": done / spent, "unit": "edges/s", "cores": torch.get_num_threads(), "kind": "reference",
            "sample": f"{chunks} chunks of 1024 destination-contiguous edges through the reference's own SO3Linear / "
                      "SphericalHarmonics on the CPU (gather + layer + index_add, fwd+bwd, float32), mean over chunks",
            "port": port}


def run_reference_triton(args):
    """The reference's own GPU path (its Triton kernels, unmodified, from baseline/_ref) on this GPU: per-edge
    SO3Linear at l_max 3, 64 channels, E = 20,000 (its per-edge intermediate is 25 KB per edge), 'uu' and 'uv',
    forward + backward.  A second, same-box bar beside the CPU arm; prints one JSON line, `unavailable` with
    the error message if the kernels do not compile or launch here."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    line = {"impl": "reference_triton", "metric": METRIC, "unit": "edges/s", "n_gpus": 1, "dtype": "f32", "data": "synthetic"}
    try:
        if not reference_available():
            raise RuntimeError("baseline/_ref is absent")
        os.environ["EQUITORCH_REFERENCE_ROOT"] = REF_DIR
        from tests.golden._reference_import import import_reference
        import_reference()
        from equitorch.nn.linears import SO3Linear as RefSO3Linear
        from equitorch.nn.sphericals import SphericalHarmonics as RefSH
        dev = torch.device("cuda", 0)
        e = 20_000
        gen = torch.Generator().manual_seed(0)
        x = torch.randn(e, DIM, CHANNELS, generator=gen).to(dev).requires_grad_(True)
        v = torch.randn(e, 3, generator=gen).to(dev).requires_grad_(True)
        cot = torch.randn(e, DIM, CHANNELS, generator=gen).to(dev)
        res = {}
        for mode in ("uu", "uv"):
            layer = RefSO3Linear(IRREPS, IRREPS, IRREPS, CHANNELS, CHANNELS, internal_weights=False, feature_mode=mode).to(dev)
            shape = (PATHS, CHANNELS) if mode == "uu" else (PATHS, CHANNELS, CHANNELS)
            w = ((torch.rand(*shape, generator=gen) * 2 - 1) * 0.2).to(dev).requires_grad_(True)
            sh = RefSH(L_MAX)

            def step():
                out = layer(x, sh(v), w)
                return torch.autograd.grad(out, [x, v, w], cot)
            for _ in range(max(3, args.warmup)):
                step()
            torch.cuda.synchronize(dev)
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(args.steps):
                step()
            t1.record()
            torch.cuda.synchronize(dev)
            ms = t0.elapsed_time(t1) / max(1, args.steps)
            res[mode] = {"edges_per_s": e / (ms * 1e-3), "ms_per_step": ms}
        line.update({"value": res["uv"]["edges_per_s"], "edges": e, "modes": res, "steps": args.steps,
                     "config": {"workload": "per-edge SO3Linear (no gather, no reduction), 20,000 edges, l_max 3, 64 channels"}})
    except Exception as exc:  # noqa: BLE001 - any failure of the reference's GPU path is the result
        line["unavailable"] = f"{type(exc).__name__}: {exc}"[:400]
    print(json.dumps(line), flush=True)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    mode = args.feature_mode
    graph, x, cot, weight, label = make_workload(args.workload if args.workload in ("cfg5", "cfg5q", "cfg2") else "cfg5", mode)
    torch.set_num_threads(os.cpu_count() or 1)
    use_ref = reference_available()
    chunks = 2          # ~5 s of CPU work per step on 8 cores

    def one_step(k):
        if not use_ref:
            return cpu_sample_step(graph, x, cot, weight, 32768, mode)
        n_tot, t_tot = 0, 0.0
        for c in range(chunks):
            n, dt = reference_chunk_step(graph, x, cot, weight, ((k * chunks + c) * 1024) % max(1, graph.src.numel() - 1024),
                                         mode=mode)
            n_tot += n
            t_tot += dt
        return n_tot, t_tot

    for k in range(args.warmup):
        one_step(k)
    total_edges, total_time = 0, 0.0
    for k in range(args.steps):
        n, dt = one_step(k)
        total_edges += n
        total_time += dt
    value = total_edges / total_time
    per_step = total_edges // max(1, args.steps)
    kind = "reference" if use_ref else "port"
    what = ("the reference package itself (baseline/_ref) on the CPU: gather + SphericalHarmonics + SO3Linear + index_add, "
            f"fwd+bwd, {chunks} chunks of 1024 destination-contiguous edges per step" if use_ref else
            "CPU port of the reference's algorithm (oracle/); baseline/_ref is absent")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "edges/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total_time / max(1, args.steps),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": label, "feature_mode": mode,
                   "note": f"{what}; all host threads; each step is a bounded sample of {per_step} edges of the workload"},
        "cpu_baseline": {"value": value, "unit": "edges/s", "cores": torch.get_num_threads(), "kind": kind,
                         "sample": f"{per_step} edges per step"},
        "e2e": {"value": value, "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ----------------------------------------------------------------------------------------------
def run_epilogue(args):
    """Side measurement (one GPU): the layers that follow the tensor product in a message-passing block -
    Gate -> BatchRMSNorm -> LayerRMSNorm, forward + backward - on the node features of cfg5."""
    from equitorch_b200 import nn as enn
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    nodes, k = 100_000, L_MAX + 1
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(nodes, DIM, CHANNELS, generator=gen).to(dev).requires_grad_(True)
    gates = torch.randn(nodes, k, CHANNELS, generator=gen).to(dev).requires_grad_(True)
    cot = torch.randn(nodes, DIM, CHANNELS, generator=gen).to(dev)
    gate = enn.Gate(IRREPS, activation=torch.nn.Sigmoid()).to(dev)
    bn = enn.BatchRMSNorm(IRREPS, CHANNELS).to(dev).train()
    ln = enn.LayerRMSNorm(IRREPS, CHANNELS).to(dev)
    params = [x, gates, bn.weight, ln.weight]

    def step():
        out = ln(bn(gate(x, gates)))
        return torch.autograd.grad(out, params, cot)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize(dev)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        step()
    t1.record()
    torch.cuda.synchronize(dev)
    ms = t0.elapsed_time(t1) / max(1, args.steps)
    feat = nodes * DIM * CHANNELS * 4
    # minimal traffic: each of the three layers reads its input and writes its output forward, and reads input +
    # output gradient and writes the input gradient backward (statistics and gates are 4/16 of a feature tensor)
    algorithmic = 3 * (2 + 3) * feat + 4 * nodes * k * CHANNELS * 4
    pk = peaks()
    print(json.dumps({
        "metric": "nodes/s, Gate -> BatchRMSNorm -> LayerRMSNorm fwd+bwd (lmax=3, C=64)", "value": nodes / (ms * 1e-3),
        "unit": "nodes/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "epilogue: 100k nodes x 16 components x 64 channels", "l2": "working set >> 126 MB L2"},
        "roofline": {"bound": "hbm", "achieved": round(algorithmic / (ms * 1e-3) / 1e9, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(algorithmic / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4),
                     "peak_source": pk["source"], "algorithmic_bytes_per_step": algorithmic, "traffic": None},
    }))


def run_small(args):
    """cfg1 / cfg3 / cfg4 on one GPU: the step of equitorch_b200/utils/workloads.py, L2 flushed between steps, every
    step timed on its own with CUDA events; end to end with the inputs copied from pinned host memory and the
    loss and gradients read back every step.  The roofline figure is the whole step against its minimal traffic."""
    from equitorch_b200 import _lib
    from equitorch_b200.utils.workloads import BUILDERS
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    wl = BUILDERS[args.workload](dev)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    for _ in range(max(args.warmup, 3)):
        wl.step()
    torch.cuda.synchronize(dev)
    sampler = ClockSampler(0).start()
    launches0 = _lib.launch_count()
    per_repeat = []
    for _ in range(max(1, args.repeats)):
        pairs = []
        for _ in range(args.steps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            wl.step()
            b.record()
            pairs.append((a, b))
        torch.cuda.synchronize(dev)
        per_repeat.append(sum(a.elapsed_time(b) for a, b in pairs))
    launches = (_lib.launch_count() - launches0) // max(1, args.repeats)
    clocks = sampler.stop()
    per_repeat.sort()
    ms = per_repeat[len(per_repeat) // 2] / max(1, args.steps)

    # the same steps replayed as a CUDA graph (these configurations are launch-bound from Python)
    graph_ms, graph_error = None, None
    if not args.no_graph:
        try:
            from equitorch_b200.utils.cuda_graph import GraphedStep
            gs = GraphedStep(wl.step, dev, warmup=2)
            for _ in range(3):
                gs.replay()
            pairs = []
            for _ in range(args.steps):
                flush.zero_()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                gs.replay()
                b.record()
                pairs.append((a, b))
            torch.cuda.synchronize(dev)
            graph_ms = sum(a.elapsed_time(b) for a, b in pairs) / max(1, args.steps)
            del gs
        except Exception as exc:  # noqa: BLE001
            graph_error = f"{type(exc).__name__}: {exc}"[:300]
            torch.cuda.synchronize(dev)

    def e2e(count):
        last = None
        for _ in range(count):
            with torch.no_grad():
                for d, h in zip(wl.dev_inputs, wl.host_inputs):
                    d.copy_(h, non_blocking=True)
            loss, results = wl.step()
            last = [loss.cpu()] + [r.cpu() for r in results[:1]]      # loss and the weight gradient
        return last
    e2e(2)
    torch.cuda.synchronize(dev)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    last = e2e(args.steps)
    t1.record()
    torch.cuda.synchronize(dev)
    e2e_ms = t0.elapsed_time(t1) / max(1, args.steps)
    pk = peaks()
    best_ms = min(ms, graph_ms) if graph_ms else ms
    gbs = wl.algorithmic_bytes_per_unit * wl.units / (best_ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": f"{wl.unit}/s, {args.workload} fwd+bwd", "value": wl.units / (best_ms * 1e-3), "unit": f"{wl.unit}/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": best_ms, "eager_ms_per_step": ms,
        "graph_ms_per_step": graph_ms, "cuda_graph_error": graph_error, "higher_is_better": True, "dtype": wl.dtype,
        "data": "synthetic", "repeats": len(per_repeat),
        "config": {"workload": wl.label, "l2": "256 MB written between steps to flush L2; steps timed individually"},
        "e2e": {"value": wl.units / (e2e_ms * 1e-3), "unit": f"{wl.unit}/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": int(sum(h.numel() * h.element_size() for h in wl.host_inputs)),
                "d2h_bytes_per_step": int(sum(t.numel() * t.element_size() for t in last)),
                "copied_back": "loss and the weight gradient"},
        "gpu_launches": int(launches), "clocks": clocks,
        "roofline": {"kernel": "whole step", "bound": "hbm", "achieved": round(gbs, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(gbs / pk["hbm_gbs"], 4), "peak_source": pk["source"],
                     "algorithmic_bytes_per_unit": wl.algorithmic_bytes_per_unit, "algorithmic_note": wl.note,
                     "traffic": None},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="cfg5", choices=["cfg5", "cfg2", "cfg5q", "cfg1", "cfg3", "cfg4", "featurize", "epilogue"])
    ap.add_argument("--feature-mode", default="uv", choices=["uv", "uu"],
                    help="uv: 64 x 64 channel mixing per path (the metric); uu: channel-wise weights per path")
    ap.add_argument("--repeats", type=int, default=5, help="how often the timed region of K steps is repeated (median reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference_triton"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="time the eager step only (no CUDA-graph replay)")
    ap.add_argument("--unfused-exchange", action="store_true",
                    help="N > 1: halo exchange and gradient all-reduce as separate operations around the layer "
                         "(concatenated buffer, nothing overlapped) instead of the fused sharded layer")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.impl == "reference_triton":
        return run_reference_triton(args)
    if args.workload == "epilogue":
        return run_epilogue(args)
    if args.workload in ("cfg1", "cfg3", "cfg4", "featurize"):
        return run_small(args)

    import torch.distributed as dist
    from equitorch_b200 import _lib, _profile
    from equitorch_b200 import nn as enn
    from equitorch_b200.dist import halo_exchange, plan_shards, replicated
    from equitorch_b200.graph import EdgeGraph
    from equitorch_b200.ops.fused_tp_op import check_status

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU arm")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    if args.workload == "cfg2" and world > 1:
        raise SystemExit("cfg2 is the single-GPU microbenchmark")

    mode = args.feature_mode
    graph, x_all, cot_all, weight, label = make_workload(args.workload, mode)
    plan = plan_shards(graph.src, graph.dst, graph.num_nodes, world)[rank]
    lo, hi, e0, e1 = plan.node_lo, plan.node_hi, plan.edge_lo, plan.edge_hi
    n_edges_total, n_edges_local = graph.src.numel(), e1 - e0

    x_host = x_all[lo:hi].contiguous().pin_memory()
    vec_host = graph.edge_vec[e0:e1].contiguous().pin_memory()
    cot = cot_all[lo:hi].contiguous().to(dev)
    egraph = EdgeGraph(plan.src_local.to(dev), plan.dst_local.to(dev), plan.num_local, plan.num_owned)
    send_index = plan.send_index.to(dev)
    layer = enn.SO3LinearGraph(IRREPS, IRREPS, IRREPS, CHANNELS, CHANNELS, internal_weights=False,
                               feature_mode=mode).to(dev)
    w_dev = weight.to(dev).requires_grad_(True)
    sh = enn.SphericalHarmonics(L_MAX)
    # one GPU: the node features themselves; several: the rank's [owned | halo] buffer, halo rows filled by the layer
    n_owned = plan.num_owned
    x_dev = torch.zeros(plan.num_local if world > 1 else n_owned, *x_host.shape[1:], device=dev)
    x_dev[:n_owned].copy_(x_host)
    x_dev.requires_grad_(True)
    vec_dev = vec_host.to(dev).requires_grad_(True)
    loss_host = torch.empty(2, dtype=torch.float32).pin_memory()             # two slots: results are read one step late
    gw_host = torch.empty(2, *weight.shape).pin_memory()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev) if args.workload == "cfg2" else None

    def step(x, vec):
        if world > 1 and not args.unfused_exchange:
            out = layer.forward_sharded(x, sh(vec), egraph, plan, send_index, w_dev)
        elif world > 1:       # the exchange as separate differentiable operations around the single-GPU layer
            out = layer(halo_exchange(x[:n_owned], plan, send_index), sh(vec), egraph, replicated(w_dev))
        else:
            out = layer(x, sh(vec), egraph, w_dev)
        gx, gv, gw = torch.autograd.grad(out, [x, vec, w_dev], cot)
        return out, gx[:n_owned], gv, gw

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(args.warmup, 3)):      # at least three untimed steps
        step(x_dev, vec_dev)
    check_status()

    # ---- device-resident timing -----------------------------------------------------------
    sampler = ClockSampler(local_rank).start()
    _profile.enable(True)
    launches0 = _lib.launch_count()
    barrier()
    if flush is None:
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        host0 = time.perf_counter()
        for _ in range(args.steps):
            step(x_dev, vec_dev)
        host_enqueue_ms = (time.perf_counter() - host0) * 1e3   # time the host needed to enqueue the steps
        t1.record()
        barrier()
        elapsed_ms = t0.elapsed_time(t1)
    else:
        host_enqueue_ms = None
        pairs = []
        for _ in range(args.steps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            step(x_dev, vec_dev)
            b.record()
            pairs.append((a, b))
        barrier()
        elapsed_ms = sum(a.elapsed_time(b) for a, b in pairs)
    launches = _lib.launch_count() - launches0
    kernels = _profile.collect()
    _profile.enable(False)
    check_status()
    graph_error = None

    # ---- the same step replayed as a CUDA graph (removes the Python launch overhead, which bounds the step at
    # small per-GPU sizes); two graphs on two sets of input buffers so that the end-to-end loop can overlap the
    # next step's copy.  The eager numbers above stay in the line as `eager_ms_per_step`.
    eager_ms, graphed = elapsed_ms, None
    bufs = [(x_dev, vec_dev),
            (torch.empty_like(x_dev).requires_grad_(True), torch.empty_like(vec_dev).requires_grad_(True))]
    with torch.no_grad():
        bufs[1][0].copy_(x_dev)
        bufs[1][1].copy_(vec_dev)
    if flush is None and not args.no_graph:
        try:
            from equitorch_b200.utils.cuda_graph import GraphedStep
            graphed = [GraphedStep(lambda xb=xb, vb=vb: step(xb, vb), dev, warmup=2) for xb, vb in bufs]
        except Exception as exc:  # noqa: BLE001 - any capture failure falls back to the eager loop
            graphed, graph_error = None, f"{type(exc).__name__}: {exc}"[:300]
            torch.cuda.synchronize(dev)
        if world > 1:                       # replay on every rank or on none
            flag = torch.tensor([1 if graphed is not None else 0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag.item()) == 0:
                graphed = None
    repeat_ms = [elapsed_ms]
    if graphed is not None:
        for _ in range(3):
            graphed[0].replay()
        check_status()
        repeat_ms = []
        for _ in range(max(1, args.repeats)):       # the timed region of K steps, repeated; the median is reported
            barrier()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for i in range(args.steps):
                graphed[i % 2].replay()
            t1.record()
            barrier()
            repeat_ms.append(t0.elapsed_time(t1))
        check_status()
    clocks = sampler.stop()
    rep = torch.tensor(repeat_ms, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(rep, op=dist.ReduceOp.MAX)          # every repeat: the slowest rank
    repeat_ms = sorted(float(v) for v in rep.tolist())
    elapsed_ms = repeat_ms[len(repeat_ms) // 2] if len(repeat_ms) % 2 else 0.5 * (repeat_ms[len(repeat_ms) // 2 - 1] + repeat_ms[len(repeat_ms) // 2])

    # ---- checksum of one step (comparable across N: everything is summed over ranks) ----------------
    out_c, gx_c, gv_c, gw_c = (t.detach() for t in step(x_dev, vec_dev))
    sums = torch.stack([torch.dot(out_c.double().reshape(-1), cot.double().reshape(-1)), gx_c.double().sum(),
                        gx_c.double().square().sum(), gv_c.double().sum(), gv_c.double().square().sum()])
    if world > 1:
        dist.all_reduce(sums)
    checksum = {"loss": float(sums[0]), "gw_norm": float(gw_c.double().norm()), "gx_sum": float(sums[1]),
                "gx_norm": float(sums[2]) ** 0.5, "gv_sum": float(sums[3]), "gv_norm": float(sums[4]) ** 0.5}
    del out_c, gx_c, gv_c, gw_c

    # ---- end-to-end timing: host buffers in, result out, every step ----------------------------
    # Every step copies its own inputs from pinned host memory and reads its result back.  The copy of step
    # i + 1 runs on a second stream into the other of two device buffers while step i computes, as a data
    # loader would do it; all copies are inside the timed region.
    copy_stream = torch.cuda.Stream(dev)
    main_stream = torch.cuda.current_stream(dev)
    ready = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]

    def enqueue_inputs(i):
        slot = i % 2
        with torch.cuda.stream(copy_stream), torch.no_grad():
            if i >= 2:
                copy_stream.wait_event(consumed[slot])      # step i - 2 has finished with this buffer
            bufs[slot][0][:n_owned].copy_(x_host, non_blocking=True)
            bufs[slot][1].copy_(vec_host, non_blocking=True)
            ready[slot].record(copy_stream)

    read_back = [torch.cuda.Event() for _ in range(2)]
    results = []

    def e2e_steps(count):
        enqueue_inputs(0)
        for i in range(count):
            if i + 1 < count:
                enqueue_inputs(i + 1)
            main_stream.wait_event(ready[i % 2])
            if graphed is not None:
                out, gx, gv, gw = graphed[i % 2].replay()
            else:
                out, gx, gv, gw = step(*bufs[i % 2])
            consumed[i % 2].record(main_stream)
            # the step's result (loss = <out, cotangent>, weight gradient) goes to the host every step; the host
            # reads it while the next step is already running, so the device never waits for Python
            loss_host[i % 2: i % 2 + 1].copy_(torch.dot(out.reshape(-1), cot.reshape(-1)).reshape(1), non_blocking=True)
            gw_host[i % 2].copy_(gw, non_blocking=True)
            read_back[i % 2].record(main_stream)
            if i > 0:
                read_back[(i - 1) % 2].synchronize()
                results.append(float(loss_host[(i - 1) % 2].detach()))
        read_back[(count - 1) % 2].synchronize()
        results.append(float(loss_host[(count - 1) % 2]))

    e2e_steps(2)                      # untimed: first use of the copy stream, the reduction and the host buffers
    barrier()
    e0_, e1_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0_.record()
    e2e_steps(args.steps)
    e1_.record()
    barrier()
    e2e_ms = e0_.elapsed_time(e1_)
    check_status()

    # ---- N > 1: what the exchanges cost on their own (nothing to overlap with), and how large the halo is -----
    exchange = None
    if world > 1:
        with torch.no_grad():
            buf = x_dev.detach()
            back = buf.new_empty((send_index.shape[0], *buf.shape[1:]))
            gw_tmp = torch.zeros_like(w_dev)

            def exchange_only():
                dist.all_to_all_single(buf[n_owned:], buf[:n_owned].index_select(0, send_index), plan.recv_counts,
                                       plan.send_counts)
                dist.all_to_all_single(back, buf[n_owned:], plan.send_counts, plan.recv_counts)
                dist.all_reduce(gw_tmp)

            for _ in range(3):
                exchange_only()
            barrier()
            x0, x1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            x0.record()
            for _ in range(10):
                exchange_only()
            x1.record()
            barrier()
            stats = torch.tensor([x0.elapsed_time(x1) / 10, (plan.num_local - n_owned) / max(1, n_owned)],
                                 dtype=torch.float64, device=dev)
            dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        exchange = {"fused_with_layer": not args.unfused_exchange,
                    "standalone_ms_per_step": round(float(stats[0]), 4),
                    "standalone_is": "halo rows out + halo gradients back (all-to-all) + weight-gradient all-reduce, "
                                     "back to back with no compute, maximum over ranks",
                    "halo_rows_over_owned_rows_max": round(float(stats[1]), 4)}

    times = torch.tensor([e2e_ms, eager_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    e2e_ms, eager_ms = (float(v) for v in times.tolist())
    steps = max(1, args.steps)
    value = n_edges_total * steps / (elapsed_ms * 1e-3)
    e2e_value = n_edges_total * steps / (e2e_ms * 1e-3)

    # ---- roofline of the kernel with the largest share -------------------------------------------
    n_dst, n_src = plan.num_owned, plan.num_local
    s_bytes = ROWS * CHANNELS * 4
    row_bytes = DIM * CHANNELS * 4
    algorithmic = {   # bytes one launch must move (this rank's shard)
        "cg_segment_sum[fwd]": n_edges_local * (row_bytes + DIM * 4 + 8) + n_dst * (s_bytes + 8),
        "cg_segment_sum[grad_x]": n_edges_local * (row_bytes + DIM * 4 + 16) + n_src * (s_bytes + 8),
        "cg_inner[grad_y]": n_edges_local * (row_bytes + DIM * 4 + 8) + n_dst * (s_bytes + 8),
        "channel_mix[fwd]": n_dst * (s_bytes + row_bytes) + weight.numel() * 4,
        "channel_mix[grad_inter]": n_dst * (s_bytes + row_bytes) + weight.numel() * 4,
        "channel_mix[grad_x]": n_src * (s_bytes + row_bytes) + weight.numel() * 4,
        "weight_grad": n_dst * (s_bytes + row_bytes) + weight.numel() * 4,
        "spherical_harmonics[fwd]": n_edges_local * (12 + DIM * 4),
        "spherical_harmonics[bwd]": n_edges_local * (12 + DIM * 4 + 12),
    }
    pk = peaks()
    table = {}
    tracked_ms = sum(ms for _, ms in kernels.values())
    for name, (count, ms) in sorted(kernels.items(), key=lambda kv: -kv[1][1]):
        per_launch_ms = ms / max(1, count)
        gbs = algorithmic.get(name, 0) / (per_launch_ms * 1e-3) / 1e9 if per_launch_ms > 0 else 0.0
        table[name] = {"launches": count, "ms_per_launch": round(per_launch_ms, 4),
                       "share": round(ms / tracked_ms, 4) if tracked_ms else None,
                       "algorithmic_GBps": round(gbs, 1), "frac_of_hbm_peak": round(gbs / pk["hbm_gbs"], 4)}
    top = next(iter(table)) if table else None
    roofline = None
    # dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures of the 499,040-edge profiling
    # workload (profiles/), scaled to this launch by its edge count (same degree, so nodes scale alike).  The node
    # features of the profiling workload fit L2 and those of the full workload do not, so for the gathering
    # kernels the scaled figure is a lower bound.
    ncu_dram_bytes_cfg5q = {
        "cg_segment_sum[fwd]": 181.1e6 + 577.5e6, "cg_segment_sum[grad_x]": 188.3e6 + 578.6e6,
        "cg_inner[grad_y]": 796.4e6 + 33.2e6, "channel_mix[fwd]": 723.7e6, "channel_mix[grad_x]": 723.7e6,
    }
    if top:
        roofline = {"kernel": top, "bound": "hbm", "achieved": table[top]["algorithmic_GBps"], "peak": pk["hbm_gbs"],
                    "unit": "GB/s", "frac": table[top]["frac_of_hbm_peak"], "peak_source": pk["source"],
                    "algorithmic_bytes_per_launch": algorithmic.get(top),
                    "traffic": (int(ncu_dram_bytes_cfg5q[top] * n_edges_local / 499040)
                                if top in ncu_dram_bytes_cfg5q else None),
                    "traffic_source": ("ncu capture of the 499,040-edge profiling workload (profiles/), scaled by edges; "
                                       "a lower bound for the gathering kernels (its node table fits L2)"
                                       if top in ncu_dram_bytes_cfg5q else None),
                    # whole step against the operator-boundary traffic of the per-edge layer (20,672 B per edge: x, y,
                    # out forward; g, x, y, gx, gy backward) - the figure the 70 % target is stated on
                    "step_frac_opboundary": round(20672.0 * value / world / 1e9 / pk["hbm_gbs"], 4),
                    "step_opboundary_bytes_per_edge": 20672}

    result = {
        "metric": METRIC, "value": value, "unit": "edges/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": elapsed_ms / steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "repeats": {"count": len(repeat_ms), "ms_per_step_min": repeat_ms[0] / steps, "ms_per_step_max": repeat_ms[-1] / steps,
                    "value_is": "median over the repeats of K steps (each the maximum over ranks)"},
        "checksum": checksum,
        "config": {"workload": label, "edges": n_edges_total, "nodes": graph.num_nodes, "irreps": IRREPS,
                   "channels": CHANNELS, "feature_mode": mode, "paths": PATHS,
                   "parallelism": f"edges sharded by destination-node range over {world} GPU(s), halo rows by all-to-all"
                                  + (" received in place, gradient exchanges asynchronous inside the backward pass"
                                     if world > 1 and not args.unfused_exchange else ""),
                   "l2": ("working set >> 126 MB L2, no flush" if flush is None
                          else "256 MB written between steps to flush L2; steps timed individually")},
        "e2e": {"value": e2e_value, "unit": "edges/s", "ms_per_step": e2e_ms / steps,
                "h2d_bytes_per_step": int(x_host.numel() * 4 + vec_host.numel() * 4) * world if world == 1
                else int(x_all.numel() * 4 + graph.edge_vec.numel() * 4),
                "d2h_bytes_per_step": int(4 + gw_host[0].numel() * 4) * world,
                "copied_back": "loss <out, cotangent> and the weight gradient; out, grad_x and grad_vec stay on the device "
                               "as they would in a training step"},
        "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline, "kernels": table,
        "host_enqueue_ms_per_step": (round(host_enqueue_ms / steps, 3) if host_enqueue_ms is not None else None),
        "cuda_graph": graphed is not None, "cuda_graph_error": graph_error,
        "eager_ms_per_step": round(eager_ms / steps, 4),
    }
    if exchange is not None:
        result["exchange"] = exchange
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            result["cpu_baseline"] = cpu_baseline(graph, x_all, cot_all, weight, mode)
        print(json.dumps(result), flush=True)
    # Tear down in a fixed order: graphs that captured collectives first, then the process group.  Destroying the
    # NCCL communicator while such graphs were alive left the ranks waiting at exit; after the final barrier every
    # rank leaves through os._exit so that no finaliser can wait on a peer that has already gone.
    graphed = None
    import gc
    gc.collect()
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize(dev)
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
