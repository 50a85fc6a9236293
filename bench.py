#!/usr/bin/env python
"""Benchmark of the K-quant dequantize-and-multiply hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--m M]

Workload (N = 1): the dense 27B-class decode projection set of a layer (q 5120->6144, k/v 5120->1024,
o 6144->5120, gate/up 5120->17408 in Q4_K; down 17408->5120 in Q6_K; 214,671,360 packed bytes), fp32
activations N(0,1) at M = 1, over LAYERS distinct layers of seeded synthetic blocks so that every
step streams far more than L2 from HBM.  One step = one pass over all layers' projections.
`value` = packed weight bytes / device time (the reference's GB/s, src/hybrid/bench.rs:127-132), with
inputs resident in HBM.  `e2e` = the same through the host-buffer C-ABI calls, host<->device copies
inside the timed region.  Extra keys report M = 8 / 16 and the prefill dequant-GEMM.

With --gpus N > 1 (under torchrun) the workload is the tensor-parallel sweep: a 64-layer stack of the same
layer set (448 matrices, 13,738,967,040 packed bytes), every matrix row-sharded over the N ranks, each fused
group (q|k|v, o, gate|up, down) computing its row shard and exchanging it over NVLink peer memory in one
launch.  Total work is fixed ("strong" scaling), `value` is the aggregate of all ranks at M = 1, and the
line also carries the M = 8 figure and the per-layer latency.  Before the timed region every rank's shard of
layer 0 is checked: the gathered rows against the CPU oracle on the whole matrix, and an expert-parallel MoE
block against the single-GPU block bit for bit; the line carries the result under `parity` and the run
fails if it is off.

--impl reference times the reference's CPU path for the same projections: the oracle restatement
of its CPU dequant + matmul on all host cores, `--layers` layers per step.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

Q8_0, Q4_K, Q6_K = 8, 12, 14
# (name, rows, cols, format) of one dense 27B-class layer; groups share their input.
LAYER = [("q", 6144, 5120, Q4_K), ("k", 1024, 5120, Q4_K), ("v", 1024, 5120, Q4_K), ("o", 5120, 6144, Q4_K),
         ("gate", 17408, 5120, Q4_K), ("up", 17408, 5120, Q4_K), ("down", 5120, 17408, Q6_K)]
GROUPS = [("q", "k", "v"), ("o",), ("gate", "up"), ("down",)]
BLOCK = {Q8_0: (32, 34), Q4_K: (256, 144), Q6_K: (256, 210)}
LAYER_BYTES = sum(r * c // BLOCK[f][0] * BLOCK[f][1] for _, r, c, f in LAYER)  # 214,671,360
LAYER_WEIGHTS = sum(r * c for _, r, c, _ in LAYER)


def profile_value(name: str, key: str):
    """`key: value` line of a tracked profile summary (profiles/<name>), or None."""
    path = os.path.join(ROOT, "profiles", name)
    try:
        with open(path) as f:
            for line in f:
                if line.strip().startswith(key + ":"):
                    return int(line.split(":", 1)[1].strip().split()[0])
    except OSError:
        pass
    return None


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm = [float(r[0]) for r in self.rows if len(r) >= 7 and r[0].replace(".", "").isdigit()]
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        reasons = []
        for i, name in enumerate(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]):
            if any(len(r) >= 7 and r[3 + i].lower().startswith("active") for r in self.rows):
                reasons.append(name)
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(self.rows[0][1]), "samples": len(sm),
                "power_w_max": max(float(r[2]) for r in self.rows if len(r) >= 7), "reasons": reasons}


def random_blocks(fmt: int, blocks: int, seed: int) -> np.ndarray:
    """Packed blocks with the benchmark's distributions: d (and dmin) = fp16(|N(0,1)| * 1e-2), scale
    bytes and quant bytes uniform; draw order d -> dmin -> scales -> quants (numpy default_rng(seed))."""
    rng = np.random.default_rng(seed)
    out = np.empty((blocks, BLOCK[fmt][1]), dtype=np.uint8)
    half = lambda: (np.abs(rng.standard_normal(blocks)) * 1e-2).astype(np.float16).view(np.uint8).reshape(blocks, 2)
    if fmt == Q4_K:
        out[:, 0:2], out[:, 2:4] = half(), half()
        out[:, 4:16] = rng.integers(0, 256, size=(blocks, 12), dtype=np.uint8)
        out[:, 16:144] = rng.integers(0, 256, size=(blocks, 128), dtype=np.uint8)
    elif fmt == Q6_K:
        out[:, 208:210] = half()
        out[:, 192:208] = rng.integers(-128, 128, size=(blocks, 16), dtype=np.int8).view(np.uint8)
        out[:, 0:192] = rng.integers(0, 256, size=(blocks, 192), dtype=np.uint8)
    else:
        out[:, 0:2] = half()
        out[:, 2:34] = rng.integers(-127, 128, size=(blocks, 32), dtype=np.int8).view(np.uint8)
    return out.reshape(-1)


def random_matrix(fmt: int, rows: int, cols: int, seed: int) -> np.ndarray:
    return random_blocks(fmt, rows * cols // BLOCK[fmt][0], seed)


def shard_rows(rows: int, rank: int, world: int):
    per = rows // world
    assert per * world == rows, "rows must divide evenly over the ranks"
    return rank * per, per


# ---------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------

def run_ours(args):
    import torch
    import torch.distributed as dist
    from ferrum_b200 import surface as S

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    if world > 1:
        # stdout carries one JSON line: whatever libraries print meanwhile (NCCL's version banner when NCCL_DEBUG
        # asks for one) goes to stderr, until the line itself is printed.
        sys.stdout.flush()
        stdout_fd = os.dup(1)
        os.dup2(2, 1)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    # The library enqueues on its own stream; torch sees that stream as an ExternalStream so that
    # CUDA events are recorded on the stream the kernels are launched on.
    dev = S.Device(local, use_torch_stream=False)
    stream = torch.cuda.ExternalStream(dev.stream_ptr(), device=torch.device("cuda", local))
    # One GPU: `--layers` distinct layers per step (far more than L2).  More GPUs: the 64-layer stack, every
    # matrix sharded by rows, so a rank streams 1 / N of 13.7 GB per step.
    from ferrum_b200 import tp
    m = args.m
    layers = args.layers if world == 1 else (args.tp_layers or 64)
    distinct = min(layers, 3)

    # Weights: layer l, matrix i is drawn from seed 7 l + i -- the same whole matrix on every rank, of which the
    # rank keeps its rows; blocks as the benchmark configurations 0 and 1 define them.  The stack repeats
    # `distinct` layers' bytes in separate device copies (the stream does not care what the bytes are).
    host_layers = []
    for l in range(distinct):
        layer = {}
        for i, (name, rows, cols, fmt) in enumerate(LAYER):
            full = random_matrix(fmt, rows, cols, seed=7 * l + i)
            layer[name] = (full if world == 1 else tp.shard_packed(full, fmt, rows, cols, rank, world), full if l == 0 else None)
        host_layers.append(layer)
    mats = []
    for l in range(layers):
        layer = {}
        for name, rows, cols, fmt in LAYER:
            layer[name] = S.Matrix.from_packed(dev, rows // world, cols, 1, fmt, host_layers[l % distinct][name][0])
        mats.append(layer)
    shapes = {name: (rows // world, cols) for name, rows, cols, _ in LAYER}
    full_layer0 = {name: host_layers[0][name][1] for name, _, _, _ in LAYER}

    comm_box = {}

    def layout(mm):
        """Offsets (in floats) of the per-group inputs and the per-matrix outputs for `mm` activation rows."""
        xs, ys, xo, yo = {}, {}, 0, 0
        for g in GROUPS:
            xs[g[0]] = (xo, mm * shapes[g[0]][1])
            xo += (mm * shapes[g[0]][1] + 63) // 64 * 64
        # Outputs of one input group are adjacent, without gaps: one exchange per group moves them together.
        for g in GROUPS:
            for name in g:
                ys[name] = (yo, mm * shapes[name][0])
                yo += (mm * shapes[name][0] + 3) // 4 * 4
            yo = (yo + 63) // 64 * 64
        span_of = {g[0]: (ys[g[0]][0], (ys[g[-1]][0] + ys[g[-1]][1] + 63) // 64 * 64) for g in GROUPS}
        return xs, ys, xo, yo, span_of

    def buffers(mm, shared=False, region_base=0):
        """One contiguous input buffer (a slice per group) and one output buffer (a slice per matrix).  With
        `shared` (more than one rank) the outputs live in the exchange buffer from byte `region_base`: per input
        group a region [world][span], this rank writing slice `rank`."""
        xs, ys, xo, yo, span_of = layout(mm)
        X = torch.zeros(xo, dtype=torch.float32, device="cuda")
        if shared and not args.nccl:
            comm = comm_box["comm"]
            regions, yv = {}, {}
            for g in GROUPS:
                lo, hi = span_of[g[0]]
                region = region_base + world * lo * 4
                regions[g[0]] = (region, (hi - lo) * 4)
                for n in g:
                    yv[n] = comm.view(region + rank * (hi - lo) * 4 + (ys[n][0] - lo) * 4, ys[n][1])
            Y = comm.view(region_base, world * yo)
            return X, Y, {k: X[o:o + n] for k, (o, n) in xs.items()}, yv, regions
        Y = torch.zeros(yo, dtype=torch.float32, device="cuda")
        spans = {k: Y[lo:hi] for k, (lo, hi) in span_of.items()}
        return X, Y, {k: X[o:o + n] for k, (o, n) in xs.items()}, {k: Y[o:o + n] for k, (o, n) in ys.items()}, spans

    if world > 1 and not args.nccl:
        # One symmetric buffer for the run: the regions of the headline width, then those of M = 8.
        comm_box["comm"] = S.Comm(dev, rank, world, world * (layout(m)[3] + layout(8)[3]) * 4)

    rng = np.random.default_rng(1234)
    X, Y, x_dev, y_dev, y_spans = buffers(m, shared=world > 1)
    x_pinned = torch.from_numpy(rng.standard_normal(X.numel()).astype(np.float32)).pin_memory()
    y_pinned = torch.zeros(Y.numel(), dtype=torch.float32).pin_memory()
    X.copy_(x_pinned)
    gathered = ({k: torch.zeros(world * v.numel(), dtype=torch.float32, device="cuda") for k, v in y_spans.items()}
                if world > 1 and args.nccl else None)
    torch.cuda.synchronize()

    def enqueue_layers(xd, yd, mm, only=None):
        for layer in mats:
            for group in GROUPS:
                names = [n for n in group if only is None or n in only]
                if world > 1 and only is None and not args.nccl and not args.no_fuse:
                    # compute and exchange in one launch per input group
                    S.project_many_gather(dev, comm_box["comm"], *y_spans[group[0]], [layer[n] for n in names], xd[group[0]], mm,
                                          [yd[n] for n in names])
                    continue
                if names and not args.no_fuse:
                    S.project_many(dev, [layer[n] for n in names], xd[group[0]], mm, [yd[n] for n in names])
                else:
                    for n in names:
                        S.project(dev, layer[n], xd[group[0]], mm, yd[n])
                if world > 1 and only is None:
                    if args.nccl:
                        dist.all_gather_into_tensor(gathered[group[0]], y_spans[group[0]])
                    else:
                        comm_box["comm"].all_gather(*y_spans[group[0]])

    def make_step(xd, yd, mm, only=None):
        if (world > 1 and args.nccl) or args.eager:  # NCCL collectives are enqueued by torch: no capture, same stream
            return lambda: enqueue_layers(xd, yd, mm, only)
        dev.capture_begin()
        enqueue_layers(xd, yd, mm, only)
        graph = dev.capture_end()
        return graph.launch

    def make_host_step(xh, yh):
        """The end-to-end step: upload of the step's activations from pinned host memory, the projections (and
        exchanges), download of every output -- recorded once, replayed with one launch -- and the wait."""
        if (world > 1 and args.nccl) or args.eager:
            def host_step():
                dev.upload(X, xh)
                enqueue_layers(x_dev, y_dev, m)
                dev.download_async(yh, Y)
                dev.synchronize()
            return host_step
        dev.capture_begin()
        dev.upload(X, xh)
        enqueue_layers(x_dev, y_dev, m)
        dev.download_async(yh, Y)
        graph = dev.capture_end()

        def host_step():
            graph.launch()
            dev.synchronize()
        return host_step

    def timed(fn, steps):
        with torch.cuda.stream(stream):
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            if world > 1:
                t = torch.tensor([ms], device="cuda")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
        return ms

    parity = None
    if world > 1 and not args.nccl:
        parity = tp_parity(S, dev, torch, dist, comm_box["comm"], mats[0], full_layer0, x_pinned.numpy(), x_dev, y_dev, y_spans, m, rank, world)
        parity.update(ep_parity(S, dev, torch, dist, rank, world))
        if rank == 0 and not (parity["tp_rel_err"] <= 1e-3 and parity["ep_bits_equal"]):
            print(json.dumps({"error": "sharded results differ from the single-GPU results", "parity": parity}), flush=True)
            raise SystemExit(1)

    with torch.cuda.stream(stream):
        step = make_step(x_dev, y_dev, m)
        for _ in range(max(args.warmup, 3)):
            step()
    c0 = dev.counters().dispatches
    with ClockSampler(local) as clocks:
        ms = timed(step, args.steps)
    launches = dev.counters().dispatches - c0
    ms_per_step = ms / args.steps
    total_bytes = layers * LAYER_BYTES  # whole job: all ranks together stream every byte once per step
    value = total_bytes / (ms_per_step * 1e-3) / 1e9

    P = peaks()
    out = {
        "metric": "Q4_K_M decode projection weight GB/s (27B-class dense layer set)", "value": round(value, 2),
        "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak" if world == 1 else "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": (f"cfg1 dense 27B decode projection set (q,k,v,o,gate,up Q4_K; down Q6_K), M={m}, "
                                f"{layers} distinct layers = {total_bytes} packed bytes per step (inputs larger than L2)") if world == 1 else
                               (f"cfg4 tensor-parallel sweep: {layers}-layer dense stack of the cfg1 layer set ({7 * layers} Q4_K/Q6_K matrices, "
                                f"{total_bytes} packed bytes), M={m}, every matrix row-sharded over {world} GPUs, one exchange per input group"),
                   "m": m, "layers": layers, "parallelism": f"tp{world}" if world > 1 else "single",
                   "submission": ("one captured graph per step" if world == 1 else
                                  "eager + one NCCL all-gather per input group" if args.nccl else
                                  "one captured graph per step; per input group (q|k|v, o, gate|up, down) one kernel computes the row shard and pushes it to every peer over NVLink"),
                   "l2": "inputs larger than L2"},
        "gpu_launches": int(launches),
        "clocks": clocks.summary(),
        "per_layer_us": round(ms_per_step * 1e3 / layers, 2),
        "roofline_step": {"bytes_per_step_per_gpu": total_bytes // world, "achieved_per_gpu": round(value / world, 1), "peak": peaks()["hbm_gbs"],
                          "frac": round(value / world / peaks()["hbm_gbs"], 4), "unit": "GB/s"},
    }
    if parity is not None:
        out["parity"] = parity

    if rank == 0 and world == 1:
        def alone(names, mm, xd, yd):
            with torch.cuda.stream(stream):
                fn = make_step(xd, yd, mm, only=names)
                for _ in range(3):
                    fn()
            reps = max(5, args.steps)
            return timed(fn, reps) / reps / layers  # ms per layer's worth of these projections

        # Dominant kernel: the Q4_K GEMV on gate|up (one launch over 2 x 17408 rows, 100,270,080
        # packed bytes), timed alone over `layers` distinct layers with CUDA events on its stream.
        gms = alone(("gate", "up"), m, x_dev, y_dev)
        pair_bytes = 2 * 17408 * 5120 // 256 * 144
        achieved = pair_bytes / (gms * 1e-3) / 1e9
        stream_gbs = read_stream_probe(S, dev, stream, torch, timed)
        out["roofline"] = {"bound": "hbm", "kernel": "k_gemv_i8s<Q4_K> (gate|up, 2 x 17408 x 5120, M = 1, one launch)",
                           "achieved": round(achieved, 1), "peak": P["hbm_gbs"], "peak_source": P["source"], "unit": "GB/s",
                           "frac": round(achieved / P["hbm_gbs"], 4), "frac_of_8TBs_nominal": round(achieved / 8000.0, 4),
                           # what a kernel that only reads the same bytes reaches here, measured in this run
                           "read_stream_gbs": stream_gbs, "frac_of_read_stream": round(achieved / stream_gbs, 4),
                           # dram__bytes_read.sum + dram__bytes_write.sum of this launch, from the tracked ncu summary
                           "traffic": profile_value("gemv_i8s_q4k_gate_up_m1.md", "dram_bytes_per_launch"),
                           "traffic_source": "profiles/gemv_i8s_q4k_gate_up_m1.md (one ncu capture of this launch)",
                           "algorithmic_bytes": pair_bytes, "us_per_launch": round(gms * 1e3, 2)}
        per = {}
        for names in (("q", "k", "v"), ("o",), ("gate", "up"), ("down",)):
            t = alone(names, m, x_dev, y_dev)
            nbytes = sum(r * c // BLOCK[f][0] * BLOCK[f][1] for n, r, c, f in LAYER if n in names)
            per["|".join(names)] = {"us": round(t * 1e3, 2), "gbs": round(nbytes / (t * 1e-3) / 1e9, 1)}
        out["per_group"] = per
        if args.quick:
            print(json.dumps({"value": out["value"], "ms_per_step": out["ms_per_step"], "roofline_gbs": out["roofline"]["achieved"],
                              "per_group": per}), flush=True)
            return
        # The other decode / verify widths, same workload.
        extra = {}
        for mm in (4, 8, 16):
            Xm, Ym, xs, ys, _ = buffers(mm)
            Xm.copy_(torch.from_numpy(rng.standard_normal(Xm.numel()).astype(np.float32)))
            with torch.cuda.stream(stream):
                fn = make_step(xs, ys, mm)
                for _ in range(3):
                    fn()
            reps = max(3, args.steps // 2)
            t = timed(fn, reps) / reps
            extra[f"m{mm}_gbs"] = round(total_bytes / (t * 1e-3) / 1e9, 1)
        out["decode_widths"] = extra

        # Prefill dequant-GEMM (config 2): the same 7 matrices of layer 0 at M = 512 and 2048, bf16
        # activations and outputs, tcgen05 with fp32 accumulation; flops = 2 M N K per matrix.
        prefill = {}
        for mm in (512, 2048):
            xs = {g[0]: torch.randn(mm * shapes[g[0]][1], device="cuda").to(torch.bfloat16) for g in GROUPS}
            ys = {n: torch.zeros(mm * shapes[n][0], dtype=torch.bfloat16, device="cuda") for n in shapes}
            torch.cuda.synchronize()

            def gemm_layer():
                for layer in mats:
                    for group in GROUPS:  # matrices that share an input go out as one launch
                        S.project_many(dev, [layer[n] for n in group], xs[group[0]], mm, [ys[n] for n in group])
            with torch.cuda.stream(stream):
                for _ in range(2):
                    gemm_layer()
            reps = 3
            t = timed(gemm_layer, reps) / reps / layers
            flops = 2.0 * mm * LAYER_WEIGHTS
            per_mat = {}
            for n in ("q", "k", "o", "gate", "down"):
                def one(n=n):
                    for layer in mats:
                        S.project(dev, layer[n], xs[[g[0] for g in GROUPS if n in g][0]], mm, ys[n])
                tt = timed(one, reps) / reps / layers
                per_mat[n] = round(2.0 * mm * shapes[n][0] * shapes[n][1] / (tt * 1e-3) / 1e12, 1)
                per_mat[n + "_us"] = round(tt * 1e3, 1)
            prefill[f"m{mm}"] = {"tflops": round(flops / (t * 1e-3) / 1e12, 1), "ms_per_layer": round(t, 4),
                                 "frac_of_measured_bf16_peak": round(flops / (t * 1e-3) / 1e12 / P["bf16_tflops"], 4),
                                 "per_matrix_tflops": per_mat}
        out["prefill_gemm"] = prefill

        # MoE FFN (config 3), 35B-A3B-class: hidden 2048, 256 experts (gate/up 2048->512 Q4_K, down 512->2048
        # Q6_K) + shared expert, Q8_0 router, softmax -> top-8 -> renormalise.  T = 1 takes the per-route GEMVs,
        # T = 1024 the expert-sorted tensor-core GEMM.  GB/s = packed bytes of the weights a call must read.
        out["moe_ffn"] = moe_bench(S, dev, stream, torch, timed_ms=timed)

        # End to end through the C ABI with HOST buffers: every step uploads the step's activations
        # from pinned memory, replays the step, downloads every output and waits.
        xh, yh = x_pinned.numpy(), y_pinned.numpy()
        step_host = make_host_step(xh, yh)
        for _ in range(3):
            step_host()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            step_host()
        dt = (time.perf_counter() - t0) / args.steps
        out["e2e"] = {"value": round(total_bytes / dt / 1e9, 2), "unit": "GB/s", "h2d_bytes_per_step": int(xh.nbytes),
                      "d2h_bytes_per_step": int(yh.nbytes), "ms_per_step": round(dt * 1e3, 4),
                      "call": "one captured graph per step (fq_upload from pinned memory + the projections + fq_download_async), then fq_graph_launch + fq_synchronize"}

        # CPU baseline: the oracle port on all host cores, one layer at M = 1 (a bounded sample).
        out["cpu_baseline"] = cpu_baseline(m=m, budget_s=12.0)
    else:
        # End to end on every rank: upload this step's (replicated) activations from pinned memory, replay the
        # step (projections + exchanges), download the gathered outputs, wait; wall clock, max over ranks.
        e2e = None
        if not args.nccl:
            xh, yh = x_pinned.numpy(), y_pinned.numpy()
            step_host = make_host_step(xh, yh)
            for _ in range(3):
                step_host()
            dist.barrier()
            t0 = time.perf_counter()
            for _ in range(args.steps):
                step_host()
            dt = torch.tensor([(time.perf_counter() - t0) / args.steps], device="cuda")
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
            dt = float(dt.item())
            e2e = {"value": round(total_bytes / dt / 1e9, 2), "unit": "GB/s", "h2d_bytes_per_step": int(xh.nbytes),
                   "d2h_bytes_per_step": int(yh.nbytes), "ms_per_step": round(dt * 1e3, 4),
                   "call": "per rank: one captured graph per step (fq_upload from pinned memory + projections + exchanges + fq_download_async), then fq_graph_launch + fq_synchronize"}
        # The verify width of the sweep: the same stack at M = 8.
        tp_m8 = None
        if not args.nccl and m != 8:
            X8, Y8, x8, y8, spans8 = buffers(8, shared=True, region_base=Y.numel() * 4)
            X8.copy_(torch.from_numpy(rng.standard_normal(X8.numel()).astype(np.float32)))
            saved = dict(y_spans)
            y_spans.clear()
            y_spans.update(spans8)
            with torch.cuda.stream(stream):
                step8 = make_step(x8, y8, 8)
                for _i in range(3):
                    step8()
            reps = max(3, args.steps // 2)
            t8 = timed(step8, reps) / reps
            y_spans.clear()
            y_spans.update(saved)
            tp_m8 = {"value": round(total_bytes / (t8 * 1e-3) / 1e9, 2), "unit": "GB/s", "ms_per_step": round(t8, 4),
                     "per_layer_us": round(t8 * 1e3 / layers, 2)}
        # Expert parallelism over the same ranks (config 3 sharded by expert): every rank takes part.
        ep = moe_ep_bench(S, dev, stream, torch, dist, timed, rank, world)
        if rank == 0:
            out["e2e"] = e2e
            out["tp_m8"] = tp_m8
            out["moe_ffn_ep"] = ep
    if world > 1:
        sys.stdout.flush()
        os.dup2(stdout_fd, 1)
        os.close(stdout_fd)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def tp_parity(S, dev, torch, dist, comm, layer0, full0, x_host, x_dev, y_dev, y_spans, m, rank, world):
    """Sharded projections of layer 0 with the exchange, once per input group: every rank's gathered rows must be
    what the CPU oracle computes from the whole matrix (sampled rows, max |d| / max |y| <= 1e-3).  Checked on
    rank 0, which sees the rows of every rank after the exchange."""
    from oracle import ref  # the checker
    worst = 0.0
    xs_off, ys_off, _, _, span_of = None, None, None, None, None
    for group in GROUPS:
        S.project_many_gather(dev, comm, *y_spans[group[0]], [layer0[n] for n in group], x_dev[group[0]], m, [y_dev[n] for n in group])
    dev.synchronize()
    dist.barrier()
    if rank == 0:
        rng = np.random.default_rng(99)
        for group in GROUPS:
            region, span_bytes = y_spans[group[0]]
            gathered = comm.view(region, world * span_bytes // 4).cpu().numpy().reshape(world, span_bytes // 4)
            x = x_dev[group[0]].cpu().numpy().reshape(m, -1)
            at = 0
            for n in group:
                name, rows, cols, fmt = next(e for e in LAYER if e[0] == n)
                per = rows // world
                y = np.concatenate([gathered[r, at:at + m * per].reshape(m, per) for r in range(world)], axis=1)  # [m, rows]
                at += (m * per + 3) // 4 * 4
                pick = np.sort(rng.choice(rows, 16, replace=False))
                rb = cols // BLOCK[fmt][0] * BLOCK[fmt][1]
                sub = np.concatenate([full0[n][r * rb:(r + 1) * rb] for r in pick])
                want = ref.matmul(fmt, sub, len(pick), cols, x, m, mode=0)
                worst = max(worst, float(np.abs(y[:, pick] - want).max() / np.abs(y).max()))
    dist.barrier()
    return {"tp_rel_err": worst, "tp_checked": "layer 0, every input group, 16 sampled rows per matrix against the CPU oracle on the unsharded matrix"}


def ep_parity(S, dev, torch, dist, rank, world):
    """The expert-parallel MoE block (config 3 geometry; 40 tokens: the integer grouped kernel, and 1024 tokens:
    the fp16 tensor-core one) against the single-GPU block on the same weights: bit for bit."""
    from ferrum_b200 import tp
    H, E, F, USED = 2048, 256, 512, 8
    local = E // world
    M = S.Matrix.from_packed
    full = {k: random_matrix(fmt, rows, cols, seed) for k, (fmt, rows, cols, seed) in
            dict(gate=(Q4_K, E * F, H, 911), up=(Q4_K, E * F, H, 912), down=(Q6_K, E * H, F, 913)).items()}
    shared = [M(dev, E, H, 1, Q8_0, random_matrix(Q8_0, E, H, 910)), M(dev, F, H, 1, Q4_K, random_matrix(Q4_K, F, H, 914)),
              M(dev, F, H, 1, Q4_K, random_matrix(Q4_K, F, H, 915)), M(dev, H, F, 1, Q6_K, random_matrix(Q6_K, H, F, 916))]
    mine = S.MoeFfn(shared[0], M(dev, F, H, local, Q4_K, tp.shard_experts(full["gate"], Q4_K, F, H, E, rank, world)),
                    M(dev, F, H, local, Q4_K, tp.shard_experts(full["up"], Q4_K, F, H, E, rank, world)),
                    M(dev, H, F, local, Q6_K, tp.shard_experts(full["down"], Q6_K, H, F, E, rank, world)),
                    shared[1], shared[2], shared[3], None, E, USED, H, F, F, False, True)
    whole = None
    if rank == 0:
        whole = S.MoeFfn(shared[0], M(dev, F, H, E, Q4_K, full["gate"]), M(dev, F, H, E, Q4_K, full["up"]), M(dev, H, F, E, Q6_K, full["down"]),
                         shared[1], shared[2], shared[3], None, E, USED, H, F, F, False, True)
    widths = (40, 1024)
    equal = True
    for T in widths:
        torch.manual_seed(11 + T)
        x = (torch.randn(T * H, device="cuda") * 0.12).contiguous()
        comm = S.Comm(dev, rank, world, 8192 + T * USED * H * 4 + (T + 8 * world) * H * 4)
        scratch = torch.zeros(S.moe_ffn_scratch_elems(dev, mine, T), dtype=torch.float32, device="cuda")
        out = torch.zeros(T * H, dtype=torch.float32, device="cuda")
        S.moe_ffn_ep(dev, comm, 4096, mine, rank * local, x, T, scratch, out)
        dev.synchronize()
        if rank == 0:
            ref_out = torch.zeros(T * H, dtype=torch.float32, device="cuda")
            S.moe_ffn(dev, whole, x, T, torch.zeros(S.moe_ffn_scratch_elems(dev, whole, T), dtype=torch.float32, device="cuda"), ref_out)
            dev.synchronize()
            equal = equal and bool(torch.equal(out, ref_out))
        dist.barrier()
        comm.close()
    return {"ep_bits_equal": equal,
            "ep_checked": f"fq_moe_ffn_ep ({E} experts over {world} ranks, {' and '.join(str(t) for t in widths)} tokens) against fq_moe_ffn on rank 0"}


def moe_ep_bench(S, dev, stream, torch, dist, timed_ms, rank, world):
    """Config 3 with the 256 experts split over the ranks (router, shared expert and x replicated); the
    expert-sorted rows are exchanged by the peer-push all-gather inside the captured step."""
    H, E, F, USED = 2048, 256, 512, 8
    local = E // world
    from ferrum_b200 import tp
    M = S.Matrix.from_packed
    f = S.MoeFfn(M(dev, E, H, 1, Q8_0, random_matrix(Q8_0, E, H, 900)),
                 M(dev, F, H, local, Q4_K, tp.shard_experts(random_matrix(Q4_K, E * F, H, 901), Q4_K, F, H, E, rank, world)),
                 M(dev, F, H, local, Q4_K, tp.shard_experts(random_matrix(Q4_K, E * F, H, 902), Q4_K, F, H, E, rank, world)),
                 M(dev, H, F, local, Q6_K, tp.shard_experts(random_matrix(Q6_K, E * H, F, 903), Q6_K, H, F, E, rank, world)),
                 M(dev, F, H, 1, Q4_K, random_matrix(Q4_K, F, H, 904)), M(dev, F, H, 1, Q4_K, random_matrix(Q4_K, F, H, 905)),
                 M(dev, H, F, 1, Q6_K, random_matrix(Q6_K, H, F, 906)), None, E, USED, H, F, F, False, True)
    # Two exchange regions used in turn: consecutive exchanges of a communicator may not share a region.
    region_bytes = 1024 * USED * H * 4 + 1024 * H * 4  # the expert rows, then the combined outputs
    comm = S.Comm(dev, rank, world, 4096 + 2 * region_bytes)
    res = {}
    for T in (1, 1024):
        torch.manual_seed(7)  # the same tokens, hence the same routing, on every rank
        x = (torch.randn(T * H, device="cuda") * 0.12).contiguous()
        scratch = torch.zeros(S.moe_ffn_scratch_elems(dev, f, T), dtype=torch.float32, device="cuda")
        o = torch.zeros(T * H, dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        graphs = []
        for region in (4096, 4096 + region_bytes):
            dev.capture_begin()
            S.moe_ffn_ep(dev, comm, region, f, rank * local, x, T, scratch, o)
            graphs.append(dev.capture_end())

        def pair():
            graphs[0].launch()
            graphs[1].launch()
        with torch.cuda.stream(stream):
            for _ in range(2):
                pair()
        reps = 5
        ms = timed_ms(pair, reps) / (2 * reps)
        inbound = (T * USED * H * 4 * (world - 1) // world if T * USED <= 32 else
                   (T * USED * H * 4 // world + T * H * 4) * (world - 1) // world)
        res[f"t{T}"] = {"us": round(ms * 1e3, 1), "experts_per_rank": local, "inbound_bytes_per_rank": inbound,
                        "exchange": "all rows to all ranks" if T * USED <= 32 else "rows to the token's owner, then the outputs gathered"}
    dev.synchronize()
    dist.barrier()
    comm.close()
    return res


def read_stream_probe(S, dev, stream, torch, timed_ms, verbose=False):
    """GB/s of a kernel that only reads: four 100 MB buffers in turn (more than L2), the best grid of a few."""
    n = 100_270_080  # the bytes of the gate|up launch
    bufs = [torch.full((n,), i + 1, dtype=torch.uint8, device="cuda") for i in range(4)]
    torch.cuda.synchronize()
    best, table = 0.0, {}
    for per_sm in (4, 8, 16, 32):
        def go(per_sm=per_sm):
            for b in bufs:
                dev.probe_read_stream(b, per_sm)
        with torch.cuda.stream(stream):
            go()
        ms = timed_ms(go, 5) / (5 * len(bufs))
        table[per_sm] = round(n / (ms * 1e-3) / 1e9, 1)
        best = max(best, table[per_sm])
    return (best, table) if verbose else best


def run_stream_probe(args):
    import torch
    from ferrum_b200 import surface as S
    torch.cuda.set_device(0)
    dev = S.Device(0, use_torch_stream=False)
    stream = torch.cuda.ExternalStream(dev.stream_ptr(), device=torch.device("cuda", 0))

    def timed(fn, steps):
        with torch.cuda.stream(stream):
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            torch.cuda.synchronize()
        return e0.elapsed_time(e1)
    best, table = read_stream_probe(S, dev, stream, torch, timed, verbose=True)
    print(json.dumps({"probe": "read_stream", "bytes_per_launch": 100270080, "buffers": 4, "gbs_by_blocks_per_sm": table, "best_gbs": best,
                      "copy_peak_gbs": peaks()["hbm_gbs"]}), flush=True)


def run_moe_probe(args):
    """Only the MoE block and the Q8_0 head (what the default line reports under `moe`): the command a launch
    list of the block is taken on."""
    import torch
    from ferrum_b200 import surface as S
    torch.cuda.set_device(0)
    dev = S.Device(0, use_torch_stream=False)
    stream = torch.cuda.ExternalStream(dev.stream_ptr(), device=torch.device("cuda", 0))

    def timed(fn, steps):
        with torch.cuda.stream(stream):
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            torch.cuda.synchronize()
        return e0.elapsed_time(e1)
    print(json.dumps({"probe": "moe", **moe_bench(S, dev, stream, torch, timed)}), flush=True)


def moe_bench(S, dev, stream, torch, timed_ms):
    H, E, F, USED = 2048, 256, 512, 8
    M = S.Matrix.from_packed
    f = S.MoeFfn(M(dev, E, H, 1, Q8_0, random_matrix(Q8_0, E, H, 900)),
                 M(dev, F, H, E, Q4_K, random_matrix(Q4_K, E * F, H, 901)), M(dev, F, H, E, Q4_K, random_matrix(Q4_K, E * F, H, 902)),
                 M(dev, H, F, E, Q6_K, random_matrix(Q6_K, E * H, F, 903)),
                 M(dev, F, H, 1, Q4_K, random_matrix(Q4_K, F, H, 904)), M(dev, F, H, 1, Q4_K, random_matrix(Q4_K, F, H, 905)),
                 M(dev, H, F, 1, Q6_K, random_matrix(Q6_K, H, F, 906)), None, E, USED, H, F, F, False, True)
    per_expert = 2 * (F * H // 256 * 144) + H * F // 256 * 210
    router_bytes = E * H // 32 * 34
    res = {}
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1234)  # the same tokens, hence the same routing, in every run
    for T in (1, 1024):
        x = (torch.randn(T * H, device="cuda", generator=gen) * 0.12).contiguous()
        scratch = torch.zeros(S.moe_ffn_scratch_elems(dev, f, T), dtype=torch.float32, device="cuda")
        o = torch.zeros(T * H, dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        dev.capture_begin()
        S.moe_ffn(dev, f, x, T, scratch, o)
        g = dev.capture_end()
        with torch.cuda.stream(stream):
            for _ in range(3):
                g.launch()
        reps = 20
        ms = min(timed_ms(g.launch, reps) for _ in range(3)) / reps
        touched = (min(E, T * USED) if T == 1 else E) * per_expert + per_expert + router_bytes
        flops = 2.0 * T * (USED + 1) * 3 * F * H
        res[f"t{T}"] = {"us": round(ms * 1e3, 1), "weight_gbs": round(touched / (ms * 1e-3) / 1e9, 1),
                        "tflops": round(flops / (ms * 1e-3) / 1e12, 2), "weight_bytes": touched}
        if T > 1:
            # Where the block's time goes: the library's own per-operation table over five eager passes (device
            # time between each operation's first and last kernel; operations on the side stream overlap the rest).
            dev.set_profiling(True)
            for _ in range(5):
                S.moe_ffn(dev, f, x, T, scratch, o)
            table = dev.take_profile()
            dev.set_profiling(False)
            res[f"t{T}"]["profile_us"] = {k: round(v["gpu_ns"] / max(1, v["gpu_samples"]) / 1e3 * (v["calls"] / 5), 1) for k, v in table.items()}
    # The same model's Q8_0 output head at M = 1 (65,536 of its 151,936 rows: 142 MB, larger than L2).
    rows = 65536
    head = M(dev, rows, H, 1, Q8_0, random_matrix(Q8_0, rows, H, 907))
    x = (torch.randn(H, device="cuda") * 0.12).contiguous()
    yh = torch.zeros(rows, dtype=torch.float32, device="cuda")
    dev.capture_begin()
    S.project(dev, head, x, 1, yh)
    g = dev.capture_end()
    with torch.cuda.stream(stream):
        for _ in range(3):
            g.launch()
    ms = timed_ms(g.launch, 20) / 20
    res["q8_0_head_m1"] = {"us": round(ms * 1e3, 1), "gbs": round(rows * (H // 32 * 34) / (ms * 1e-3) / 1e9, 1)}
    return res


# ---------------------------------------------------------------------------------------------------
# CPU baseline / reference arm
# ---------------------------------------------------------------------------------------------------

def cpu_layer(seed0=0):
    mats = []
    for i, (name, rows, cols, fmt) in enumerate(LAYER):
        mats.append((name, rows, cols, fmt, random_matrix(fmt, rows, cols, seed=seed0 + i)))
    return mats


def cpu_pass(ref, mats, xs, m, threads):
    for name, rows, cols, fmt, packed in mats:
        ref.gemv_threads(fmt, packed, rows, cols, xs[cols], m, threads)


def cpu_baseline(m, budget_s):
    from oracle import ref  # the CPU oracle is executed here only to be timed as the baseline
    threads = os.cpu_count() or 1
    mats = cpu_layer()
    rng = np.random.default_rng(1234)
    xs = {c: rng.standard_normal((m, c)).astype(np.float32) for c in (5120, 6144, 17408)}
    cpu_pass(ref, mats, xs, m, threads)  # warm-up
    best, t_start, reps = None, time.perf_counter(), 0
    while reps < 2 or (time.perf_counter() - t_start < budget_s and reps < 20):
        t0 = time.perf_counter()
        cpu_pass(ref, mats, xs, m, threads)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
        reps += 1
    return {"value": round(LAYER_BYTES / best / 1e9, 3), "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"one layer ({LAYER_BYTES} packed bytes) at M={m}, best of {reps} passes, "
                      f"C restatement of the reference's CPU dequant + fp32 dot, {threads} threads"}


def run_reference(args):
    """The reference's CPU path for the same step: `--layers` distinct layers of the layer set per step, `--steps`
    timed steps after `--warmup`, on all host cores (the oracle restatement; the reference itself is a macOS-only
    Rust/Metal crate and cannot be built here)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import ref  # the reference arm is the CPU oracle, timed
    threads = os.cpu_count() or 1
    m, layers = args.m, args.layers
    stack = [cpu_layer(seed0=7 * l) for l in range(layers)]
    rng = np.random.default_rng(1234)
    xs = {c: rng.standard_normal((m, c)).astype(np.float32) for c in (5120, 6144, 17408)}

    def step():
        for mats in stack:
            cpu_pass(ref, mats, xs, m, threads)
    steps, warm = args.steps, max(args.warmup, 1)
    for _ in range(warm):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    total = layers * LAYER_BYTES
    value = round(total / dt / 1e9, 3)
    sample = (f"each step = {layers} distinct layers ({total} packed bytes) at M={m} on {threads} host threads; the C restatement of "
              f"the reference's CPU dequant + fp32 dot")
    print(json.dumps({
        "impl": "reference", "metric": "Q4_K_M decode projection weight GB/s (27B-class dense layer set)",
        "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps, "warmup": warm,
        "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"cfg1 dense 27B decode projection set (q,k,v,o,gate,up Q4_K; down Q6_K), M={m}, "
                               f"{layers} distinct layers = {total} packed bytes per step, on the host cores", "m": m, "layers": layers},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def run_prefill_probe(args):
    """One matrix of the layer set at M bf16 activation rows, `steps` launches: the small case a profiler
    capture of the prefill kernel runs on.  Prints the mean device time per launch."""
    import torch
    from ferrum_b200 import surface as S

    name, m = args.prefill_probe.split(":")
    m = int(m)
    _, rows, cols, fmt = next(e for e in LAYER if e[0] == name)
    torch.cuda.set_device(0)
    dev = S.Device(0, use_torch_stream=False)
    stream = torch.cuda.ExternalStream(dev.stream_ptr(), device=torch.device("cuda", 0))
    w = S.Matrix.from_packed(dev, rows, cols, 1, fmt, random_matrix(fmt, rows, cols, seed=3))
    x = torch.randn(m * cols, device="cuda").to(torch.bfloat16)
    y = torch.zeros(m * rows, dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            S.project(dev, w, x, m, y)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            S.project(dev, w, x, m, y)
        e1.record()
        torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / args.steps
    print(json.dumps({"probe": "prefill", "matrix": name, "rows": rows, "cols": cols, "m": m, "us_per_launch": round(us, 2),
                      "tflops": round(2.0 * rows * cols * m / us / 1e6, 1)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--m", type=int, default=1, help="activation rows (1 = decode)")
    ap.add_argument("--layers", type=int, default=3, help="one GPU: distinct layers streamed per step")
    ap.add_argument("--tp-layers", type=int, default=0, help="more GPUs: layers of the row-sharded stack (default 64)")
    ap.add_argument("--eager", action="store_true", help="enqueue every step call by call instead of replaying a graph")
    ap.add_argument("--no-fuse", action="store_true", help="one launch per matrix instead of one per input group")
    ap.add_argument("--nccl", action="store_true", help="multi-GPU: gather with NCCL (torch.distributed) instead of the peer-push kernel")
    ap.add_argument("--quick", action="store_true", help="headline and per-group timings only")
    ap.add_argument("--stream-probe", action="store_true", help="time a kernel that only reads 100 MB buffers: the read-only streaming ceiling")
    ap.add_argument("--moe-probe", action="store_true", help="time only the MoE block (T = 1 and 1024) and the Q8_0 head")
    ap.add_argument("--prefill-probe", default=None, metavar="NAME:M",
                    help="time only the bf16 prefill GEMM of one matrix of the layer set (q, k, o, gate, down ...) at M rows")
    args = ap.parse_args()
    if args.stream_probe:
        run_stream_probe(args)
    elif args.moe_probe:
        run_moe_probe(args)
    elif args.prefill_probe:
        run_prefill_probe(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
