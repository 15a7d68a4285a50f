#!/usr/bin/env python
"""Benchmark of the ViG forward (bi-GLA + block kernels) on B200: images/s, roofline of the scan kernel,
end-to-end number through the public API with host buffers, and the CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload vig_t_1024|vig_s_224|vig_t_224]
    python bench.py --impl reference ...        # the reference's CPU path (oracle port) on the host cores

Under torchrun (N > 1) every rank runs the same per-GPU batch on its own GPU (image shards, no collective
on the data path); time is the max over ranks of CUDA-event time; rank 0 prints one JSON line.
Protocol follows the reference's ``throughput()`` (classification/main.py:389-406): eval mode, one fixed
batch, warm-up forwards, then timed forwards.  Data are synthetic N(0,1) images and seeded random weights.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (preset, image size, per-GPU batch)
    "vig_t_1024": ("vig_t_dk64", 1024, 64),
    "vig_s_224": ("vig_s_dk64", 224, 128),
    "vig_t_224": ("vig_t_dk64", 224, 128),
    # the reference's shipped head size (EXPAND_K 0.5 -> dk = 32, classification/configs/vig/vig-t.yaml:13)
    "vig_t_1024_dk32": ("vig_t", 1024, 64),
    "vig_s_224_dk32": ("vig_s", 224, 128),
    # ViG-B at 2048x2048 (L = 16384): under torchrun the token sequence of every image is split across the ranks
    # (boundary states + one conv halo row per block over NCCL); the batch is the same on every rank
    "vig_b_2048_seq": ("vig_b_dk64", 2048, 8),
}
SEQ_SPLIT = {"vig_b_2048_seq"}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="vig_t_1024", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=0, help="per-GPU batch (default: the workload's)")
    ap.add_argument("--graph", type=int, default=1, help="1 (default): the forward is captured once and replayed as a CUDA graph in the "
                    "timed regions (eager if the capture fails, and for the sequence-split workload, whose forward holds collectives); 0: eager")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-seq-split", action="store_true", help="skip the sequence-split measurement that multi-GPU runs append")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []
        self.t_mark = None                      # wall-clock start of the timed region: samples from then on are "under load"

    def mark(self):
        self.t_mark = time.time()

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.thread.join(timeout=2)
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        # the sampler is started before the warm-up (nvidia-smi takes a while to come up) and read from the start of the
        # timed region on; a region too short to catch a sample falls back to the warm-up's samples (same load)
        in_region = [ln for t, ln in self.lines if self.t_mark is None or t >= self.t_mark]
        for ln in in_region or [ln for _, ln in self.lines]:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx = float(f[1])
            except ValueError:
                continue
            for n, val in zip(names, f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "samples": len(sm), "reasons": sorted(reasons)}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def cpu_model_throughput(preset, size, seconds_cap=40.0):
    """The oracle (port of the reference's naive PyTorch path) on the host cores: images/s on one image."""
    import oracle
    torch.set_num_threads(os.cpu_count() or 1)
    shape = oracle.PRESETS[preset]
    sd = oracle.make_state_dict(shape, seed=0)
    img = oracle.make_images(1, size, seed=0)
    t0 = time.perf_counter()
    with torch.no_grad():
        oracle.vig_forward(sd, img, shape)
    dt = time.perf_counter() - t0
    return 1.0 / dt, dt


def cpu_baseline(preset, size, budget_s=12.0, max_images=8):
    """``cpu_baseline`` object of the product arm's line: the oracle timed on a bounded sample of the workload -- one
    untimed image (thread pool, first-touch allocations), then whole images until about ``budget_s`` seconds are spent."""
    _, first = cpu_model_throughput(preset, size)
    n, spent = 0, 0.0
    while n < max_images and (n == 0 or spent + spent / n <= budget_s):
        _, dt = cpu_model_throughput(preset, size)
        n, spent = n + 1, spent + dt
    return {"value": n / spent, "unit": "images/s", "cores": os.cpu_count() or 1, "kind": "port",
            "sample": f"{n} image{'s' if n != 1 else ''} of {size}x{size} through the CPU oracle (naive recurrent bi-GLA) in {spent:.1f} s, after one untimed image ({first:.1f} s)"}


def run_reference(args, rank):
    """Reference arm: the reference's own CPU implementation of the path (its naive recurrent bi-GLA inside its
    module graph, restated in ``oracle/``) on all host threads; one step = one image of the workload."""
    if rank != 0:
        return
    preset, size, batch = WORKLOADS[args.workload]
    ips, dt = cpu_model_throughput(preset, size)          # doubles as warm-up and as the cost probe
    budget = 150.0
    warm = max(0, min(args.warmup, int(0.2 * budget / dt)))
    steps = max(1, min(args.steps, int(0.8 * budget / dt)))
    for _ in range(warm):
        cpu_model_throughput(preset, size)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_model_throughput(preset, size)
    el = time.perf_counter() - t0
    value = steps / el
    cores = os.cpu_count() or 1
    sample = f"1 image of {size}x{size} per step ({steps} of the requested {args.steps} steps fit the time bound)"
    line = {"impl": "reference", "metric": "images_per_sec", "value": value, "unit": "images/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": warm, "ms_per_step": 1e3 * el / steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args, batch),
            "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "reference_gpu_path": "not run: the reference's GPU operators are Triton kernels (fla/ops/gla/*.py), a tracing "
                                  "compiler path this arm does not execute; this arm is its naive PyTorch recurrence on the host cores"}
    print(json.dumps(line), flush=True)


def workload_config(args, batch):
    preset, size, _ = WORKLOADS[args.workload]
    dk = 64 if preset.endswith("dk64") else 32
    return {"workload": f"{args.workload}: ViG {preset} forward, {size}x{size} images, patch 16 (L={(size // 16) ** 2}), "
                        f"batch {batch} per GPU, 12 blocks, dk={dk}, dv=64",
            "per_gpu_batch": batch, "image_size": size,
            "sharding": ("token sequence across GPUs by image rows (all-gather of boundary states and conv halo rows per block)"
                         if args.workload in SEQ_SPLIT else "images across GPUs, no collective"),
            "cache": "inputs and activations larger than L2 (126 MB)" if batch * 3 * size * size * 2 > 126e6 else "L2 flushed between steps"}


def main():
    args = parse()
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    import torch.distributed as dist
    import oracle
    import vig_b200
    from vig_b200 import ops as vops

    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    preset, size, batch = WORKLOADS[args.workload]
    batch = args.batch or batch
    shape = oracle.PRESETS[preset]
    model = vig_b200.ViG.from_shape(shape)
    model.load_state_dict(oracle.make_state_dict(shape, seed=0))
    model = model.to(dev, torch.bfloat16).eval()
    seq_split = args.workload in SEQ_SPLIT and world > 1
    host_images = oracle.make_images(min(batch, 8), size, seed=0 if args.workload in SEQ_SPLIT else rank).to(torch.bfloat16)
    host_images = host_images.repeat((batch + host_images.shape[0] - 1) // host_images.shape[0], 1, 1, 1)[:batch].contiguous().pin_memory()
    images = host_images.to(dev)
    host_logits = torch.empty(batch, shape.num_classes, dtype=torch.bfloat16).pin_memory()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev) if batch * 3 * size * size * 2 <= 126e6 else None

    # count launches of this library's kernels and time the scan operator with events on its stream
    counts = {"launches": 0}
    scan_events = []
    timing = {"on": False}
    orig = {n: getattr(vops, n) for n in ("bi_gla", "dwconv3x3", "gate_inject", "add_rmsnorm", "swiglu", "linear_swiglu",
                                          "linear_add_rmsnorm", "layernorm_act", "stem_unfold", "stem_fold", "stem_conv_ln", "linear_bias")
            if hasattr(vops, n)}
    L = (size // 16) ** 2
    nseg = (L + 255) // 256                       # 256-token segments of the tensor-core scan
    scan_launches = 1 if nseg == 1 or 8 <= nseg <= 32 else 3   # one persistent launch, or states + scan + outputs

    def wrap(name, n_launch):
        fn = orig[name]

        def inner(*a, **k):
            counts["launches"] += n_launch
            if name == "bi_gla" and timing["on"]:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                r = fn(*a, **k)
                e1.record()
                scan_events.append((e0, e1))
                return r
            return fn(*a, **k)
        return inner

    for n in orig:
        w = wrap(n, scan_launches if n == "bi_gla" else 1)
        setattr(vops, n, w)
        if hasattr(vig_b200, n):
            setattr(vig_b200, n, w)

    from vig_b200 import seqsplit

    def forward(x):
        with torch.no_grad():
            return seqsplit.vig_forward_sequence_parallel(model, x) if seq_split else model(x)

    def step():
        if flush is not None:
            flush.fill_(1)
        return forward(images)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # before anything is timed: the scan at the workload's shape, default routing against the three-launch tensor-core form
    # on the same seeded inputs (two different kernels of the product; the oracle is not involved)
    output_check = scan_self_check(vig_b200, batch, shape.num_heads, L, shape.key_dim // shape.num_heads,
                                   shape.value_dim // shape.num_heads, dev)
    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    vops.check_status()          # no kernel reported a run-out wait or an out-of-range gate during warm-up
    graph = None
    e2e_graphs = None
    if args.graph and not seq_split:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_out = step()
        except Exception as exc:                            # a failed capture leaves the eager path intact
            sys.stderr.write(f"bench: CUDA graph capture failed ({exc}); running eagerly\n")
            graph = None
            torch.cuda.synchronize()
    sync_all()
    counts["launches"] = 0
    timing["on"] = graph is None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    sampler.mark()
    e0.record()
    for _ in range(args.steps):
        if graph is not None:
            graph.replay()
        else:
            step()
    e1.record()
    sync_all()
    timing["on"] = False
    vops.check_status()          # ... nor inside the timed region (read after it, outside the timing)
    ms = e0.elapsed_time(e1)
    if graph is not None:
        # a replayed graph has no per-call events: the scan operator is timed with events around every call of three
        # eager steps run right after the timed region (same stream, same inputs, same neighbouring kernels)
        timing["on"] = True
        for _ in range(3):
            step()
        timing["on"] = False
        sync_all()
    launches = counts["launches"] if graph is None else None
    clocks = sampler.stop()
    if graph is not None:                                   # launches per replay = launches of one eager step
        counts["launches"] = 0
        step()
        launches = counts["launches"] * args.steps
        torch.cuda.synchronize()

    # end to end through the public API: every step copies its images from pinned host memory to the device,
    # runs the forward and copies the logits back.  The upload of step i+1 runs on a copy stream while step i
    # computes (two device buffers), as a serving loop would do it; all copies are inside the timed region.
    sync_all()
    copy_stream = torch.cuda.Stream(device=dev)
    main_stream = torch.cuda.current_stream()
    dbuf = [torch.empty_like(images), torch.empty_like(images)]
    uploaded = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]

    def upload(i):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[i % 2])          # the forward that last read this buffer is done
            dbuf[i % 2].copy_(host_images, non_blocking=True)
            uploaded[i % 2].record(copy_stream)

    if graph is not None:                                   # one captured forward per device buffer
        try:
            e2e_graphs, e2e_outs = [], []
            for k in range(2):
                gk = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gk):
                    ok = forward(dbuf[k])
                e2e_graphs.append(gk)
                e2e_outs.append(ok)
        except Exception as exc:
            sys.stderr.write(f"bench: CUDA graph capture of the end-to-end forward failed ({exc}); running it eagerly\n")
            e2e_graphs = None
            torch.cuda.synchronize()
    for ev in consumed:
        ev.record(main_stream)
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    f0.record()
    upload(0)
    for i in range(args.steps):
        if i + 1 < args.steps:
            upload(i + 1)
        main_stream.wait_event(uploaded[i % 2])
        if e2e_graphs is not None:
            e2e_graphs[i % 2].replay()
            out = e2e_outs[i % 2]
        else:
            out = forward(dbuf[i % 2])
        consumed[i % 2].record(main_stream)
        host_logits.copy_(out, non_blocking=True)
    f1.record()
    sync_all()
    vops.check_status()
    ms_e2e = f0.elapsed_time(f1)

    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(t[0]), float(t[1])

    # roofline of the scan operator: algorithmic bytes = (4 dk + 2 dv) * element size per token and head
    H, dk, dv = shape.num_heads, shape.key_dim // shape.num_heads, shape.value_dim // shape.num_heads
    alg_bytes = batch * H * L * (4 * dk + 2 * dv) * 2
    alg_flops = batch * H * L * 2 * (2 * 64 * dk + 2 * 64 * dv + 4 * dk * dv)
    if scan_events:
        scan_ms = sum(a.elapsed_time(b) for a, b in scan_events) / len(scan_events)
    else:                                                   # graph mode: time the operator alone, same shapes
        scan_ms = time_scan_alone(vig_b200, batch, H, L, dk, dv, dev)
    peak, peak_kind = peaks()
    achieved = alg_bytes / (scan_ms * 1e-3) / 1e9
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "bigla_traffic.json")
    if os.path.exists(tpath):
        with open(tpath) as f:
            tj = json.load(f)
        # same rule as the library's default routing (bigla_wave_preferred): the wavefront kernel for large batches
        sms = torch.cuda.get_device_properties(0).multi_processor_count
        entry = tj.get("wave") if (dk == 64 and dv == 64 and L > 256 and 2 * batch * H >= sms) else tj.get("single_launch")
        if dk != 64:
            entry = None                                    # the captures are of dk = dv = 64 calls
        per_unit = (entry or {}).get("dram_bytes_per_token_head")
        traffic = per_unit * batch * H * L if per_unit else None
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": traffic, "kernel": "bi-GLA scan operator (all launches of one call)", "peak_kind": peak_kind,
                "ms_per_launch": scan_ms, "algorithmic_bytes": alg_bytes,
                "timed_over": ("every scan call of the timed region (CUDA events on its stream)" if graph is None else
                               "every scan call of three eager steps run right after the timed region, which replays a CUDA graph "
                               "(CUDA events on its stream)"),
                "tensor_tflops_accounting": alg_flops / (scan_ms * 1e-3) / 1e12,
                "share_of_step": scan_ms * shape.depth / (ms / args.steps)}

    seq_split_line = None
    if world > 1 and args.workload == "vig_t_1024" and not args.no_seq_split:
        del model, images, dbuf
        torch.cuda.empty_cache()
        seq_split_line = run_seq_split(vig_b200, vops, oracle, dev, rank, world)
    if rank == 0:
        total_images = batch * (1 if args.workload in SEQ_SPLIT else world) * args.steps
        line = {"metric": "images_per_sec", "value": total_images / (ms * 1e-3), "unit": "images/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
                "scaling": "strong" if args.workload in SEQ_SPLIT else "weak", "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic", "config": workload_config(args, batch), "clocks": clocks, "gpu_launches": launches,
                "e2e": {"value": total_images / (ms_e2e * 1e-3), "unit": "images/s",
                        "h2d_bytes_per_step": host_images.numel() * 2, "d2h_bytes_per_step": host_logits.numel() * 2},
                "roofline": roofline, "graph": graph is not None, "output_check": output_check}
        if seq_split_line is not None:
            line["seq_split"] = seq_split_line
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(preset, size)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def scan_self_check(vig_b200, B, H, L, dk, dv, dev, bar=1e-2):
    """The bi-GLA operator at the benchmark's shape: default routing vs ``IMPL_TC_SPLIT`` on seeded inputs laid out as the
    block hands them over (strided views of packed projections, raw gate logits).  Raises if they differ by more than
    ``bar`` (max-norm relative; both are bf16 kernels with different summation orders)."""
    from vig_b200 import _lib
    gen = torch.Generator(device=dev).manual_seed(7)
    z = torch.randn(B, L, 2 * H * dk + H * dv, generator=gen, device=dev).to(torch.bfloat16)
    x = (2.0 * torch.randn(B, L, 2 * H * dk, generator=gen, device=dev)).to(torch.bfloat16)
    heads = lambda t, d: t.unflatten(-1, (H, d)).permute(0, 2, 1, 3)
    a = (heads(z[..., :H * dk], dk), heads(z[..., H * dk:2 * H * dk], dk), heads(z[..., 2 * H * dk:], dv),
         heads(x[..., :H * dk], dk), heads(x[..., H * dk:], dk))
    kw = dict(out_scale=0.25, gate_logit_normalizer=16.0)
    o = vig_b200.bi_gla(*a, **kw).float()
    o_ref = vig_b200.bi_gla(*a, impl=_lib.IMPL_TC_SPLIT, **kw).float()
    vig_b200.check_status()
    err = float((o - o_ref).abs().max() / o_ref.abs().max())
    if not err < bar:
        raise RuntimeError(f"scan self-check failed: default routing vs three-launch form differ by {err:.3e}")
    return {"scan_default_vs_three_launch_rel_err": err, "bar": bar, "shape": [B, H, L, dk, dv]}


def run_seq_split(vig_b200, vops, oracle, dev, rank, world, steps=5, warmup=3):
    """The second multi-GPU mode, measured in the same run: ViG-B at 2048x2048 (L = 16384), batch 8, the token sequence
    of every image split across the ranks by rows of the patch grid (per block: conv halo rows from the two neighbours,
    one all-gather of the per-head boundary states; one all-reduce for the pool).  Every rank holds the same images;
    times are CUDA-event times, max over ranks; the unsplit forward of the same batch on one GPU is timed beside it and
    the two results are compared."""
    import torch.distributed as dist
    from vig_b200 import seqsplit
    preset, size, batch = WORKLOADS["vig_b_2048_seq"]
    shape = oracle.PRESETS[preset]
    model = vig_b200.ViG.from_shape(shape)
    model.load_state_dict(oracle.make_state_dict(shape, seed=0))
    model = model.to(dev, torch.bfloat16).eval()
    images = oracle.make_images(batch, size, seed=0).to(dev, torch.bfloat16)

    def timed(fn):
        for _ in range(warmup):
            out = fn()
        torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            out = fn()
        e1.record()
        torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0]) / steps, out

    with torch.no_grad():
        ms_split, split = timed(lambda: seqsplit.vig_forward_sequence_parallel(model, images))
        vops.check_status()
        ms_one, whole = timed(lambda: model(images))
        vops.check_status()
        try:                                                # rank 0's view of where a split forward's time goes
            phases = seqsplit.phase_times(model, images)
        except Exception as exc:                            # a diagnostic: never in the way of the measurement
            sys.stderr.write(f"bench: phase times unavailable ({exc})\n")
            phases = None
    err = float((split.float() - whole.float()).abs().max() / whole.float().abs().max())
    line = {"workload": f"vig_b_2048_seq: ViG {preset} forward, {size}x{size} images (L={(size // 16) ** 2}), batch {batch}, "
                        "token sequence split across the GPUs", "n_gpus": world, "steps": steps, "warmup": warmup,
            "images_per_s": batch / (ms_split * 1e-3), "ms_per_step": ms_split,
            "single_gpu_images_per_s": batch / (ms_one * 1e-3), "single_gpu_ms_per_step": ms_one,
            "strong_scaling_efficiency": ms_one / (ms_split * world), "split_vs_unsplit_rel_err": err}
    if phases is not None:
        line["phases_ms_per_step"] = phases
    return line


def time_scan_alone(vig_b200, batch, H, L, dk, dv, dev, reps=10):
    q = torch.randn(batch, L, H * (2 * dk + dv), device=dev, dtype=torch.bfloat16)
    g = torch.randn(batch, L, 2 * H * dk, device=dev, dtype=torch.bfloat16)
    heads = lambda t, d: t.unflatten(-1, (H, d)).permute(0, 2, 1, 3)
    a = (heads(q[..., :H * dk], dk), heads(q[..., H * dk:2 * H * dk], dk), heads(q[..., 2 * H * dk:], dv),
         heads(g[..., :H * dk], dk), heads(g[..., H * dk:], dk))
    o = torch.empty(batch, L, H, dv, device=dev, dtype=torch.bfloat16).permute(0, 2, 1, 3)
    for _ in range(3):
        vig_b200.ops.bi_gla(*a, out=o, gate_logit_normalizer=16.0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        vig_b200.ops.bi_gla(*a, out=o, gate_logit_normalizer=16.0)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


if __name__ == "__main__":
    main()
