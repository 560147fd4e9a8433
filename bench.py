"""Benchmark of the sparse-convolution forward path (rulebook generation +
convolution) on the SECOND-style backbone.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c2]

A step is one forward pass of the 12-layer backbone (8 rulebooks, 12
convolutions) over one batch of synthetic voxels through the C ABI of
libmluops_b200.so.  At N GPUs every rank runs its own batch of 4 samples x
120,000 voxels (weak scaling: samples are independent), then the final features
and out_indices of all ranks are gathered on rank 0 with NCCL.

Printed (rank 0, one JSON line):
  value      active input voxels per second, inputs already resident in HBM
  e2e        the same metric with host buffers: pinned host -> device copies of
             the step's indices and features and the device -> host read of the
             final features and out_indices are inside the timed region
  roofline   the kernel with the largest share of device time: algorithmic bytes
             per launch / measured duration, against the measured HBM bandwidth
  cpu_baseline  the reference's CPU implementation of the path, one core, on a
             bounded sample (one sample of the workload)

--impl reference times the CPU implementation of the path on all host cores, on
the same workload (the full batch, every sample at its full size): the C
restatement built for speed as the line's value, and one pass of the
reference's own single-threaded code (oracle/_ref) beside it.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "active voxels/sec for sparse-conv fwd incl. indice pairs"
UNIT = "voxels/s"
HBM_FALLBACK_GBS = 6650.0
TENSOR_FALLBACK_TFLOPS = 1400.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", TENSOR_FALLBACK_TFLOPS)), "measured"
    return HBM_FALLBACK_GBS, TENSOR_FALLBACK_TFLOPS, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 25 ms while running."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = str(gpu_index)
        self.lines = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits", "-lms", "25",
                 "-i", self.gpu_index], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self, t_begin=None, t_end=None):
        """Summary of the samples taken between the two wall-clock times (all samples if none given)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        import datetime
        sm, smax, power = [], [], []
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                stamp = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                if t_begin is not None and not (t_begin - 0.05 <= stamp <= t_end + 0.05):
                    continue
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm), "power_w_max": max(power) if power else None}


# Folder (under the repository root) for the files a diagnostic run writes.
OUT_DIR = os.environ.get("BENCH_OUT_DIR", "gpurun_out")

# Size of the pieces in which the end-to-end steps copy their results to the host.  The rulebook
# counts the host waits for reach it as stores of a kernel over the same PCIe link, behind whatever
# piece is on its way: 1 MiB keeps that delay at 20-60 us (measured: 4.37 ms per step with 4 MiB
# pieces, 4.32 with 1 MiB, 5.08 with 256 KiB, whose 170 copy launches cost the host 1 ms).
D2H_CHUNK_BYTES = int(os.environ.get("BENCH_D2H_CHUNK", 1 << 20))


def gpu_cpu_affinities():
    """{gpu index: CPU ids the driver reports as local to it} from `nvidia-smi topo -m` (column
    "CPU Affinity"); empty when the tool or the column is missing."""
    try:
        out = subprocess.run(["nvidia-smi", "topo", "-m"], capture_output=True, text=True, timeout=20).stdout
    except (OSError, subprocess.SubprocessError):
        return {}
    header, found = None, {}
    for line in out.splitlines():
        cols = [c.strip() for c in line.split("\t") if c.strip()]
        if not cols:
            continue
        if header is None and any(c.startswith("CPU Affinity") for c in cols):
            header = cols
            continue
        if header is not None and cols[0].startswith("GPU") and cols[0][3:].isdigit():
            # data rows have one more leading column (the row label) than the header
            at = [i for i, c in enumerate(header) if c.startswith("CPU Affinity")][0] + 1
            if at >= len(cols):
                continue
            cpus = set()
            for part in cols[at].split(","):
                lo, _, hi = part.partition("-")
                if lo.isdigit():
                    cpus.update(range(int(lo), int(hi or lo) + 1))
            if cpus:
                found[int(cols[0][3:])] = sorted(cpus)
    return found


def pin_rank_to_cores(local_rank, local_world, gpu_index, gpu_indices=None):
    """Binds this process to its share of the cores that are local to its GPU (falling back to an
    even split of all cores), before any pinned host buffer is allocated, so that the buffers
    land on that socket's memory.  Ranks whose GPUs report the same set of local cores divide
    that set among themselves by their position in the group.  `gpu_indices`: the GPU of every
    local rank (default: rank r uses GPU r).  Returns the description that goes into the JSON line."""
    try:
        allowed = sorted(os.sched_getaffinity(0))
    except AttributeError:
        return None
    affinities = gpu_cpu_affinities()
    local = [c for c in affinities.get(gpu_index, []) if c in allowed]
    if local:
        gpus = list(gpu_indices) if gpu_indices is not None else list(range(local_world))
        same = [r for r, g in enumerate(gpus) if affinities.get(g) == affinities.get(gpu_index)]
        if local_rank not in same:
            same = sorted(same + [local_rank])
        share = max(1, len(local) // len(same))
        first = same.index(local_rank) * share
        mine, how = local[first:first + share], "cores local to the GPU"
    else:
        share = max(1, len(allowed) // local_world)
        mine, how = allowed[local_rank * share:(local_rank + 1) * share], "even split of all cores"
    if not mine:
        return None
    os.sched_setaffinity(0, mine)
    return "%s: %d-%d (%d)" % (how, mine[0], mine[-1], len(mine))


def read_trace(ops):
    """Parses the library's kernel trace into {name: (launches, total_ms, bytes, flops)}."""
    lib = ops.lib()
    buf = ctypes.create_string_buffer(1 << 16)
    lib.mluOpTraceKernelReport(buf, len(buf), None)
    rows = {}
    for line in buf.value.decode().splitlines()[1:]:
        name, launches, ms, nbytes, flops = line.rsplit(",", 4)
        rows[name] = (int(launches), float(ms), float(nbytes), float(flops))
    return rows


def run_b200(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry

    ops, workloads, backbone = entry.load_package()
    import importlib
    sharding = importlib.import_module("mluops_b200.sharding")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path for the product)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    pinned = None
    if world > 1 and not args.no_pin_cores:
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        local_world = int(os.environ.get("LOCAL_WORLD_SIZE", world))
        ids = [int(v) for v in visible.split(",")] if visible and all(v.strip().isdigit() for v in visible.split(",")) else []
        gpus = ids[:local_world] if len(ids) >= local_world else list(range(local_world))
        pinned = pin_rank_to_cores(local_rank, local_world, gpus[local_rank], gpus)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    cfg = workloads.CONFIGS[args.workload]
    batch = cfg["batch"]
    grid = list(cfg["grid"])
    # every rank draws its own samples (seed offset by rank); weights are shared
    if args.workload == "c4":
        assert batch % world == 0, "c4 shards 16 samples over the ranks"
        batch //= world
    if args.workload == "c4":  # the ranks' shards of one fixed 16-sample job
        idx_np, feat_np, layers, weights_np = workloads.make_inputs("c4", batch=batch, first_sample=rank * batch)
    else:
        idx_np, feat_np, layers, weights_np = workloads.make_inputs(args.workload, batch=batch,
                                                                    seed=cfg["seed"] + 1000 * rank)
    L = idx_np.shape[0]
    elem = feat_np.dtype.itemsize

    stream = torch.cuda.current_stream()
    handle = ops.Handle(stream.cuda_stream)
    weights = [torch.from_numpy(w).to(dev) for w in weights_np]
    # Rulebooks depend only on coordinates: they run through a second handle on a second stream,
    # where the host waits for their counts while the convolutions already enqueued on the first
    # stream keep the GPU busy (--serial-rulebooks: everything on one stream).
    rb_stream = rb_handle = None
    if not args.serial_rulebooks:
        rb_stream = torch.cuda.Stream(dev)
        rb_handle = ops.Handle(rb_stream.cuda_stream)
    if args.config_only:
        # one configuration alone (profiling captures of a small case): its object, nothing else
        hbm_gbs, tensor_tflops, _ = measured_peaks()
        env = dict(torch=torch, dist=dist, ops=ops, workloads=workloads, backbone=backbone, sharding=sharding,
                   dev=dev, rank=rank, world=world, flush=torch.empty((256 << 20,), dtype=torch.uint8, device=dev),
                   stream=stream, handle=handle, rb_handle=rb_handle, rb_stream=rb_stream, flush_at=0,
                   pipelined=args.pipeline and rb_handle is not None, hbm_gbs=hbm_gbs,
                   tensor_tflops=tensor_tflops, fp32_tflops=64.0, batch_override=args.config_batch)
        print(json.dumps({args.config_only: time_config(args.config_only, args.steps, env)}))
        return
    net = backbone.SparseNetwork(handle, layers, weights, grid, batch, rulebook_handle=rb_handle,
                                 rulebook_stream=rb_stream)

    h_idx = torch.from_numpy(idx_np).pin_memory()
    h_feat = torch.from_numpy(feat_np).pin_memory()
    d_idx = torch.empty_like(h_idx, device=dev)
    d_feat = torch.empty_like(h_feat, device=dev)
    d_idx.copy_(h_idx)
    d_feat.copy_(h_feat)
    flush = torch.empty((256 << 20,), dtype=torch.uint8, device=dev)
    host_out = {}

    first_sample = rank * batch  # batch index of this rank's first sample in the whole job

    # Final features and out_indices of every rank -> rank 0 over NCCL (exact sizes): the row
    # counts and the coordinate rows leave on a second stream as soon as the last rulebook
    # exists, the feature rows after the last convolution.
    # the ranks' row counts travel host to host (a gloo group beside the NCCL one)
    host_group = dist.new_group(backend="gloo") if world > 1 else None
    gather = sharding.RowGather(first_sample, rank, world, device=dev, host_group=host_group)

    # The gather of step i is enqueued during step i+1, at the point of the layer loop where
    # the host would otherwise wait with the most convolution work queued on the GPU: its
    # host cost (three collectives) is hidden there and its NVLink traffic overlaps step
    # i+1's kernels.  The rows that are in flight are kept in `pending`.
    queued, best, flush_at = 0, -1, 0
    seen = set()
    for li, ly in enumerate(layers):
        if ly.rulebook not in seen:
            seen.add(ly.rulebook)
            if queued > best:
                best, flush_at = queued, li
            queued = 0
        queued += ly.ci * ly.co * ly.kernel_volume
    pending = []

    def flush_pending(li=None):
        if pending and (li is None or li == flush_at):
            out, out_idx, done = pending.pop()
            gather.begin(out_idx, ready=done)
            gather.finish(out, wait=False, ready=done)

    # With --pipeline a stream of batches is software-pipelined one level further: rulebooks
    # depend only on coordinates, so the rulebooks of batch i+1 (their kernels on the second stream
    # and the host waits for their counts) run while the convolutions of batch i, already enqueued,
    # keep the first stream busy.  Every step still does one batch's rulebooks and one batch's
    # convolutions inside the timed region; they just belong to neighbouring batches.
    pipelined = args.pipeline and rb_handle is not None
    next_plan = {}

    def step_resident():
        """One step of a stream of batches."""
        if pipelined:
            plan = next_plan.pop("resident", None) or net.plan_rulebooks(d_idx)
            if world > 1 and not args.no_gather:
                flush_pending()  # rows of the step before: their convolutions have long been enqueued
            out, out_idx, records = net.run_convolutions(plan, d_feat)
            if world > 1 and not args.no_gather:
                done = torch.cuda.Event()
                done.record(stream)
                pending.append((out, out_idx, done))
            next_plan["resident"] = net.plan_rulebooks(d_idx)
            return records
        if args.no_gather or world == 1:  # --no-gather: diagnostic, nothing crosses NVLink
            return net.forward(d_idx, d_feat)[2]
        out, out_idx, records = net.forward(d_idx, d_feat, on_host_idle=flush_pending)
        flush_pending()  # only when the layer list has no such point
        done = torch.cuda.Event()
        done.record(stream)
        pending.append((out, out_idx, done))
        return records

    # End-to-end steps are pipelined the way a serving loop would run them: while step i computes,
    # the inputs of step i+1 travel host -> device on a second stream (into the other half of a
    # double buffer) and the results of step i-1 travel device -> host on a third.  Every step
    # still pays for its own copies inside the timed region; they just overlap other steps' kernels.
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    d_in = [(d_idx, d_feat), (torch.empty_like(d_idx), torch.empty_like(d_feat))]
    in_ready, buf_free = [None, None], [None, None]
    out_pending = []
    e2e_state = {"i": 0}

    copy_events = None  # e2e breakdown: [(kind, start event, end event)]

    def prefetch(slot):
        if buf_free[slot] is not None:
            s_in.wait_event(buf_free[slot])  # the step that last read this half has finished
        with torch.cuda.stream(s_in):
            if copy_events is not None:
                e0 = torch.cuda.Event(enable_timing=True)
                e0.record(s_in)
            d_in[slot][0].copy_(h_idx, non_blocking=True)
            d_in[slot][1].copy_(h_feat, non_blocking=True)
            ev = torch.cuda.Event(enable_timing=copy_events is not None)
            ev.record(s_in)
            if copy_events is not None:
                copy_events.append(("h2d", e0, ev))
        in_ready[slot] = ev

    def read_back():
        while out_pending:
            out, out_idx, done, slot = out_pending.pop(0)
            key = (slot, out.shape[0], out.shape[1])
            if key not in host_out:
                host_out[key] = (torch.empty(out.shape, dtype=out.dtype).pin_memory(),
                                 torch.empty(out_idx.shape, dtype=out_idx.dtype).pin_memory())
            s_out.wait_event(done)
            with torch.cuda.stream(s_out):
                if copy_events is not None:
                    e0 = torch.cuda.Event(enable_timing=True)
                    e0.record(s_out)
                # in pieces: the step's own small device -> host reads (rulebook counts) share the
                # copy engine with this transfer and would otherwise wait for all of it
                rows = max(1, D2H_CHUNK_BYTES // (out.shape[1] * elem))
                for r0 in range(0, out.shape[0], rows):
                    host_out[key][0][r0:r0 + rows].copy_(out[r0:r0 + rows], non_blocking=True)
                host_out[key][1].copy_(out_idx, non_blocking=True)
                if copy_events is not None:
                    e1 = torch.cuda.Event(enable_timing=True)
                    e1.record(s_out)
                    copy_events.append(("d2h", e0, e1))
            out.record_stream(s_out)
            out_idx.record_stream(s_out)

    def drain():
        flush_pending()
        gather.wait()
        read_back()
        stream.wait_stream(s_out)
        stream.wait_stream(s_in)  # a prefetch for a step that never came must not outlive the region

    def step_e2e(host=None):
        """Host buffers in, host buffers out: pinned-host -> device copies of this rank's
        indices and features, the layer stack, the NCCL gather, and the device -> host read
        of this rank's final features and out_indices (every rank reads its own rows back
        over its own PCIe link, in parallel)."""
        slot = e2e_state["i"] % 2
        e2e_state["i"] += 1
        if in_ready[slot] is None:
            prefetch(slot)      # very first step: nothing was prefetched yet
        copies = {"done": False}

        def enqueue_copies(li=None):
            """Inputs of the next step in, results of the previous step out: enqueued where the host
            would otherwise sit waiting for a rulebook with the most convolution work queued (a third
            of a millisecond of copy launches that, done before the step, left the GPU idle)."""
            t_a = time.perf_counter()
            if not copies["done"] and (li is None or li == flush_at):
                copies["done"] = True
                prefetch(1 - slot)
                read_back()
            t_b = time.perf_counter()
            if world > 1 and not args.no_gather and not pipelined:
                flush_pending(li)
            if host is not None:
                host["prefetch_and_readback_enqueue_s"] += t_b - t_a
                host["gather_enqueue_s"] += time.perf_counter() - t_b
        if pipelined:
            enqueue_copies()
        idx_in, feat_in = d_in[slot]
        if pipelined:
            plan = next_plan.pop(("e2e", slot), None) or net.plan_rulebooks(idx_in, ready=in_ready[slot])
            stream.wait_event(in_ready[slot])
            in_ready[slot] = None
            if not args.no_gather:
                gather.begin(plan.out_indices, ready=plan.done)  # the coordinates can leave before the convolutions
            out, out_idx, records = net.run_convolutions(plan, feat_in)
            if not args.no_gather:
                gather.finish(out, wait=True)
        else:
            stream.wait_event(in_ready[slot])
            in_ready[slot] = None
            # like the resident steps: the rows of the step before leave for rank 0 at the point of
            # this step where the host would otherwise sit waiting for a rulebook, so neither the
            # collectives' host cost nor their NVLink traffic holds up a step; the last step's
            # gather is waited for before the region's closing event (drain)
            t_f = time.perf_counter()
            out, out_idx, records = net.forward(idx_in, feat_in, on_host_idle=enqueue_copies)
            enqueue_copies()  # only when the layer list has no such point
            if host is not None:
                host["forward_s"] += time.perf_counter() - t_f  # includes the two enqueue phases
        done = torch.cuda.Event()
        done.record(stream)
        buf_free[slot] = done
        if world > 1 and not args.no_gather and not pipelined:
            pending.append((out, out_idx, done))
        out_pending.append((out, out_idx, done, slot))
        if pipelined:
            # rulebooks of the next batch (its inputs are on their way since the start of this step)
            next_plan[("e2e", 1 - slot)] = net.plan_rulebooks(d_in[1 - slot][0], ready=in_ready[1 - slot])
        return records, (out.shape[0] * out.shape[1] * elem + out_idx.shape[0] * 16)

    def timed(step, steps):
        """One region of `steps` steps between two CUDA events on the launching stream,
        bracketed by a barrier and a device synchronize on both sides.  L2 is flushed after
        every step inside the region (its 256 MiB write is part of the measured time), and the
        last step's gather is waited for before the closing event.  Returns the region's ms."""
        flush.fill_(1)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(stream)
        for _ in range(steps):
            step()
            flush.fill_(1)
        drain()
        t1.record(stream)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        return t0.elapsed_time(t1)

    # the sampler starts before the warm-up (nvidia-smi needs a moment to come up); only
    # the samples that fall inside the timed regions are summarised
    sampler = ClockSampler(local_rank if "CUDA_VISIBLE_DEVICES" not in os.environ else
                           os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local_rank])
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step_resident()
        step_e2e()
    drain()
    torch.cuda.synchronize()
    t_begin = time.time()
    res_ms = timed(step_resident, args.steps)
    d2h = [0]

    def e2e_once():
        _, nbytes = step_e2e()
        d2h[0] = nbytes
    e2e_ms = timed(e2e_once, args.steps)
    clocks = sampler.stop(t_begin, time.time()) if rank == 0 else None

    if args.e2e_breakdown:
        # Where an end-to-end step spends its time on this rank: host seconds per phase
        # (perf_counter around the calls) and device time of the copies (events on their streams).
        copy_events = []
        net.timers = {}
        host = {"prefetch_and_readback_enqueue_s": 0.0, "gather_enqueue_s": 0.0, "forward_s": 0.0, "step_s": 0.0}

        def step_instrumented():
            t0 = time.perf_counter()
            step_e2e(host)
            host["step_s"] += time.perf_counter() - t0

        region_ms = timed(step_instrumented, args.steps)
        torch.cuda.synchronize()
        sums = {"h2d": [], "d2h": []}
        for kind, e0, e1 in copy_events:
            sums[kind].append(e0.elapsed_time(e1))
        n = args.steps
        report = {"rank": rank, "world": world, "pinned": pinned, "steps": n, "e2e_ms_per_step": round(region_ms / n, 4),
                  "host_ms_per_step": {k: round(v / n * 1e3, 4) for k, v in host.items()},
                  "rulebook_wait_ms_per_step": round(net.timers.get("rulebook_wait_s", 0.0) / n * 1e3, 4),
                  "h2d_ms": {"mean": round(sum(sums["h2d"]) / max(1, len(sums["h2d"])), 4),
                             "max": round(max(sums["h2d"] or [0]), 4), "bytes": int(h_idx.numel() * 4 + h_feat.numel() * elem)},
                  "d2h_ms": {"mean": round(sum(sums["d2h"]) / max(1, len(sums["d2h"])), 4),
                             "max": round(max(sums["d2h"] or [0]), 4), "bytes": int(d2h[0])}}
        net.timers = None
        copy_events = None
        os.makedirs(os.path.join(ROOT, OUT_DIR), exist_ok=True)
        with open(os.path.join(ROOT, OUT_DIR, "e2e_breakdown_rank%d_of_%d.json" % (rank, world)), "w") as f:
            json.dump(report, f)

    # traced pass: per-kernel durations (CUDA events around every launch) and launch counts
    ops.lib().mluOpTraceKernelReset()
    ops.lib().mluOpTraceKernelEnable(1)
    records = None
    for _ in range(args.steps):
        flush.fill_(1)
        records = step_resident()
    drain()
    torch.cuda.synchronize()
    trace = read_trace(ops)
    ops.lib().mluOpTraceKernelEnable(0)

    # the other configurations: c4 (strong scaling of one 16-sample job) at every N, the
    # single-layer configurations c0 / c1 / c3 on one GPU
    hbm_gbs, tensor_tflops, peak_kind = measured_peaks()
    extra = {}
    if args.workload == "c2" and not args.headline_only:
        fp32_tflops = measure_fp32_fma_peak(torch, dev) if world == 1 else None
        env = dict(torch=torch, dist=dist, ops=ops, workloads=workloads, backbone=backbone, sharding=sharding,
                   dev=dev, rank=rank, world=world, flush=flush, stream=stream, handle=handle, rb_handle=rb_handle,
                   rb_stream=rb_stream, flush_at=flush_at, pipelined=pipelined, hbm_gbs=hbm_gbs, tensor_tflops=tensor_tflops,
                   fp32_tflops=fp32_tflops, host_group=host_group)
        extra["c4"] = time_config("c4", max(5, args.steps // 2), env)
        if world == 1:
            extra["per_config"] = {name: time_config(name, max(5, args.steps // 2), env) for name in ("c0", "c1", "c3")}
            extra["fp32_fma_peak_tflops"] = round(fp32_tflops, 2)

    def reduce_max(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ranks_ms = [res_ms / args.steps]
    if world > 1:
        t = torch.zeros((world,), dtype=torch.float64, device=dev)
        t[rank] = res_ms / args.steps
        dist.all_reduce(t)
        ranks_ms = [round(x, 4) for x in t.tolist()]
    total_res = reduce_max(res_ms)
    total_e2e = reduce_max(e2e_ms)
    if world > 1:
        t = torch.tensor([d2h[0]], dtype=torch.int64, device=dev)
        dist.all_reduce(t)
        d2h[0] = int(t.item())
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    voxels = L * world * args.steps
    value = voxels / (total_res * 1e-3)
    e2e_value = voxels / (total_e2e * 1e-3)

    kernels = {k: v for k, v in trace.items() if not k.startswith(("memset:", "memcpy:"))}
    gpu_launches = sum(v[0] for v in kernels.values()) // args.steps
    total_kernel_ms = sum(v[1] for v in trace.values())
    top = max(kernels.items(), key=lambda kv: kv[1][1])
    top_name, (top_launches, top_ms, top_bytes, top_flops) = top
    achieved = (top_bytes / top_launches) / ((top_ms / top_launches) * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                "frac": round(achieved / hbm_gbs, 4), "traffic": None, "traffic_kind": None,
                "kernel": top_name, "launches_per_step": top_launches // args.steps,
                "avg_launch_ms": round(top_ms / top_launches, 5), "peak_source": peak_kind + " copy bandwidth",
                "share_of_device_time": round(top_ms / total_kernel_ms, 4),
                "tensor_tflops_achieved": round(top_flops / (top_ms * 1e-3) / 1e12, 2)}

    # whole-step roofline: sum over layers of max(flops/peak, bytes/BW) + rulebook bytes / BW
    conv_rows, pair_bytes = backbone.roofline_bytes_and_flops(records, elem)
    if top_name.startswith("convTcgen05Kernel<"):
        ci_co = top_name[top_name.index("<") + 1:-1].split(",")
        same = [dict(c, K=rec.layer.kernel_volume) for c, rec in zip(conv_rows, records)
                if c["ci"] == int(ci_co[0]) and c["co"] == int(ci_co[1])]
        roofline["traffic"] = modelled_conv_traffic(same, elem)
        roofline["traffic_kind"] = ("modelled: one ncu capture of this kernel (dram bytes read + written) scaled to "
                                    "this run's launches by rows_in*Ci*2 + rows_out*Co*2 + 4*K*rows_out; not "
                                    "measured in this run")
    t_roof = sum(max(c["flops"] / (tensor_tflops * 1e12), c["bytes"] / (hbm_gbs * 1e9)) for c in conv_rows)
    t_roof += pair_bytes / (hbm_gbs * 1e9)
    ms_per_step = total_res / args.steps
    whole = {"t_roof_ms": round(t_roof * 1e3, 4), "frac_resident": round(t_roof * 1e3 / ms_per_step, 4),
             "frac_e2e": round(t_roof * 1e3 / (total_e2e / args.steps), 4),
             "conv_bytes": sum(c["bytes"] for c in conv_rows), "conv_flops": sum(c["flops"] for c in conv_rows),
             "rulebook_bytes": pair_bytes, "pairs_per_step": sum(c["P"] for c in conv_rows)}

    line = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "strong" if args.workload == "c4" else "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": "%s: SECOND-style sparse backbone (12 convs, 8 rulebooks), batch %d x %d voxels "
                               "per GPU, grid %dx%dx%d, fp16 storage / fp32 accumulate" %
                               (args.workload, batch, cfg["per_sample"], *grid),
                   "voxels_per_gpu": L, "l2": "flushed after every step (256 MiB write, inside the timed region)",
                   "rulebooks": "same stream as the convolutions" if args.serial_rulebooks else
                                ("second handle on a second stream; the rulebooks of batch i+1 run during the "
                                 "convolutions of batch i (every step holds one batch of each)" if pipelined else
                                 "second handle on a second stream, overlapping the convolutions of earlier layers"),
                   "e2e_pipeline": "inputs of step i+1 and results of step i-1 are copied on two more streams while "
                                   "step i computes; every step's copies are inside the timed region",
                   "parallelism": ("batch samples per rank, NO gather (diagnostic)" if args.no_gather else "batch samples per rank; NCCL gather of final rows to rank 0 on a second stream, overlapping the next step") if world > 1 else "1 GPU"},
        "e2e": {"value": round(e2e_value, 1), "unit": UNIT,
                "h2d_bytes_per_step": int(h_idx.numel() * 4 + h_feat.numel() * elem) * world,
                "d2h_bytes_per_step": int(d2h[0]), "ms_per_step": round(total_e2e / args.steps, 4)},
        "gpu_launches": int(gpu_launches),
        "ranks_ms_per_step": ranks_ms, "host_cores": os.cpu_count(), "rank0_cores": pinned,
        "clocks": clocks,
        "roofline": roofline,
        "roofline_whole_step": whole,
        "layers": [{"ci": c["ci"], "co": c["co"], "sub_m": c["sub_m"], "n_in": c["n_in"], "n_out": c["n_out"],
                    "pairs": c["P"]} for c in conv_rows],
        "kernels": {k: {"launches_per_step": v[0] // args.steps, "ms_per_step": round(v[1] / args.steps, 4)}
                    for k, v in sorted(trace.items(), key=lambda kv: -kv[1][1])},
    }
    if "c4" in extra:
        line["c4"] = extra["c4"]
    if "per_config" in extra:
        line["per_config"] = extra["per_config"]
        line["fp32_fma_peak_tflops"] = {"value": extra["fp32_fma_peak_tflops"],
                                        "how": "8192^3 float matmul, TF32 off, best of 5, CUDA events, this run"}
    if world == 1 and args.backward:
        line["training"] = training_step(args, ops, backbone, net, d_idx, d_feat, flush, elem, hbm_gbs,
                                         tensor_tflops)
    if world == 1 and (args.fast_path or (args.workload == "c2" and not args.headline_only)):
        def step_fast():
            if pipelined:
                plan = next_plan.pop("fast", None) or net.plan_rulebooks(d_idx, reuse_tables=True)
                net.run_convolutions(plan, d_feat)
                next_plan["fast"] = net.plan_rulebooks(d_idx, reuse_tables=True)
            else:
                net.forward(d_idx, d_feat, reuse_tables=True, defer_counts=True)
        for _ in range(3):
            step_fast()
        fast_ms = timed(step_fast, args.steps) / args.steps
        line["fast_path"] = {"ms_per_step": round(fast_ms, 4), "value": round(L / (fast_ms * 1e-3), 1), "unit": UNIT,
                             "what": "one neighbour table per rulebook instead of one per convolution call; "
                                     "submanifold rulebooks emit their table themselves and are not waited for "
                                     "on the host"}
    if world == 1 and args.voxelization:
        line["voxelization"] = voxelization_step(args, ops, handle, flush, hbm_gbs)
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_one_sample(args.workload)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def measure_fp32_fma_peak(torch, dev):
    """FP32 FMA throughput of this GPU (TFLOP/s): an 8192^3 float matmul with TF32 switched
    off (the reference forbids TF32 for this path's matmul, reference
    kernels/sparse_conv/indice_convolution_forward/indice_convolution_forward.cpp:227-234),
    best of five, CUDA events.  It is the denominator of the fp32 configuration's flop term,
    measured the way the bf16 figure of MEASURED_PEAKS.json was."""
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        n = 8192
        a = torch.randn((n, n), dtype=torch.float32, device=dev)
        b = torch.randn((n, n), dtype=torch.float32, device=dev)
        c = torch.empty_like(a)
        best = None
        for i in range(6):
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            torch.matmul(a, b, out=c)
            t1.record()
            torch.cuda.synchronize()
            ms = t0.elapsed_time(t1)
            if i > 0 and (best is None or ms < best):
                best = ms
        return 2.0 * n ** 3 / (best * 1e-3) / 1e12
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


def time_config(name, steps, env):
    """One more configuration beside the headline: `steps` passes of its layer list (rulebook
    generation + convolutions through the C ABI, inputs resident), its whole-step roofline from
    the run's own pair counts and its dominant kernel from a traced pass.

    c0 / c1 / c3 (one layer each, 1 GPU): every step sits between its own pair of CUDA events
    and L2 is flushed between steps, outside the events.  c4 (the backbone at 16 x 150,000
    voxels, strong scaling): the 16 samples are split over the ranks, the final rows are
    gathered on rank 0 with NCCL as in the headline run, and the steps are timed as one
    region (barrier + synchronize on both sides, L2 flush inside), max over ranks."""
    torch, dist = env["torch"], env["dist"]
    ops, workloads, backbone, sharding = env["ops"], env["workloads"], env["backbone"], env["sharding"]
    dev, rank, world, flush, stream = env["dev"], env["rank"], env["world"], env["flush"], env["stream"]
    cfg = workloads.CONFIGS[name]
    batch, sharded = cfg["batch"], name == "c4"
    if sharded:
        assert batch % world == 0
        batch //= world
        # the shards of one fixed 16-sample job: rank r draws samples [r*batch, (r+1)*batch)
        idx_np, feat_np, layers, weights_np = workloads.make_inputs(name, batch=batch, first_sample=rank * batch)
    else:
        if env.get("batch_override"):
            batch = int(env["batch_override"])
        idx_np, feat_np, layers, weights_np = workloads.make_inputs(name, batch=batch)
    L = idx_np.shape[0]
    elem = feat_np.dtype.itemsize
    weights = [torch.from_numpy(w).to(dev) for w in weights_np]
    net = backbone.SparseNetwork(env["handle"], layers, weights, list(cfg["grid"]), batch,
                                 rulebook_handle=env["rb_handle"], rulebook_stream=env["rb_stream"])
    d_idx, d_feat = torch.from_numpy(idx_np).to(dev), torch.from_numpy(feat_np).to(dev)
    gather = sharding.RowGather(rank * batch, rank, world, device=dev, host_group=env.get("host_group")) if sharded and world > 1 else None
    pending = []

    def flush_pending(li=None):
        if pending and (li is None or li == env["flush_at"]):
            out, out_idx, done = pending.pop()
            gather.begin(out_idx, ready=done)
            gather.finish(out, wait=False, ready=done)

    next_plan = {}

    def step():
        if env["pipelined"]:  # rulebooks of the next batch during this batch's convolutions, as in the headline
            plan = next_plan.pop("plan", None) or net.plan_rulebooks(d_idx)
            if gather is not None:
                flush_pending()
            out, out_idx, records = net.run_convolutions(plan, d_feat)
            if gather is not None:
                done = torch.cuda.Event()
                done.record(stream)
                pending.append((out, out_idx, done))
            next_plan["plan"] = net.plan_rulebooks(d_idx)
            return records
        if gather is None:
            return net.forward(d_idx, d_feat)[2]
        out, out_idx, records = net.forward(d_idx, d_feat, on_host_idle=flush_pending)
        flush_pending()
        done = torch.cuda.Event()
        done.record(stream)
        pending.append((out, out_idx, done))
        return records

    def drain():
        if gather is not None:
            flush_pending()
            gather.wait()

    for _ in range(3):
        step()
    drain()
    torch.cuda.synchronize()
    if sharded:
        flush.fill_(1)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(stream)
        for _ in range(steps):
            step()
            flush.fill_(1)
        drain()
        t1.record(stream)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = t0.elapsed_time(t1) / steps
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        timing = "one region of %d steps, L2 flush inside, max over ranks" % steps
    else:
        times = []
        for _ in range(steps):
            flush.fill_(1)
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record(stream)
            step()
            t1.record(stream)
            torch.cuda.synchronize()
            times.append(t0.elapsed_time(t1))
        ms = sum(times) / len(times)
        timing = "mean of %d steps, each between its own events, L2 flushed between steps" % steps
    if env["pipelined"]:
        timing += "; rulebooks of batch i+1 during the convolutions of batch i"

    ops.lib().mluOpTraceKernelReset()
    ops.lib().mluOpTraceKernelEnable(1)
    records = None
    for _ in range(min(steps, 5)):
        flush.fill_(1)
        records = step()
    drain()
    torch.cuda.synchronize()
    trace = read_trace(ops)
    ops.lib().mluOpTraceKernelEnable(0)
    traced = min(steps, 5)
    net.close()
    if rank != 0:
        return None

    is_half = feat_np.dtype.itemsize == 2
    flop_peak = env["tensor_tflops"] if is_half else env["fp32_tflops"]
    conv_rows, pair_bytes = backbone.roofline_bytes_and_flops(records, elem)
    t_roof = sum(max(c["flops"] / (flop_peak * 1e12), c["bytes"] / (env["hbm_gbs"] * 1e9)) for c in conv_rows)
    t_roof += pair_bytes / (env["hbm_gbs"] * 1e9)
    kernels = {k: v for k, v in trace.items() if not k.startswith(("memset:", "memcpy:"))}
    top_name, (top_n, top_ms, top_bytes, top_flops) = max(kernels.items(), key=lambda kv: kv[1][1])
    total_ms = sum(v[1] for v in trace.values())
    achieved = top_bytes / (top_ms * 1e-3) / 1e9
    return {
        "workload": "%s: batch %d x %d voxels%s, %s" % (
            name, batch * (world if sharded else 1), cfg["per_sample"], " split over %d ranks" % world if sharded and world > 1 else "",
            "12-layer backbone" if len(layers) > 1 else "one %s convolution %d -> %d, %s" % (
                "submanifold" if layers[0].sub_m else "strided", layers[0].ci, layers[0].co, cfg["dtype"])),
        "value": round(L * world / (ms * 1e-3), 1) if sharded else round(L / (ms * 1e-3), 1), "unit": UNIT,
        "ms_per_step": round(ms, 4), "timing": timing, "voxels": L * (world if sharded else 1),
        "pairs_per_step": sum(c["P"] for c in conv_rows), "n_out": records[-1].n_out,
        "t_roof_ms": round(t_roof * 1e3, 4), "roofline_frac": round(t_roof * 1e3 / ms, 4),
        "flop_peak_tflops": round(flop_peak, 1), "scaling": "strong" if sharded else None,
        "dominant_kernel": {"name": top_name, "launches_per_step": top_n // traced,
                            "avg_launch_ms": round(top_ms / top_n, 5),
                            "share_of_device_time": round(top_ms / total_ms, 4),
                            "algorithmic_GBps": round(achieved, 1), "frac_of_copy_bandwidth": round(achieved / env["hbm_gbs"], 4),
                            "tflops": round(top_flops / (top_ms * 1e-3) / 1e12, 2)},
        "kernels": {k: {"launches_per_step": v[0] // traced, "ms_per_step": round(v[1] / traced, 4)}
                    for k, v in sorted(trace.items(), key=lambda kv: -kv[1][1])},
    }


def voxelization_step(args, ops, handle, flush, hbm_gbs):
    """mluOpVoxelization on one synthetic frame: 300,000 points (x, y from a wide normal, z from a
    narrow one, one intensity), 0.05 x 0.05 x 0.1 m voxels over 80 x 80 x 4 m, at most 5 points per
    voxel and 160,000 voxels.  Algorithmic bytes: the points read once, the four outputs written once."""
    import numpy as np
    import torch
    rng = np.random.default_rng(0x70)
    n, f, mp, mv = 300000, 4, 5, 160000
    pts = np.concatenate([rng.normal(0, 18, (n, 2)), rng.normal(-1, 0.8, (n, 1)), rng.random((n, 1))], 1)
    d_pts = torch.from_numpy(pts.astype(np.float32)).cuda()
    d_vs = torch.tensor([0.05, 0.05, 0.1], dtype=torch.float32, device="cuda")
    d_cr = torch.tensor([-40, -40, -3, 40, 40, 1], dtype=torch.float32, device="cuda")
    ws = torch.empty((256 << 20,), dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream()
    for _ in range(3):
        out = ops.voxelization(handle, d_pts, d_vs, d_cr, mp, mv, workspace=ws)
    torch.cuda.synchronize()
    times = []
    for _ in range(args.steps):
        flush.fill_(1)
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(stream)
        out = ops.voxelization(handle, d_pts, d_vs, d_cr, mp, mv, workspace=ws)
        t1.record(stream)
        torch.cuda.synchronize()
        times.append(t0.elapsed_time(t1))
    ms = sum(times) / len(times)
    ops.lib().mluOpTraceKernelReset()
    ops.lib().mluOpTraceKernelEnable(1)
    for _ in range(args.steps):
        flush.fill_(1)
        ops.voxelization(handle, d_pts, d_vs, d_cr, mp, mv, workspace=ws)
    torch.cuda.synchronize()
    trace = read_trace(ops)
    ops.lib().mluOpTraceKernelEnable(0)
    # dynamic voxelization of the same frame: integer coordinates on the same grid, mean of the features
    lo, size = np.array([-40, -40, -3], dtype=np.float32), np.array([0.05, 0.05, 0.1], dtype=np.float32)
    c = np.floor((pts[:, :3].astype(np.float32) - lo) / size).astype(np.int32)[:, ::-1]
    c[np.any((c < 0) | (c >= np.array([40, 1600, 1600])), 1)] = -1
    d_coors0 = torch.from_numpy(np.ascontiguousarray(c)).cuda()
    d_coors = d_coors0.clone()
    for _ in range(3):
        dyn = ops.dynamic_point_to_voxel_forward(handle, d_pts, d_coors, "mean", workspace=ws)
    torch.cuda.synchronize()
    dyn_times = []
    for _ in range(args.steps):
        flush.fill_(1)
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(stream)
        dyn = ops.dynamic_point_to_voxel_forward(handle, d_pts, d_coors, "mean", workspace=ws)
        t1.record(stream)
        torch.cuda.synchronize()
        dyn_times.append(t0.elapsed_time(t1))
    dyn_ms = sum(dyn_times) / len(dyn_times)
    algo = n * f * 4 + mv * mp * f * 4 + mv * 12 + mv * 4 + 4
    dyn_voxels = int(dyn[4].item())
    dyn_algo = n * f * 4 + n * 12 + n * 4 + dyn_voxels * (f * 4 + 12 + 4)
    dynamic = {"voxel_num": dyn_voxels, "ms": round(dyn_ms, 4), "points_per_s": round(n / (dyn_ms * 1e-3), 1),
               "algorithmic_bytes": dyn_algo, "GBps": round(dyn_algo / (dyn_ms * 1e-3) / 1e9, 1)}
    return {"points": n, "dynamic_point_to_voxel_mean": dynamic, "voxel_num": int(out[3].item()), "ms": round(ms, 4), "points_per_s": round(n / (ms * 1e-3), 1),
            "algorithmic_bytes": algo, "GBps": round(algo / (ms * 1e-3) / 1e9, 1),
            "frac_of_copy_bandwidth": round(algo / (ms * 1e-3) / 1e9 / hbm_gbs, 4),
            "kernels": {k: {"launches": v[0] // args.steps, "ms": round(v[1] / args.steps, 4)}
                        for k, v in sorted(trace.items(), key=lambda kv: -kv[1][1])}}


def training_step(args, ops, backbone, net, d_idx, d_feat, flush, elem, hbm_gbs, tensor_tflops):
    """Forward (rulebooks + convolutions) followed by the input and filter gradients of every
    layer, timed like the forward step; per-kernel times from a traced pass.  The roofline of
    the backward half is twice the forward's convolution term (same pairs, same bytes and
    flops per pair for each of the two gradients)."""
    import torch
    stream = torch.cuda.current_stream()

    def step(tables=False):
        out, _, records = net.forward(d_idx, d_feat, keep=True, reuse_tables=tables)
        grad = torch.ones_like(out)
        net.backward(records, grad, reuse_tables=tables)
        return records

    def time_steps(tables):
        for _ in range(3):
            step(tables)
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        flush.fill_(1)
        torch.cuda.synchronize()
        t0.record(stream)
        for _ in range(args.steps):
            step(tables)
            flush.fill_(1)
        t1.record(stream)
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / args.steps

    ms = time_steps(False)
    # the same step through the table extensions: one forward and one input table per rulebook
    ms_tables = time_steps(True)
    ops.lib().mluOpTraceKernelReset()
    ops.lib().mluOpTraceKernelEnable(1)
    records = None
    for _ in range(args.steps):
        flush.fill_(1)
        records = step()
    torch.cuda.synchronize()
    trace = read_trace(ops)
    ops.lib().mluOpTraceKernelEnable(0)
    conv_rows, pair_bytes = backbone.roofline_bytes_and_flops(records, elem)
    t_conv = sum(max(c["flops"] / (tensor_tflops * 1e12), c["bytes"] / (hbm_gbs * 1e9)) for c in conv_rows)
    t_roof = 3 * t_conv + pair_bytes / (hbm_gbs * 1e9)
    return {"ms_per_step": round(ms, 4), "t_roof_ms": round(t_roof * 1e3, 4), "frac": round(t_roof * 1e3 / ms, 4),
            "fast_path": {"ms_per_step": round(ms_tables, 4), "frac": round(t_roof * 1e3 / ms_tables, 4),
                          "what": "neighbour tables built once per rulebook and shared by its layers' forward "
                                  "convolutions, input gradients and (64 input channels) filter gradients: "
                                  "extensions with no counterpart in the reference"},
            "kernels": {k: {"launches_per_step": v[0] // args.steps, "ms_per_step": round(v[1] / args.steps, 4),
                            "GBps": round(v[2] / (v[1] * 1e-3) / 1e9, 1) if v[1] > 0 else None,
                            "TFLOPs": round(v[3] / (v[1] * 1e-3) / 1e12, 2) if v[1] > 0 else None}
                        for k, v in sorted(trace.items(), key=lambda kv: -kv[1][1])}}


# DRAM traffic of the tensor-core convolution kernel.  One ncu capture measured dram__bytes_read.sum +
# dram__bytes_write.sum = 370.9 MB for the launch with 1,079,296 padded rows in and out, 64 -> 64 channels, 27
# offsets; the kernel streams features once, writes outputs once and reads the neighbour table once, i.e.
# rows_in*Ci*2 + rows_out*Co*2 + 4*K*rows_out = 392.9 MB by that model.  Other launches of the kernel are scaled by
# the same measured/model ratio (traffic grows in proportion to rows).
MEASURED_OVER_MODEL_TRAFFIC = 370.9e6 / (1079296 * (64 * 2 + 64 * 2 + 4 * 27))


def modelled_conv_traffic(layer_rows, elem):
    """Average DRAM bytes per launch over the given layers ({ci, co, n_in, n_out, K})."""
    if not layer_rows:
        return None
    total = 0.0
    for c in layer_rows:
        total += c["n_in"] * c["ci"] * elem + c["n_out"] * c["co"] * elem + 4.0 * c["K"] * c["n_out"]
    return round(MEASURED_OVER_MODEL_TRAFFIC * total / len(layer_rows), 0)


def cpu_backend():
    import oracle
    return ("reference", True) if oracle.ref_lib() is not None else ("port", False)


def cpu_baseline_one_sample(workload):
    """The reference's CPU implementation of the path on one sample of the workload, one core."""
    import __graft_entry__ as entry
    _, workloads, _ = entry.load_package()
    import oracle
    from oracle import backbone_cpu
    oracle.build()
    kind, use_ref = cpu_backend()
    cfg = workloads.CONFIGS[workload]
    idx, feat, layers, weights = workloads.make_inputs(workload, batch=1)
    t0 = time.perf_counter()
    backbone_cpu.run_layers(idx, feat, layers, weights, cfg["grid"], 1, True, use_ref=use_ref, fast=not use_ref)
    dt = time.perf_counter() - t0
    return {"value": round(idx.shape[0] / dt, 1), "unit": UNIT, "cores": 1, "kind": kind,
            "sample": "one sample of the workload (%d voxels, batch 1), full 12-layer backbone, %.1f s" %
                      (idx.shape[0], dt)}


_REF_CACHE = {}


def _reference_inputs(workload):
    """The workload's full batch, split by sample (batch index relabelled to 0), cached per process."""
    if workload not in _REF_CACHE:
        import numpy as np
        import __graft_entry__ as entry
        _, workloads, _ = entry.load_package()
        cfg = workloads.CONFIGS[workload]
        idx, feat, layers, weights = workloads.make_inputs(workload)
        samples = []
        for b in range(cfg["batch"]):
            rows = idx[:, 0] == b
            local = idx[rows].copy()
            local[:, 0] = 0
            samples.append((np.ascontiguousarray(local), np.ascontiguousarray(feat[rows])))
        _REF_CACHE[workload] = (samples, layers, weights, cfg["grid"])
    return _REF_CACHE[workload]


def _reference_sample(task):
    """One full-size sample of the workload through the CPU layer stack.
    mode "port": the C restatement, vectorised, the pairs of an offset shared among this
    process's OpenMP threads.  mode "reference": the reference's own function bodies, one thread."""
    workload, sample, mode = task
    from oracle import backbone_cpu
    samples, layers, weights, grid = _reference_inputs(workload)
    idx, feat = samples[sample % len(samples)]
    t0 = time.perf_counter()
    if mode == "reference":
        backbone_cpu.run_layers(idx, feat, layers, weights, grid, 1, True, use_ref=True)
    else:
        backbone_cpu.run_layers(idx, feat, layers, weights, grid, 1, True, threads=True)
    return idx.shape[0], time.perf_counter() - t0


def run_reference(args):
    """Reference arm: the CPU implementation of the path on all host cores, on the SAME
    workload as the other arm (the full batch, every sample at its full size).

    A step is one pass over the batch: one process per sample, the host's cores divided
    among them as OpenMP threads, running the C restatement of the reference's CPU code
    built for speed (-O3, AVX2, OpenMP; bit-identical to its scalar build).  That is the
    line's `value` (kind "port").  The reference's own function bodies are single-threaded
    and take about 35 s per sample, so they are timed beside it in one pass only
    ("reference_code": one full-size sample per core, all cores busy)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import multiprocessing as mp
    import __graft_entry__ as entry
    _, workloads, _ = entry.load_package()
    import oracle
    oracle.build()
    cores = os.cpu_count() or 1
    cfg = workloads.CONFIGS[args.workload]
    batch = cfg["batch"]
    workers = max(1, min(batch, cores))
    threads = max(1, cores // workers)
    os.environ["OMP_NUM_THREADS"] = str(threads)  # inherited by the workers, read when OpenMP starts
    warmup = max(args.warmup, 1)
    ctx = mp.get_context("fork")
    times, voxels = [], 0
    with ctx.Pool(workers) as pool:
        pool.map(_reference_inputs, [args.workload] * workers, chunksize=1)  # generate the inputs once per worker
        # every step is the whole batch at full size; so that the run still ends within a few
        # minutes, no more steps are timed than fit about 150 s (at least 3)
        steps_timed = args.steps
        for step in range(warmup + args.steps):
            if step >= warmup + steps_timed:
                break
            t0 = time.perf_counter()
            results = pool.map(_reference_sample, [(args.workload, b, "port") for b in range(batch)], chunksize=1)
            dt = time.perf_counter() - t0
            if step == warmup - 1:
                steps_timed = min(args.steps, max(3, int(150.0 / max(dt, 1e-3))))
            if step >= warmup:
                times.append(dt)
                voxels += sum(r[0] for r in results)
    total = sum(times)
    value = voxels / total
    sample = ("the full batch per step: %d samples x %d voxels, one process per sample with %d OpenMP threads each, "
              "full 12-layer backbone" % (batch, cfg["per_sample"], threads))
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "steps_timed": len(times), "warmup": warmup,
        "ms_per_step": round(total / len(times) * 1e3, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "%s: SECOND-style sparse backbone (12 convs, 8 rulebooks), batch %d x %d voxels, grid "
                               "%dx%dx%d, CPU implementation of the reference's algorithm, fp32 arithmetic on "
                               "half-rounded values" % (args.workload, batch, cfg["per_sample"], *cfg["grid"]),
                   "voxels_per_step": batch * cfg["per_sample"]},
        "cpu_baseline": {"value": round(value, 1), "unit": UNIT, "cores": workers * threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": round(value, 1), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "host_cores": cores,
    }
    if oracle.ref_lib() is not None and not args.no_reference_code:
        procs = max(1, cores)
        try:
            import psutil
            procs = max(1, min(procs, int(psutil.virtual_memory().available / (3 << 30))))
        except Exception:
            pass
        os.environ["OMP_NUM_THREADS"] = "1"
        with ctx.Pool(procs) as pool:
            t0 = time.perf_counter()
            results = pool.map(_reference_sample, [(args.workload, b, "reference") for b in range(procs)], chunksize=1)
            dt = time.perf_counter() - t0
        line["reference_code"] = {
            "value": round(sum(r[0] for r in results) / dt, 1), "unit": UNIT, "cores": procs, "kind": "reference",
            "per_core": round(sum(r[0] / r[1] for r in results) / procs, 1),
            "sample": "one pass: %d processes, each one full-size sample (%d voxels) through the reference's own "
                      "single-threaded function bodies, %.1f s" % (procs, cfg["per_sample"], dt)}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c2", "c4"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--config-only", default=None, choices=["c0", "c1", "c3", "c4"],
                    help="time this configuration alone and print its object (profiling captures of a small case)")
    ap.add_argument("--config-batch", type=int, default=None,
                    help="with --config-only c0/c1/c3: number of samples instead of the configuration's own")
    ap.add_argument("--no-reference-code", action="store_true",
                    help="--impl reference: skip the one-pass timing of the reference's own single-threaded code")
    ap.add_argument("--headline-only", action="store_true",
                    help="skip the c0 / c1 / c3 / c4 objects that the default line carries beside the c2 headline")
    ap.add_argument("--backward", action="store_true",
                    help="1 GPU: also time forward + backward (input and filter gradients of every layer) and "
                         "add a \"training\" object with its per-kernel times to the JSON line")
    ap.add_argument("--fast-path", action="store_true",  # (the default c2 line carries it anyway)
                    help="1 GPU: also time the step with one neighbour table per rulebook "
                         "(mluOpBuildIndiceNeighbourTable + mluOpIndiceConvolutionForwardFromTable, extensions with no "
                         "counterpart in the reference) and add a \"fast_path\" object to the JSON line")
    ap.add_argument("--voxelization", action="store_true",
                    help="1 GPU: also time mluOpVoxelization on a synthetic 300,000-point LiDAR-like frame and add a "
                         "\"voxelization\" object to the JSON line")
    ap.add_argument("--serial-rulebooks", action="store_true",
                    help="run the rulebooks on the same stream as the convolutions instead of a second one")
    ap.add_argument("--no-pin-cores", action="store_true",
                    help="N>1: do not bind each rank to the cores local to its GPU")
    ap.add_argument("--e2e-breakdown", action="store_true",
                    help="also write e2e_breakdown_rank<r>_of_<n>.json into the output folder (BENCH_OUT_DIR): where "
                         "each rank's end-to-end step spends "
                         "its host time (rulebook waits, library calls, copies) and how long its copies take")
    ap.add_argument("--pipeline", action="store_true",
                    help="generate the rulebooks of batch i+1 during the convolutions of batch i instead of inside "
                         "their own step (measured: no gain on one GPU, where the two kinds of kernels already share "
                         "the SMs through the second stream and the step is bound by their total kernel time)")
    ap.add_argument("--no-gather", action="store_true",
                    help="diagnostic for N>1: skip the NCCL gather (independent replicas) to separate its cost "
                         "from host-side contention between the ranks' processes")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
