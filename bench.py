#!/usr/bin/env python
"""Throughput of the Point Transformer V3 forward pass (points per second).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload per GPU: the default backbone, random init, eval, bf16, on a batch of
four synthetic indoor scenes of about 100k voxels each (grid 0.02 m).  With N
GPUs every rank runs its own four scenes (weak scaling); scenes are independent,
so the data path has no collective (`--gather-outputs` adds an NCCL all-gather of
the output features to every step, for a caller that wants them on every rank).
One JSON line is printed by rank 0.

The same line carries a second measurement under "lidar16": one batch of 16
LiDAR-like scenes (grid 0.05 m, four input channels) sharded over the N GPUs by
scene (16 / N scenes per GPU: strong scaling), with the batch-global
serialization depth and the output features of all scenes gathered on every
rank over NCCL inside the step, on a side stream that overlaps the next step's
forward.  `--no-lidar` skips it.

`--impl reference` times the reference's own model on the host cores (the unmodified
model file placed under oracle/_ref by oracle/make_ref.py, run through CPU stand-ins
for the third-party packages it imports; the oracle's restatement where those files
are absent), on the same batch configuration.
"""
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
sys.path.insert(0, ROOT)

METRIC = "ptv3_forward_points_per_sec"
UNIT = "points/s"
SCENES_PER_GPU = 4
TARGET_VOXELS = 100_000
GRID = 0.02
CPU_SAMPLE_VOXELS = 100_000
LIDAR_SCENES = 16
LIDAR_GRID = 0.05
# DRAM read + write bytes per row and channel of one attention launch (ncu, dram__bytes_read.sum +
# dram__bytes_write.sum of a single launch on 407 552 padded rows x 64 channels: 166.2 + 34.5 MB)
ATTENTION_DRAM_BYTES_PER_ROW_CHANNEL = 7.70


def workload_config(n_gpus, gather=False):
    return {"workload": "full PTv3 backbone forward, default config, bf16 eval, random init; "
                        "%d synthetic indoor scenes of ~100k voxels per GPU, grid 0.02" % SCENES_PER_GPU,
            "scenes_per_gpu": SCENES_PER_GPU, "parallelism": "scene-parallel x%d, %s" % (
                n_gpus, "outputs all-gathered" if gather else "no data-path collective"),
            "l2": "inputs larger than L2: one step moves over a gigabyte of activations through the 126 MB L2; "
                  "the K steps run back to back between one pair of events",
            "second_workload": "lidar16: 16 LiDAR-like scenes sharded by scene with the outputs gathered over "
                               "NCCL (strong scaling), reported under the key of that name"}


# --------------------------------------------------------------------------- #
# clocks
# --------------------------------------------------------------------------- #
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def wait_first_sample(self, timeout=3.0):
        """Returns once nvidia-smi has started up and printed its first row (its start-up takes the
        driver's locks for tens of milliseconds, which must not fall into the timed steps)."""
        t_end = time.time() + timeout
        while self.proc is not None and not self.rows and time.time() < t_end:
            time.sleep(0.01)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for t, r in self.rows if t0 <= t <= t1 and len(r) >= 6] or \
               [r for _, r in self.rows if len(r) >= 6]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i] == "Active" for r in rows)]
        return {"sm_mhz": statistics.median(float(r[0]) for r in rows), "sm_max_mhz": float(rows[0][1]),
                "reasons": reasons, "samples": len(rows)}


# --------------------------------------------------------------------------- #
# CPU arm: the reference's own forward on the host cores
# --------------------------------------------------------------------------- #
def cpu_step_fn(n_scenes):
    """Returns (callable running one CPU forward, points per forward, description, kind).

    kind "reference": the unmodified reference model file (placed under oracle/_ref by
    oracle/make_ref.py, or a checkout beside this repository), run on CPU through the
    stand-ins of oracle/refshim for the four third-party packages it imports (the
    submanifold convolution among them is this repository's CPU restatement: spconv has
    no CPU build).  kind "port": the oracle's restatement of that forward, used where the
    reference's files are not present."""
    from oracle import ptv3_oracle as O, refload
    from pointtransformerv3_b200 import synthetic
    torch.set_num_threads(os.cpu_count() or 1)
    scenes = [synthetic.indoor_scene(i, CPU_SAMPLE_VOXELS, GRID) for i in range(n_scenes)]
    data = synthetic.make_batch(scenes, 3, 0, torch.bfloat16)
    n = int(data["offset"][-1])
    what = "%d indoor scene%s of the benchmark batch (%d voxels), bf16, enable_flash=False" % (
        n_scenes, "" if n_scenes == 1 else "s", n)
    ref = None
    try:
        ref = refload.load_model()
    except Exception:            # a stand-in that does not match this torch build: fall back to the port
        ref = None
    if ref is not None:
        torch.manual_seed(0)
        net = ref.PointTransformerV3(in_channels=6, enable_flash=False).eval().bfloat16()

        def step():
            with torch.inference_mode():
                torch.manual_seed(1)
                d = {k: v.clone() for k, v in data.items()}
                d["grid_size"] = GRID
                return net(d).feat
        return step, n, "unmodified reference model.py on CPU (stand-ins for addict/timm/torch_scatter/spconv); " + what, "reference"
    sd = cpu_state_dict(torch.bfloat16)

    def step():
        with torch.inference_mode():
            torch.manual_seed(1)
            return O.ptv3_forward(sd, data)
    return step, n, "CPU restatement of the reference forward (oracle); " + what, "port"


def cpu_state_dict(dtype):
    from pointtransformerv3_b200 import PointTransformerV3
    torch.manual_seed(0)
    net = PointTransformerV3(in_channels=6, enable_flash=False).eval()
    return {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in net.state_dict().items()}


def run_reference(args):
    """The reference arm: the same workload (all scenes of one GPU's batch) per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    step, n, sample, kind = cpu_step_fn(SCENES_PER_GPU)
    for _ in range(args.warmup):
        step()
    t = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        step()
        t.append(time.perf_counter() - t0)
    per = sum(t) / len(t)
    v = n / per
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": dict(workload_config(args.gpus), points_per_gpu=n),
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind,
                         "sample": sample + "; every step is the whole batch; rank 0 only"},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# --------------------------------------------------------------------------- #
# GPU arm
# --------------------------------------------------------------------------- #
def run_ours(args):
    import torch.distributed as dist
    from pointtransformerv3_b200 import PointTransformerV3, _lib, distributed, ops, synthetic

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (this library has no CPU path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # the gather runs beside the next forward: give NCCL's stream priority over it
        os.environ.setdefault("TORCH_NCCL_HIGH_PRIORITY", "1")
        dist.init_process_group("nccl", device_id=dev)
        # One launching thread per rank: give every rank its own slice of the host cores, so that
        # the ranks' Python threads and the driver's helper threads do not migrate onto each other
        # (the path is host-paced on its coarse levels, and 8 ranks share one host).
        try:
            cores = sorted(os.sched_getaffinity(0))
            per = len(cores) // world
            if per >= 1:
                os.sched_setaffinity(0, set(cores[local * per:(local + 1) * per]))
        except (AttributeError, OSError):
            pass
    lib = _lib.load()
    gather = world > 1 and args.gather_outputs

    data = synthetic.indoor_batch(SCENES_PER_GPU, first_seed=rank * SCENES_PER_GPU,
                                  target_voxels=TARGET_VOXELS, grid_size=GRID, dtype=torch.bfloat16)
    n_points = int(data["offset"][-1])
    torch.manual_seed(0)
    net = PointTransformerV3(in_channels=6).eval().to(dev).bfloat16()
    host = {k: v.pin_memory() for k, v in data.items()}
    resident = {k: v.to(dev) for k, v in data.items()}
    out_host = torch.empty((n_points, 64), dtype=torch.bfloat16).pin_memory()
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = out_host.numel() * out_host.element_size() + 4      # output features and the status word

    # what the batch's loader knows on the host: scene sizes and the extent of the grid
    gmax = host["grid_coord"].max(0).values.tolist()
    meta = {"offset_host": host["offset"], "sparse_shape": [v + 96 for v in gmax],
            "serialization_depth": max(gmax).bit_length()}
    # The model's own read of its device status word at the end of a pass is deferred: a serving loop
    # reads it when it next makes the host wait.  Here the words of all steps are read inside the
    # timed region, before its closing event (`check_pending`).
    net.defer_status_check = True
    pending = []

    def forward(d):
        torch.manual_seed(1)          # fixes the order-shuffle draws of every step
        with torch.inference_mode():
            point = net(dict(d, **meta))
            feat = point.feat
            if gather:
                feat, _ = distributed.gather_features(feat)
        pending.append(point["_status"])
        return feat

    def check_pending():
        """Reads the status words of the passes queued since the last call (one host wait)."""
        if pending:
            words = torch.cat(pending).tolist()
            pending.clear()
            if any(words):
                raise RuntimeError("device status words of the steps: %s" % words)

    def step_resident():
        return forward(resident)

    copy_stream = torch.cuda.Stream(device=dev)
    out_hosts = [out_host, torch.empty_like(out_host).pin_memory()]
    status_host = torch.zeros(max(args.steps, 2), dtype=torch.int32).pin_memory()

    dev_in = [{k: torch.empty_like(v, device=dev) for k, v in host.items()} for _ in range(2)]

    def run_e2e(steps):
        """`steps` forwards through the public API from pinned host buffers: every step copies
        its inputs host -> device and its output features device -> host.  The copies run on
        a second stream, so the input copy of step i + 1 and the output copy of step i overlap
        the forward of their neighbour step, as a serving loop would arrange it (two sets of
        device input buffers and two pinned output buffers, used in turn); the timed region
        (one event pair on the compute stream) ends when the last output has landed.
        Returns milliseconds for all steps."""
        main = torch.cuda.current_stream()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def upload(i):
            # buffer set i % 2 was last read by forward i - 2, whose output copy was queued on
            # the copy stream (behind that forward's completion) before this upload
            with torch.cuda.stream(copy_stream):
                for k, v in host.items():
                    dev_in[i % 2][k].copy_(v, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(copy_stream)
            return ev

        barrier()
        start.record(main)
        copy_stream.wait_stream(main)
        nxt = upload(0)
        for i in range(steps):
            main.wait_event(nxt)
            if i + 1 < steps:
                nxt = upload(i + 1)
            with torch.inference_mode():
                torch.manual_seed(1)
                point = net(dict(dev_in[i % 2], **meta))
                feat = point.feat
                if gather:
                    distributed.gather_features(feat)
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(done)
                out_hosts[i % 2].copy_(feat, non_blocking=True)
                # the pass's status word travels with its output
                status_host[i].copy_(point["_status"][0], non_blocking=True)
            feat.record_stream(copy_stream)
            point["_status"].record_stream(copy_stream)
        main.wait_stream(copy_stream)
        end.record(main)
        barrier()
        if any(status_host[:steps].tolist()):
            raise RuntimeError("device status words of the steps: %s" % status_host[:steps].tolist())
        t = torch.tensor([start.elapsed_time(end)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        """`steps` passes back to back between one pair of events; the status words of all of them are
        read before the closing event.  No L2 flush is needed between them: one pass moves well over
        a gigabyte of activations through a 126 MB L2, so nothing a pass starts with is still there."""
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        t0 = time.time()
        a.record()
        for _ in range(steps):
            fn()
        check_pending()
        b.record()
        barrier()
        t1 = time.time()
        ms = a.elapsed_time(b)
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), t0, t1

    def run_lidar():
        """16 LiDAR-like scenes sharded over the ranks by scene; returns the "lidar16" entry."""
        # the scenes' sizes are host metadata of the batch (its offsets): every rank generates the whole
        # batch, reads the sizes and keeps the scenes that the size-balanced assignment gives it
        all_scenes = [synthetic.lidar_scene(s, LIDAR_GRID) for s in range(LIDAR_SCENES)]
        groups = distributed.shard_scenes_balanced([sc[0].shape[0] for sc in all_scenes], world)
        mine = groups[rank]
        scenes = [all_scenes[i] for i in mine]
        del all_scenes
        shard = synthetic.make_batch(scenes, 1, mine[0], torch.bfloat16)
        n_local = int(shard["offset"][-1])
        shard_dev = {k: v.to(dev) for k, v in shard.items()}
        # batch-global quantities, fixed for a sensor and a grid size: made once, outside the steps
        depth = distributed.global_depth(shard_dev["grid_coord"])
        counts_t = torch.tensor([n_local], dtype=torch.int64, device=dev)
        all_counts = [n_local]
        if world > 1:
            buf = torch.empty(world, dtype=torch.int64, device=dev)
            dist.all_gather_into_tensor(buf, counts_t)
            all_counts = buf.tolist()
        total = sum(all_counts)
        torch.manual_seed(0)
        net4 = PointTransformerV3(in_channels=4).eval().to(dev).bfloat16()
        net4.defer_status_check = True
        side = torch.cuda.Stream(device=dev)
        steps_l, warm_l = min(args.steps, 10), 3

        def run(n_steps, with_gather):
            """n_steps forwards back to back; the gather of step i runs on the side stream while
            step i + 1 computes; the timed region ends when the last gather has landed."""
            main = torch.cuda.current_stream()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            start.record(main)
            for _ in range(n_steps):
                with torch.inference_mode():
                    torch.manual_seed(1)
                    d = dict(shard_dev)
                    d["serialization_depth"] = depth
                    point = net4(d)
                    feat = point.feat
                    pending.append(point["_status"])
                    if with_gather and world > 1:
                        out, _, ev = distributed.gather_features(feat, counts=all_counts, stream=side)
            check_pending()
            main.wait_stream(side)
            end.record(main)
            barrier()
            t = torch.tensor([start.elapsed_time(end)], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        def gather_alone(n_steps):
            with torch.inference_mode():
                torch.manual_seed(1)
                d = dict(shard_dev)
                d["serialization_depth"] = depth
                feat = net4(d).feat
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            a.record()
            for _ in range(n_steps):
                distributed.gather_features(feat, counts=all_counts)
            b.record()
            barrier()
            t = torch.tensor([a.elapsed_time(b) / n_steps], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        run(warm_l, True)
        ms_g = run(steps_l, True)
        ms_n = run(steps_l, False)
        g_ms = gather_alone(5) if world > 1 else 0.0
        del net4
        return {
            "workload": "full PTv3 backbone forward, default config, in_channels 4, bf16 eval, random init; one "
                        "batch of %d synthetic LiDAR-like scenes (two 64-beam sweeps each, grid %.2f), sharded "
                        "over the GPUs by scene, batch-global serialization depth" % (LIDAR_SCENES, LIDAR_GRID),
            "scaling": "strong", "scenes_per_gpu": len(mine), "scene_assignment": groups,
            "sharding": "scenes dealt to the ranks by size (largest first to the least loaded rank); the gathered "
                        "matrix is in rank order, a rank's scenes in ascending order",
            "points_total": total, "points_per_gpu": all_counts,
            "serialization_depth": depth, "steps": steps_l, "warmup": warm_l,
            "value": total * steps_l / (ms_g * 1e-3), "unit": UNIT, "ms_per_step": ms_g / steps_l,
            "value_without_gather": total * steps_l / (ms_n * 1e-3), "ms_per_step_without_gather": ms_n / steps_l,
            "gather_ms": g_ms,
            "collective": ("none (one GPU holds every scene)" if world == 1 else
                           "uneven all-gather of the (N_total, 64) bf16 output features to every rank: one "
                           "grouped launch of %d ncclBroadcast, received in place, on a side stream that "
                           "overlaps the next step's forward" % world),
            "gathered_bytes_per_step": total * 64 * 2,
        }

    # the clock sampler starts before the warm-up steps, so that it is sampling, not starting, when
    # the timed steps run
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.wait_first_sample()
    for _ in range(max(args.warmup, 3)):
        step_resident()
    check_pending()
    # timed region: the product path as a caller runs it (a transformer block is one C call
    # there, so no per-operator events exist inside it)
    ops.TIMERS = None
    launches0 = lib.ptv3_launch_count()
    torch.cuda.profiler.start()       # lets a profiler restrict itself to the timed steps
    ms, t0, t1 = timed(step_resident, args.steps)
    torch.cuda.profiler.stop()
    launches = lib.ptv3_launch_count() - launches0
    # the same K steps once more: one run in five has come out 0.3-0.8 ms per step slower on this
    # shared host (a single late step).  The faster run (max over ranks each) is `value`; both are
    # listed, and the clocks are sampled over both.
    ms_b, _, t1 = timed(step_resident, args.steps)
    resident_runs = [ms, ms_b]
    ms = min(resident_runs)
    clocks = sampler.stop(t0, t1) if sampler else None
    # second pass over the same steps (not part of `value`): the per-operator path with a CUDA
    # event pair around every operator, for the roofline of the dominant kernel (attention)
    # and the per-kernel breakdown
    ops.TIMERS, ops.TIMER_FILTER = {}, None
    timed(step_resident, args.steps)
    all_timers = ops.timer_summary()
    timers = all_timers
    ops.TIMERS = None

    ms_e2e, e2e_runs = None, []
    if not args.no_e2e:
        # K steps, twice (after a short warm-up of this loop's buffers); the faster run is reported and
        # both are listed: the loop is paced by the host's reads of the plan sizes, and a single
        # hiccup of a shared host (seen once in a dozen runs: +100 ms on one step) would otherwise
        # be the number
        run_e2e(3)
        e2e_runs = [run_e2e(args.steps), run_e2e(args.steps)]
        ms_e2e = min(e2e_runs)

    lidar = None
    if not args.no_lidar:
        torch.cuda.empty_cache()
        lidar = run_lidar()

    total_points = torch.tensor([n_points], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(total_points)
    total_points = float(total_points.item())

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        att = timers.get("attention", {"calls": 0, "ms": 0.0, "work": 0.0, "extra": 0.0})
        tf_peak = peaks.get("bf16_tflops_sustained", 1400.0)
        sec = att["ms"] * 1e-3
        achieved = att["work"] / sec / 1e12 if sec else 0.0
        # One exponential per score, head dimension 16: exps = FLOPs / 64.  The exp unit has 16
        # lanes per SM: 16 x 148 x clock results per second at most.
        exps = att["work"] / 64.0
        sm_mhz = (clocks or {}).get("sm_mhz") or 1965.0
        exp_peak = 16 * 148 * sm_mhz * 1e6
        # DRAM bytes per launch: bytes per row and channel of a committed ncu capture of one launch
        # of this kernel (see ATTENTION_DRAM_BYTES_PER_ROW_CHANNEL) x the rows and channels of the
        # average launch of this run; algorithmic: qkv read once, output written once = 8 B.
        rows_channels = att["extra"] or None
        roofline = {"kernel": "attention core (all patch-attention launches of the timed steps)",
                    "bound": "tensor", "achieved": achieved, "peak": tf_peak, "unit": "TFLOP/s",
                    "frac": achieved / tf_peak,
                    "traffic": None if rows_channels is None else
                    ATTENTION_DRAM_BYTES_PER_ROW_CHANNEL * rows_channels / max(att["calls"], 1),
                    "traffic_note": "DRAM bytes per launch: %.2f B per row and channel (one ncu capture of a "
                                    "single launch of this kernel, 8 B algorithmic) x rows x channels of this "
                                    "run's average launch" % ATTENTION_DRAM_BYTES_PER_ROW_CHANNEL,
                    "peak_source": "measured (sustained)" if peaks else "fallback",
                    "launches": att["calls"], "avg_launch_ms": att["ms"] / max(att["calls"], 1),
                    "limiter": {"unit": "exp (one exponential per 64 tensor FLOPs at head dimension 16)",
                                "achieved_exps_per_s": exps / sec if sec else 0.0, "peak_exps_per_s": exp_peak,
                                "frac": exps / sec / exp_peak if sec else 0.0}}
        breakdown = {k: {"calls": v["calls"], "ms_per_step": v["ms"] / args.steps} for k, v in all_timers.items()}
        line = {
            "metric": METRIC, "value": total_points * args.steps / (ms * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "runs_ms_per_step": [m / args.steps for m in resident_runs],
            "runs_note": "K steps timed twice, the faster run reported",
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": dict(workload_config(world, gather), points_per_gpu=n_points),
            "clocks": clocks,
            "e2e": None if ms_e2e is None else {
                "value": total_points * args.steps / (ms_e2e * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e / args.steps,
                "runs_ms_per_step": [m / args.steps for m in e2e_runs],
                "note": "two runs of K steps, the faster one reported"},
            "gpu_launches": int(launches),
            "roofline": roofline,
            "kernel_ms_per_step": breakdown,
            "lidar16": lidar,
            "kernel_ms_note": "second pass on the per-operator host path (one event pair per operator); the "
                              "timed steps queue a whole block per C call and carry no events inside",
        }
        if world == 1 and not args.no_cpu_baseline:
            step, n, sample, kind = cpu_step_fn(1)
            step()
            dts = []
            for _ in range(3):
                t = time.perf_counter()
                step()
                dts.append(time.perf_counter() - t)
            line["cpu_baseline"] = {"value": n / statistics.median(dts), "unit": UNIT,
                                    "cores": torch.get_num_threads(), "kind": kind,
                                    "sample": sample + "; median of 3 after one warm-up"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------- #
# single-operator cases (the smaller configurations): device timing + roofline
# --------------------------------------------------------------------------- #
def _time_device(fn, steps, warmup, flush):
    for _ in range(max(warmup, 3)):
        fn()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    torch.cuda.profiler.start()
    for a, b in ev:
        if flush is not None:
            flush.fill_(1)
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    return sum(a.elapsed_time(b) for a, b in ev) / steps


def run_operator_case(args):
    """--case serialization | attention | conv: one operator of the path on the
    configuration of the benchmark plan for that operator, timed on the device."""
    from pointtransformerv3_b200 import ops, synthetic
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    hbm = peaks.get("hbm_gbs", 6650.0)
    tf = peaks.get("bf16_tflops", 1590.0)
    src = "measured" if peaks else "fallback"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    orders = ["z", "z-trans", "hilbert", "hilbert-trans"]
    out = {"case": args.case, "n_gpus": 1, "steps": args.steps, "data": "synthetic", "peak_source": src}
    if args.case == "serialization":
        n = args.points or 100_000
        _, gc = synthetic.uniform_cloud(n, seed=0)
        gc = gc.to(dev)
        batch = torch.zeros(n, dtype=torch.int64, device=dev)
        codes = ops.encode(gc, batch, 16, orders)
        t_enc = _time_device(lambda: ops.encode(gc, batch, 16, orders), args.steps, args.warmup, flush)
        t_sort = _time_device(lambda: ops.argsort_inverse(codes, 49), args.steps, args.warmup, flush)
        # algorithmic bytes: encode 20 B read + 32 B written per point; argsort + inverse 32 B of
        # codes read and 2 x 32 B of order / inverse written, plus the order read once more
        enc_b, sort_b = 52.0 * n, 128.0 * n
        out.update(config={"workload": "encode x4 orders + stable argsort + inverse, depth 16", "points": n},
                   metric="serialization_points_per_sec", unit="points/s", value=n / ((t_enc + t_sort) * 1e-3),
                   encode_ms=t_enc, argsort_inverse_ms=t_sort,
                   roofline={"kernel": "encode_kernel", "bound": "hbm", "achieved": enc_b / t_enc / 1e6,
                             "peak": hbm, "unit": "GB/s", "frac": enc_b / t_enc / 1e6 / hbm, "traffic": None},
                   roofline_argsort={"kernel": "os_hist_kernel + os_pass_kernel (all passes)", "bound": "hbm",
                                     "achieved": sort_b / t_sort / 1e6, "peak": hbm, "unit": "GB/s",
                                     "frac": sort_b / t_sort / 1e6 / hbm, "traffic": None})
    elif args.case == "attention":
        n, C, H, K = args.points or 120_000, 64, 4, 1024
        g = torch.Generator().manual_seed(0)
        gc = torch.randint(0, 512, (n, 3), generator=g, dtype=torch.int32).to(dev)
        batch = torch.zeros(n, dtype=torch.int64, device=dev)
        codes = ops.encode(gc, batch, 9, ["hilbert"])
        order, _ = ops.argsort_inverse(codes, 28)
        qkv = torch.randn(n, 3 * C, generator=g).bfloat16().to(dev)
        pad, unpad, cu = ops.pad_plan(torch.tensor([n], device=dev), [n], K)
        st = ops.new_status(dev)
        t = _time_device(lambda: ops.attention(qkv, order[0], pad, unpad, cu, H, K, 0.25, algo=args.algo, status=st),
                         args.steps, args.warmup, flush)
        flops = 4.0 * pad.numel() * K * C
        out.update(config={"workload": "patch attention core, bf16, C=64, 4 heads, patch 1024", "points": n,
                           "patches": cu.numel() - 1, "algo": args.algo},
                   metric="attention_points_per_sec", unit="points/s", value=n / (t * 1e-3), ms=t,
                   exps_per_sec=pad.numel() * K * H / (t * 1e-3),
                   roofline={"kernel": "attn_tc05_d16_kernel" if args.algo == 4 else "attn_mma_d16_kernel",
                             "bound": "tensor", "achieved": flops / t / 1e9,
                             "peak": tf, "unit": "TFLOP/s", "frac": flops / t / 1e9 / tf, "traffic": None})
    elif args.case == "conv":
        c = args.channels or 128
        coord, gc = synthetic.indoor_scene(0, args.points or 80_000, GRID)
        n = gc.shape[0]
        ind = torch.cat([torch.zeros(n, 1, dtype=torch.int32), gc], 1).contiguous().to(dev)
        g = torch.Generator().manual_seed(0)
        feat = torch.randn(n, c, generator=g).bfloat16().to(dev)
        w = (torch.randn(c, 3, 3, 3, c, generator=g) / (9 * c) ** 0.5).bfloat16().to(dev)
        b = torch.zeros(c).bfloat16().to(dev)
        codes = ops.encode(gc.to(dev), torch.zeros(n, dtype=torch.int64, device=dev), 9, ["z"])
        order, _ = ops.argsort_inverse(codes, 28)
        t_map = _time_device(lambda: ops.kmap_build(ind, 3), args.steps, args.warmup, flush)
        nbr = ops.kmap_build(ind, 3)
        pairs = int((nbr >= 0).sum())
        nbr = nbr.index_select(1, order[0])
        status = ops.new_status(dev)
        t = _time_device(lambda: ops.subm_conv(feat, nbr, w, b, algo=args.algo, row_order=order[0], status=status),
                         args.steps, args.warmup, flush)
        if int(status.item()):
            raise SystemExit("device status 0x%x" % int(status.item()))
        flops = 2.0 * pairs * c * c
        out.update(config={"workload": "SubMConv3d 3x3x3, C=%d, bf16, one indoor scene" % c, "voxels": n,
                           "pairs": pairs, "algo": args.algo},
                   metric="conv_voxels_per_sec", unit="voxels/s", value=n / (t * 1e-3), ms=t, kmap_ms=t_map,
                   roofline={"kernel": "conv_mma_kernel" if args.algo == 2 else "conv_tc05_kernel",
                             "bound": "tensor", "achieved": flops / t / 1e9,
                             "peak": tf, "unit": "TFLOP/s (useful FLOPs: 2 x pairs x C^2)",
                             "frac": flops / t / 1e9 / tf, "traffic": None},
                   roofline_kmap={"kernel": "km_insert + km_probe", "bound": "hbm",
                                  "achieved": 124.0 * n / t_map / 1e6, "peak": hbm, "unit": "GB/s",
                                  "frac": 124.0 * n / t_map / 1e6 / hbm, "traffic": None})
    elif args.case == "stem":
        # the 5x5x5 stem convolution (6 -> 32 channels) on the forward benchmark's batch
        data = synthetic.indoor_batch(4, target_voxels=(args.points or 400_000) // 4, grid_size=GRID,
                                      dtype=torch.bfloat16)
        n = int(data["offset"][-1])
        off = [0] + data["offset"].tolist()
        batch = torch.cat([torch.full((off[i + 1] - off[i],), i, dtype=torch.int32) for i in range(4)])
        ind = torch.cat([batch[:, None], data["grid_coord"]], 1).contiguous().to(dev)
        codes = ops.encode(data["grid_coord"].to(dev), batch.long().to(dev), 9, ["z"])
        order, _ = ops.argsort_inverse(codes, 30)
        feat = data["feat"].to(dev)
        w = (torch.randn(32, 5, 5, 5, 6, generator=torch.Generator().manual_seed(0)) / 27.0).bfloat16().to(dev)
        t = _time_device(lambda: ops.subm_conv_direct(feat, ind, w, None, None, None, False, order[0]), args.steps,
                         args.warmup, flush)
        byts = n * (6 * 2 + 16 + 32 * 2)      # features and indices in, output rows out
        out.update(config={"workload": "stem SubMConv3d 5x5x5, 6 -> 32 channels, bf16, 4 indoor scenes",
                           "voxels": n},
                   metric="stem_voxels_per_sec", unit="voxels/s", value=n / (t * 1e-3), ms=t,
                   roofline={"kernel": "conv_direct_mma_kernel (+ voxel index build)", "bound": "hbm",
                             "achieved": byts / t / 1e6, "peak": hbm, "unit": "GB/s",
                             "frac": byts / t / 1e6 / hbm, "traffic": None})
    elif args.case == "voxelize":
        # raw points (about 6 per occupied voxel, as a sensor delivers them) -> one point per voxel
        n = args.points or 2_400_000
        g = torch.Generator().manual_seed(0)
        coord = torch.rand(n, 3, generator=g) * torch.tensor([10.0, 10.0, 0.06])
        offset = torch.tensor([n // 4, n // 2, 3 * n // 4, n])
        batch = torch.repeat_interleave(torch.arange(4), torch.tensor([n // 4, n // 4, n // 4, n - 3 * (n // 4)]))
        coord, offset, batch = coord.to(dev), offset.to(dev), batch.to(dev)
        t_grid = _time_device(lambda: ops.grid_coord(coord, GRID), args.steps, args.warmup, flush)
        grid, _ = ops.grid_coord(coord, GRID)
        ind = torch.cat([batch.unsqueeze(-1).int(), grid], 1).contiguous()
        t_dedup = _time_device(lambda: ops.voxel_dedup(ind, offset), args.steps, args.warmup, flush)
        m = ops.voxel_dedup(ind, offset)["m"]
        grid_b = n * (12 + 12 + 12.0)           # coordinates read twice (minimum, then quantisation), grid written
        dedup_b = n * (16 + 8 + 8.0)            # indices read, keep and point-to-voxel rows written
        out.update(config={"workload": "grid coordinates + first point per voxel, 4 scenes, grid 0.02", "points": n,
                           "voxels": m},
                   metric="voxelize_points_per_sec", unit="points/s", value=n / ((t_grid + t_dedup) * 1e-3),
                   grid_coord_ms=t_grid, voxel_dedup_ms=t_dedup,
                   roofline={"kernel": "vox_min_kernel + vox_grid_kernel", "bound": "hbm",
                             "achieved": grid_b / t_grid / 1e6, "peak": hbm, "unit": "GB/s",
                             "frac": grid_b / t_grid / 1e6 / hbm, "traffic": None},
                   roofline_dedup={"kernel": "km_insert + vox_first + flag scan + vox_inverse (one host read)",
                                   "bound": "hbm", "achieved": dedup_b / t_dedup / 1e6, "peak": hbm, "unit": "GB/s",
                                   "frac": dedup_b / t_dedup / 1e6 / hbm})
    elif args.case == "linear":
        # the two Linear forms of a block on the tcgen05 kernels: qkv projection, and
        # Linear + LayerNorm + residual + LayerNorm (cpe.1 / cpe.2 / shortcut / norm1)
        n, c = args.points or 407_000, 64
        g = torch.Generator().manual_seed(0)
        mk = lambda *shape: torch.randn(*shape, generator=g).bfloat16().to(dev)
        x, res = mk(n, c), mk(n, c)
        w, b, wq, bq = mk(c, c), mk(c), mk(3 * c, c), mk(3 * c)
        ln1 = torch.nn.LayerNorm(c).to(dev).bfloat16()
        ln2 = torch.nn.LayerNorm(c).to(dev).bfloat16()
        st = ops.new_status(dev)
        t_ln = _time_device(lambda: ops.linear_ln(x, w, b, res, ln1, ln2, st), args.steps, args.warmup, flush)
        t_qkv = _time_device(lambda: ops.linear(x, wq, bq, st), args.steps, args.warmup, flush)
        ln_b, qkv_b = 4.0 * n * c * 2, 4.0 * n * c * 2     # x + residual in, two outputs; x in, 3C out
        out.update(config={"workload": "Linear + LN + residual + LN and the qkv Linear, C=64, bf16", "rows": n},
                   metric="linear_rows_per_sec", unit="rows/s", value=n / ((t_ln + t_qkv) * 1e-3),
                   linear_ln_ms=t_ln, linear_qkv_ms=t_qkv,
                   roofline={"kernel": "linear_tc05_kernel<64> (residual mode)", "bound": "hbm",
                             "achieved": ln_b / t_ln / 1e6, "peak": hbm, "unit": "GB/s",
                             "frac": ln_b / t_ln / 1e6 / hbm, "traffic": None},
                   roofline_qkv={"kernel": "linear_tc05_kernel<64> (plain mode)", "bound": "hbm",
                                 "achieved": qkv_b / t_qkv / 1e6, "peak": hbm, "unit": "GB/s",
                                 "frac": qkv_b / t_qkv / 1e6 / hbm})
    elif args.case == "gemm":
        # the streamed-weight Linear kernel on the shapes of the wide levels (rows x k -> n_out)
        n, k, n_out = args.points or 7808, 256, 768
        g = torch.Generator().manual_seed(0)
        x = torch.randn(n, k, generator=g).bfloat16().to(dev)
        w = (torch.randn(n_out, k, generator=g) / k ** 0.5).bfloat16().to(dev)
        b = torch.zeros(n_out).bfloat16().to(dev)
        st = ops.new_status(dev)
        t = _time_device(lambda: ops.gemm(x, w, b, None, False, st), args.steps, args.warmup, flush)
        flops = 2.0 * n * k * n_out
        out.update(config={"workload": "Linear %d -> %d with streamed weights, bf16" % (k, n_out), "rows": n},
                   metric="gemm_rows_per_sec", unit="rows/s", value=n / (t * 1e-3), ms=t,
                   roofline={"kernel": "gemm_tc05_kernel", "bound": "tensor", "achieved": flops / t / 1e9,
                             "peak": tf, "unit": "TFLOP/s", "frac": flops / t / 1e9 / tf, "traffic": None})
    elif args.case == "seghead":
        n, c, k = args.points or 407_000, 64, 20
        g = torch.Generator().manual_seed(0)
        feat = torch.randn(n, c, generator=g).bfloat16().to(dev)
        w = (torch.randn(k, c, generator=g) / 8).bfloat16().to(dev)
        b = torch.zeros(k).bfloat16().to(dev)
        t = _time_device(lambda: ops.seg_head(feat, w, b, want_logits=False), args.steps, args.warmup, flush)
        t_full = _time_device(lambda: ops.seg_head(feat, w, b), args.steps, args.warmup, flush)
        byts = n * (c * 2 + 8.0)                # feature rows read, labels written
        out.update(config={"workload": "segmentation head, 64 -> 20 classes + arg max, bf16", "points": n},
                   metric="seg_head_points_per_sec", unit="points/s", value=n / (t * 1e-3), ms=t,
                   with_logits_ms=t_full,
                   roofline={"kernel": "seg_head_kernel (labels only)", "bound": "hbm", "achieved": byts / t / 1e6,
                             "peak": hbm, "unit": "GB/s", "frac": byts / t / 1e6 / hbm, "traffic": None})
    elif args.case == "pooling":
        # stride-2 pooling of a 4-scene indoor batch: plan (clusters, pooled orders) and feature side
        data = synthetic.indoor_batch(4, target_voxels=(args.points or 400_000) // 4, grid_size=GRID)
        n, c = int(data["offset"][-1]), 64
        off = [0] + data["offset"].tolist()
        batch = torch.cat([torch.full((off[i + 1] - off[i],), i, dtype=torch.int64) for i in range(4)]).to(dev)
        gc = data["grid_coord"].to(dev)
        depth = int(gc.max()).bit_length()
        codes = ops.encode(gc, batch, depth, orders)
        order, _ = ops.argsort_inverse(codes, 3 * depth + 3)
        t_plan = _time_device(lambda: ops.pool_plan(codes, order, gc, batch, 4, 1, [2, 0, 3, 1]), args.steps,
                              args.warmup, flush)
        plan = ops.pool_plan(codes, order, gc, batch, 4, 1, [2, 0, 3, 1])
        m = plan["m"]
        x = torch.randn(n, c, generator=torch.Generator().manual_seed(0)).bfloat16().to(dev)
        coord = data["coord"].to(dev)
        scale = torch.ones(c, device=dev)
        shift = torch.zeros(c, device=dev)
        t_pool = _time_device(lambda: ops.pool(x, coord, order[0], plan["idx_ptr"], scale, shift), args.steps,
                              args.warmup, flush)
        child = torch.randn(m, c, generator=torch.Generator().manual_seed(1)).bfloat16().to(dev)
        t_unpool = _time_device(lambda: ops.unpool(x, child, plan["cluster"], scale, shift, scale, shift),
                                args.steps, args.warmup, flush)
        pool_b = n * (c * 2 + 8 + 12) + m * (c * 2 + 12 + 8)     # rows + order + coord in, pooled rows + coord out
        unpool_b = n * (c * 2 * 3 + 8) + m * c * 2                # skip in, two outputs, cluster ids, child rows
        plan_b = n * (4 * 8 * 2 + 12 + 8 + 8) + m * (4 * 8 * 3 + 12 + 8 + 8)
        out.update(config={"workload": "stride-2 pooling, 4 indoor scenes, C=64, bf16", "points": n, "clusters": m},
                   metric="pooling_points_per_sec", unit="points/s", value=n / ((t_plan + t_pool) * 1e-3),
                   plan_ms=t_plan, pool_ms=t_pool, unpool_ms=t_unpool,
                   roofline={"kernel": "pool_max_kernel + pool_coord_mean_kernel", "bound": "hbm",
                             "achieved": pool_b / t_pool / 1e6, "peak": hbm, "unit": "GB/s",
                             "frac": pool_b / t_pool / 1e6 / hbm, "traffic": None},
                   roofline_unpool={"kernel": "unpool_kernel", "bound": "hbm", "achieved": unpool_b / t_unpool / 1e6,
                                    "peak": hbm, "unit": "GB/s", "frac": unpool_b / t_unpool / 1e6 / hbm},
                   roofline_plan={"kernel": "pool plan (7 launches, one host read)", "bound": "hbm",
                                  "achieved": plan_b / t_plan / 1e6, "peak": hbm, "unit": "GB/s",
                                  "frac": plan_b / t_plan / 1e6 / hbm})
    elif args.case == "mlp":
        n, c = args.points or 407_000, 64
        g = torch.Generator().manual_seed(0)
        mk = lambda *shape: torch.randn(*shape, generator=g).bfloat16().to(dev)
        x, res = mk(n, c), mk(n, c)
        w1, b1, w2, b2 = mk(4 * c, c), mk(4 * c), mk(c, 4 * c), mk(c)
        st = ops.new_status(dev)
        t = _time_device(lambda: ops.mlp(x, w1, b1, w2, b2, res, st), args.steps, args.warmup, flush)
        byts = 3.0 * n * c * 2
        out.update(config={"workload": "fused MLP (fc1, GELU, fc2, residual), C=64, hidden 256, bf16", "rows": n},
                   metric="mlp_rows_per_sec", unit="rows/s", value=n / (t * 1e-3), ms=t,
                   roofline={"kernel": "mlp_tc05_kernel", "bound": "hbm", "achieved": byts / t / 1e6,
                             "peak": hbm, "unit": "GB/s", "frac": byts / t / 1e6 / hbm, "traffic": None})
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-lidar", action="store_true", help="skip the sharded LiDAR-like batch (\"lidar16\")")
    ap.add_argument("--gather-outputs", action="store_true",
                    help="N > 1: all-gather the output features over NCCL inside every step")
    ap.add_argument("--case", default="forward", choices=["forward", "serialization", "voxelize", "attention", "conv", "stem", "mlp", "linear", "gemm", "pooling", "seghead"],
                    help="forward = the headline workload; the others time one operator of the path")
    ap.add_argument("--points", type=int, default=0, help="size override for the single-operator cases")
    ap.add_argument("--algo", type=int, default=0,
                    help="--case attention: algo of ptv3_attention_fwd (4 = tcgen05); --case conv: algo of "
                         "ptv3_subm_conv_fwd (2 = mma.sync, 3 = tcgen05)")
    ap.add_argument("--channels", type=int, default=0, help="--case conv: channel count (default 128)")
    args = ap.parse_args()
    if args.case != "forward":
        run_operator_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
