#!/usr/bin/env python
"""Benchmark of the contraction hot path: string contraction -> dimension binding -> GPU kernel.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload suite|cfg0..cfg4]
                    [--impl ours|reference] [--scaling weak|strong] [--scale F]

A "step" is one pass of the selected workload(s) over one batch of seeded synthetic input.
The default workload, "suite", runs the five benchmark configurations back to back; the
headline `value` is the suite's algorithmic GB/s (sum of algorithmic bytes / step time) with
inputs resident in HBM, and `per_config` carries GB/s, GFLOP/s and roofline fraction of every
configuration.  `e2e` is the same metric through the public engine API with HOST buffers
(pinned), host->device and device->host copies inside the timed region.

For N > 1 launch with torchrun (one rank per GPU).  The batch index is cut into per-rank
slabs; "strong" (default) cuts the benchmark sizes into N slabs, "weak" gives every rank a
full-size slab.  Only the README reduction (batch index contracted) needs a collective: one
all-reduce of its 3x3 result per step, inside the timed region.

`--impl reference` times the reference's own CPU executor (the unmodified sources compiled
into oracle/_ref, else the C restatement) on all host threads, on bounded samples.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

FALLBACK_HBM_GBS = 6650.0
# fp64 peak of a B200: the tensor-core (DMMA) microbenchmark figure measured on this pool, read from
# a one-number text file kept with the profile summaries; used for the compute-bound configurations.
FP64_PEAK_GFLOPS_FILE = os.path.join(ROOT, "profiles", "fp64_peak_gflops.txt")
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of ONE benchmark-size launch of each
# configuration's kernel, from ncu captures of smaller launches scaled in proportion to the batch
# (traffic of these streaming kernels grows linearly with it).  Measured once per kernel version by
# hand: these numbers do not follow a code change by themselves.
NCU_TRAFFIC_BYTES = {"cfg3": 9.79e9, "cfg0": 5.40e9, "cfg2": 2.01e9, "cfg1": 1.42e9, "cfg4": 1.36e9}

# batch of the bounded CPU sample per configuration (about 1-2 s of one core each)
CPU_SAMPLE = {"cfg0": 1 << 24, "cfg1": 1 << 12, "cfg2": 1 << 16, "cfg3": 1 << 16, "cfg4": 1 << 9}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return float(d["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def fp64_peak_gflops():
    try:
        with open(FP64_PEAK_GFLOPS_FILE) as f:
            return float(f.read().split()[0])
    except Exception:
        return 37000.0     # datasheet-level figure until the microbenchmark is recorded


class ClockSampler:
    """SM clock and throttle reasons during the timed region (read-only queries).  The timed region of a sharded run
    lasts tens of milliseconds, so the samples come from NVML polled in a thread of this process every 10 ms
    (not faster: every rank of a node polls, and the queries share the driver's locks with everything else);
    `nvidia-smi -lms` (a sample every 100 ms after a start-up of its own) is the fallback when the NVML binding
    is missing."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, gpu_index, period_s=0.01):
        self.gpu_index = gpu_index
        self.period_s = period_s
        self.proc = None
        self.path = None
        self.thread = None
        self.samples = []          # (sm_mhz, reasons bit mask, watts)
        self.sm_max = None
        self.stop_flag = threading.Event()
        self.first = 0

    def mark(self):
        """The timed region starts here: samples taken before it (an idle GPU) are left out."""
        self.first = len(self.samples)

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            uuid = str(torch.cuda.get_device_properties(self.gpu_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)

    def _poll(self, nv, handle):
        while not self.stop_flag.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                try:
                    watts = nv.nvmlDeviceGetPowerUsage(handle) / 1000.0
                except Exception:
                    watts = None
                self.samples.append((float(mhz), int(mask), watts))
            except Exception:
                pass
            self.stop_flag.wait(self.period_s)

    def start(self):
        try:
            nv, handle = self._nvml_handle()
            self.sm_max = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._poll, args=(nv, handle), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.thread is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            self.samples = self.samples[self.first:] or self.samples
            if not self.samples:
                return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": ["no samples"], "source": "nvml"}
            mask = 0
            for _, m, _ in self.samples:
                mask |= m
            watts = [w for _, _, w in self.samples if w is not None]
            return {"sm_mhz": float(np.median([c for c, _, _ in self.samples])), "sm_max_mhz": self.sm_max,
                    "reasons": sorted(name for name, bit in self.REASON_BITS if mask & bit), "samples": len(self.samples),
                    "sm_min_mhz": float(min(c for c, _, _ in self.samples)),
                    "watts_max": float(max(watts)) if watts else None, "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    smax.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        os.unlink(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"], "source": "nvidia-smi"}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(smax)), "reasons": sorted(reasons),
                "samples": len(sm), "source": "nvidia-smi"}


def host_memory_available():
    """Bytes of host memory this process may still use (cgroup limit and MemAvailable)."""
    avail = None
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    avail = int(line.split()[1]) * 1024
    except Exception:
        pass
    try:
        with open("/sys/fs/cgroup/memory.max") as f:
            lim = f.read().strip()
        with open("/sys/fs/cgroup/memory.current") as f:
            cur = int(f.read().strip())
        if lim != "max":
            room = int(lim) - cur
            avail = room if avail is None else min(avail, room)
    except Exception:
        pass
    return avail


def launch_traffic(w, batch):
    """ncu DRAM bytes of one launch over `batch` units, scaled from the benchmark-size figure."""
    full = NCU_TRAFFIC_BYTES.get(w.key)
    return None if full is None else round(full * batch / w.batch)


def selected(workload):
    from acrotensor_b200.workloads import BY_KEY, WORKLOADS
    only = os.environ.get("ACRO_BENCH_ONLY")          # debugging: a comma-separated subset of the suite
    if workload == "suite" and only:
        return [BY_KEY[k] for k in only.split(",")]
    return list(WORKLOADS) if workload == "suite" else [BY_KEY[workload]]


def local_batch(w, args, rank, world):
    from acrotensor_b200.runner import slab
    full = max(1, int(round(w.batch * args.scale)))
    if args.scaling == "weak" or world == 1:
        return full
    b0, b1 = slab(full, rank, world)
    return b1 - b0


def config_of(args, world, workloads, batches):
    """The `config` object of the record: both arms print the same one for the same command line (the
    reference arm measures the whole job on the host, whatever the number of GPUs)."""
    return {"workload": args.workload + (": cfg0..cfg4 back to back" if args.workload == "suite" else "")
                        + (", benchmark sizes" if world == 1 else
                           (", benchmark sizes cut into %d slabs (strong scaling)" % world if args.scaling == "strong"
                            else ", a benchmark-size slab on each of %d ranks (weak scaling)" % world)),
            "batches_per_gpu": {w.key: b for w, b in zip(workloads, batches)},
            "l2": ("inputs_exceed_l2 (the smallest configuration streams %.0f MB per GPU per step, L2 holds 126 MB)"
                   % (min(w.bytes(b) for w, b in zip(workloads, batches)) * 1e-6)) if args.scale >= 1 else "scaled-down run",
            "parallelism": "batch slabs x%d, all-reduce only for the contracted batch index (%s)"
                           % (world, "none needed" if world == 1 else
                              ("fused into the reduction kernel over NVLink peer memory" if args.allreduce == "fused" else "NCCL"))}


# ----------------------------------------------------------------------------- our arm

def run_ours(args):
    import torch
    import torch.distributed as dist
    import acrotensor_b200 as ab
    from acrotensor_b200.runner import Session, allreduce_partial, make_peer_group

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit("--gpus %d does not match WORLD_SIZE %d" % (args.gpus, world))
    if args.gpus > 1 and world == 1:
        raise SystemExit("launch N>1 with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...")
    if not os.path.exists(ab.LIB_PATH):
        raise SystemExit("libacrotensor.so is missing and there is no fallback: run __graft_entry__.build()")
    if not torch.cuda.is_available() or ab.device_count() == 0:
        raise SystemExit("bench.py needs a CUDA device: the contraction path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    t_start = time.perf_counter()
    if os.environ.get("ACRO_BENCH_TRACE") == "1":
        import faulthandler
        import signal
        faulthandler.register(signal.SIGUSR1, all_threads=True)      # kill -USR1 <pid>: where is the host?

    def trace(what):
        """Progress lines on stderr when ACRO_BENCH_TRACE=1 (to see where a multi-rank run spends its time)."""
        if os.environ.get("ACRO_BENCH_TRACE") == "1":
            print("[bench rank %d +%.1fs] %s" % (rank, time.perf_counter() - t_start, what), file=sys.stderr, flush=True)

    workloads = selected(args.workload)
    peer_group = None
    use_nccl = world > 1 and args.allreduce == "nccl"
    sessions, outs_dev, batches = [], [], []
    h2d = d2h = 0
    # The end-to-end leg needs every rank's inputs and results in pinned host memory, and all
    # ranks of the node share that memory.  Mode "all": everything pinned at once (allows a
    # result's download to overlap the next configuration's upload) when that takes less than
    # half of the free host memory; mode "one": one configuration pinned at a time; else skipped.
    def host_bytes(w):
        return sum(int(np.prod(shape)) * 8 for name, shape in w.shapes(local_batch(w, args, rank, world)).items()
                   if w.tensors[name][2] != "tmp")
    need_all = sum(host_bytes(w) for w in workloads) * world
    need_one = max(host_bytes(w) for w in workloads) * world
    avail = host_memory_available()
    e2e_mode = "all" if (avail is None or need_all < 0.5 * avail) else ("one" if need_one < 0.5 * avail else "skip")
    if args.e2e_mode != "auto":
        e2e_mode = args.e2e_mode
    if world > 1:
        # ranks sample the free memory at slightly different times: rank 0 decides for all
        decided = [e2e_mode, avail]
        dist.broadcast_object_list(decided, src=0)
        e2e_mode, avail = decided

    def pinned_buffers(w, dev_t):
        """Pinned host arrays for the inputs and results of one workload; inputs filled from the device."""
        bufs = {}
        for name in w.names("in") + w.names("out"):
            bufs[name] = torch.empty(dev_t[name].shape, dtype=torch.float64, pin_memory=True)
            if name in w.names("in"):
                bufs[name].copy_(dev_t[name])
        torch.cuda.synchronize()
        return bufs

    for w in workloads:
        b = local_batch(w, args, rank, world)
        batches.append(b)
        dev_t = w.make_inputs_device(b, dev, seed=args.seed, rank=rank)
        host = {}
        for name, shape in w.shapes(b).items():
            if name in dev_t:
                h2d += int(np.prod(shape)) * 8
            else:
                # results, and chain intermediates (transient, elided by the fused plan; they
                # still need real storage to bind)
                dev_t[name] = torch.zeros(shape, dtype=torch.float64, device=dev)
                if w.tensors[name][2] == "out":
                    d2h += int(np.prod(shape)) * 8
            # untouched pageable placeholder; the end-to-end leg retargets tensors to pinned buffers
            host[name] = torch.empty(shape, dtype=torch.float64).numpy()
        torch.cuda.synchronize()
        # N > 1: every batched tensor is this rank's slab of the batch index and is flagged as such; the engine
        # sums a result over the ranks of its peer group only where a string contracts that index (cfg0: reduction
        # and all-reduce in one kernel, over NVLink peer memory) and leaves every other configuration alone
        sess = Session(w, host, device=dict(dev_t), transient=True, sharded=world > 1)
        if world > 1 and args.allreduce == "fused":
            if peer_group is None:
                peer_group = make_peer_group()
            sess.te.SetPeerGroup(peer_group)
        sess.keep = dev_t
        sessions.append(sess)
        outs_dev.append({n: dev_t[n] for n in w.names("out")})

    def make_resident():
        # the device buffers already hold the generated inputs: mark them fresh
        for w, sess in zip(workloads, sessions):
            for name in w.tensors:
                sess.t[name].SwitchToGPU()
        torch.cuda.synchronize()

    sync_each = os.environ.get("ACRO_BENCH_SYNC_EACH") == "1"      # debugging: wait for every configuration and say so
    step_no = [0]

    # --streams per-config: the configurations are independent contractions, each engine launches on a stream of its
    # own (TensorEngine::SetCudaStream) and the GPU runs them side by side; the instrumented pass stays on one stream
    side = [torch.cuda.Stream(device=dev) for _ in workloads] if (args.streams == "per-config" and not use_nccl) else None

    def use_side_streams(on):
        if side is not None:
            for sess, st in zip(sessions, side):
                sess.te.SetCudaStream(st.cuda_stream if on else torch.cuda.current_stream().cuda_stream)

    def fork():
        if side is not None:
            ev0 = torch.cuda.Event()
            ev0.record()
            for st in side:
                st.wait_event(ev0)

    def join():
        if side is not None:
            for st in side:
                done = torch.cuda.Event()
                done.record(st)
                torch.cuda.current_stream().wait_event(done)

    def device_step(events=None):
        step_no[0] += 1
        for i, (w, sess) in enumerate(zip(workloads, sessions)):
            if events is not None:
                events[i][0].record()
            sess.run()
            if w.batch_contracted and use_nccl:
                allreduce_partial(outs_dev[i][w.names("out")[0]])
            if events is not None:
                events[i][1].record()
            if sync_each:
                t_sync = time.perf_counter()
                torch.cuda.synchronize()
                trace("step %d %s done (%.1f ms), device status %d" % (step_no[0], w.key, (time.perf_counter() - t_sync) * 1e3,
                                                                        ab.lib().acro_b200_device_status()))

    trace("sessions ready")
    make_resident()
    barrier()      # all ranks enter the first step together (the fused all-reduce waits at most about a second)
    plans = [sess.plan_text() for sess in sessions]
    # a chain whose intermediates are transient runs the fused plan, described after the marker line
    launches_per_step = sum(p.split("--- when every intermediate is transient ---")[-1].count("\nstep ") for p in plans)
    for _ in range(args.warmup):
        device_step()
    barrier()
    trace("warm-up done")

    def any_rank_gave_up():
        """True when a bounded device-side wait gave up on some rank since the last call (collective)."""
        flag = torch.tensor([float(ab.lib().acro_b200_device_status() != 0)], device=dev)
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        return bool(flag.item())

    # A rank whose host stalls for about a second while its launch queue is empty (a shared machine) makes
    # its peers' bounded waits give up; such a measurement is void and is taken again, four times at most.
    # The step time is taken over launches that follow each other with nothing in between (an event between two
    # launches keeps the second from being brought onto the SMs while the first drains); the per-configuration
    # times come from a second pass of the same steps with an event on either side of every configuration.
    for attempt in range(5):
        any_rank_gave_up()                       # clear what warm-up or an earlier attempt left
        sampler = ClockSampler(local_rank)
        sampler.start()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        use_side_streams(True)
        sampler.mark()
        t0.record()
        fork()
        for k in range(args.steps):
            device_step()
        join()
        t1.record()
        barrier()
        use_side_streams(False)
        ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in workloads]
              for _ in range(args.steps)]
        barrier()      # creating the events takes a different time on every rank; a peer of the fused all-reduce waits only about half a second
        for k in range(args.steps):
            device_step(ev[k])
        barrier()
        clocks = sampler.stop()      # samples of both passes: the timed one and the instrumented one
        gave_up = any_rank_gave_up()
        trace("measurement %d done%s" % (attempt + 1, ", void: a bounded wait gave up on some rank" if gave_up else ""))
        if not gave_up:
            break
    else:
        raise SystemExit("rank %d: a bounded device-side wait gave up in five measurements in a row" % rank)
    clocks["attempts"] = attempt + 1
    total_ms = t0.elapsed_time(t1)
    per_cfg_ms = [float(np.median([ev[k][i][0].elapsed_time(ev[k][i][1]) for k in range(args.steps)]))
                  for i in range(len(workloads))]

    # parity spot check of what was just computed (sampled units, untimed); the contracted configuration and
    # the rank-sum of a Gram string are checked by all ranks together
    parity = spot_check(workloads, sessions, batches, world) if rank == 0 else None
    across = contracted_parity(workloads, sessions, batches, world, rank, dev)
    if world > 1 and peer_group is not None:
        across["gram_rank_sum"] = gram_rank_sum_check(peer_group, world, rank, dev)
    trace("parity checks done")
    if rank == 0:
        parity.update(across)
        if world == 1 and args.scale >= 1 and not args.no_cpu_baseline:
            full = cfg0_against_reference(workloads, sessions, batches)
            if full is not None:
                parity["cfg0_vs_reference_full"] = full

    # end to end: host buffers, copies inside the timed region
    e2e_steps = max(1, min(args.steps, args.e2e_steps))

    # A second host thread with its own stream copies each result back (MoveFromGPU) while
    # the main thread already uploads the next configuration's inputs: PCIe is full duplex.
    import concurrent.futures
    copy_stream = torch.cuda.Stream(device=dev)
    pool = concurrent.futures.ThreadPoolExecutor(max_workers=1)

    def fetch_on_copy_stream(sess, ready):
        torch.cuda.set_device(dev)
        ab.set_stream(copy_stream.cuda_stream)          # per-thread setting
        copy_stream.wait_event(ready)                   # the kernels that produce the result
        sess.fetch()                                     # MoveFromGPU of the result (D2H), synchronous for this thread

    def retarget(i, bufs):
        w, sess = workloads[i], sessions[i]
        for name, buf in bufs.items():
            sess.t[name].Retarget(buf.numpy(), sess.keep[name])

    def e2e_step(order):
        pending = []
        for i in order:
            w, sess = workloads[i], sessions[i]
            for name in w.names("in"):
                sess.t[name].SwitchFromGPU()          # the host copy is the fresh one again
            for name in w.names("out") + w.names("tmp"):
                sess.t[name].SwitchFromGPU()
            if w.batch_contracted and world > 1 and not use_nccl:
                dist.barrier()     # uploads of several GB skew the ranks; a peer of the fused all-reduce waits only about a second
            sess.run()                                  # implicit MoveToGPU of every input (H2D), then the kernels
            if w.batch_contracted and use_nccl:
                allreduce_partial(outs_dev[i][w.names("out")[0]])
            ready = torch.cuda.Event()
            ready.record()
            pending.append(pool.submit(fetch_on_copy_stream, sess, ready))
        for f in pending:
            f.result()

    def timed_e2e(order):
        barrier()      # rank 0 comes late from the spot check; the fused all-reduce waits only about a second for a peer
        e2e_step(order)
        barrier()
        w0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step(order)
        barrier()
        return (time.perf_counter() - w0) * 1e3 / e2e_steps

    if e2e_mode == "all":
        keep_pinned = [pinned_buffers(w, sess.keep) for w, sess in zip(workloads, sessions)]
        for i, bufs in enumerate(keep_pinned):
            retarget(i, bufs)
        # largest result first, so that its download overlaps the largest remaining upload
        order = sorted(range(len(workloads)), key=lambda i: -sum(outs_dev[i][n].numel() for n in outs_dev[i]))
        e2e_ms = timed_e2e(order)
    elif e2e_mode == "one":
        e2e_ms = 0.0
        for i in range(len(workloads)):
            bufs = pinned_buffers(workloads[i], sessions[i].keep)
            retarget(i, bufs)
            e2e_ms += timed_e2e([i])
            # back to the pageable placeholders, so that the pinned buffers can be released
            retarget(i, {n: torch.from_numpy(sessions[i].host[n]) for n in bufs})
            for n in workloads[i].names("in"):
                sessions[i].t[n].SwitchToGPU()
            del bufs
    else:
        e2e_ms = float("nan")

    # a bounded device-side wait that gave up on ANY rank invalidates the whole run: no line is printed
    status = ab.lib().acro_b200_device_status()
    status_text = ab.lib().acro_b200_last_error().decode() if status != 0 else ""
    times = torch.tensor([total_ms, e2e_ms] + per_cfg_ms + [float(-status)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    times = times.tolist()
    total_ms, e2e_ms, per_cfg_ms, worst_status = times[0], times[1], times[2:-1], int(times[-1])
    if worst_status != 0:
        pool.shutdown()
        if world > 1:
            dist.destroy_process_group()
        raise SystemExit("rank %d: device status %d on this rank, %d on the worst rank: %s"
                         % (rank, status, -worst_status, status_text or "another rank's launch gave up waiting"))

    if rank == 0:
        hbm_peak, peak_kind = measured_peaks()
        fp64_peak = fp64_peak_gflops()
        ms_per_step = total_ms / args.steps
        glob = [b * world if (args.scaling == "weak" or world == 1) else max(1, int(round(w.batch * args.scale)))
                for w, b in zip(workloads, batches)]
        total_bytes = sum(w.bytes(g) for w, g in zip(workloads, glob))
        total_flops = sum(w.flops(g) for w, g in zip(workloads, glob))
        per_config = {}
        for w, g, ms, b in zip(workloads, glob, per_cfg_ms, batches):
            gbs = w.bytes(g) / ms * 1e-6
            gfl = w.flops(g) / ms * 1e-6
            frac_hbm = gbs / (hbm_peak * world)
            frac_fp64 = w.executed_flops_fn(g) / ms * 1e-6 / (fp64_peak * world)
            per_config[w.key] = {
                "batch": g, "ms": round(ms, 4), "GBps": round(gbs, 1), "GFLOPps": round(gfl, 1),
                "bound": w.bound, "frac": round(frac_hbm if w.bound == "hbm" else frac_fp64, 4),
                "frac_hbm": round(frac_hbm, 4),
                # flops the kernel executes (cfg1 computes only the 378 + 6 packed columns of its symmetric result)
                "frac_fp64_executed": round(frac_fp64, 4),
                "algorithmic_GFLOPps_over_fp64_peak": round(gfl / (fp64_peak * world), 4)}
        # the dominant kernel: the one with the largest share of the step
        dom = int(np.argmax(per_cfg_ms))
        wd = workloads[dom]
        dom_bytes = wd.bytes(batches[dom])
        if wd.bound == "hbm":
            achieved = dom_bytes / per_cfg_ms[dom] * 1e-6
            roof = {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s",
                    "frac": round(achieved / hbm_peak, 4), "traffic": launch_traffic(wd, batches[dom]),
                    "kernel": wd.key, "peak_source": peak_kind + " (MEASURED_PEAKS.json hbm_gbs)" if peak_kind == "measured" else "fallback",
                    "algorithmic_bytes_per_launch": dom_bytes}
        else:
            achieved = wd.executed_flops_fn(batches[dom]) / per_cfg_ms[dom] * 1e-9
            roof = {"bound": "tensor", "achieved": round(achieved, 2), "peak": round(fp64_peak * 1e-3, 2), "unit": "TFLOP/s",
                    "frac": round(achieved / (fp64_peak * 1e-3), 4), "traffic": launch_traffic(wd, batches[dom]),
                    "kernel": wd.key, "peak_source": "fp64 tensor-core microbenchmark on this pool (not in MEASURED_PEAKS.json)",
                    "executed_flops_per_launch": wd.executed_flops_fn(batches[dom])}
        line = {
            "metric": "contraction_throughput", "value": round(total_bytes / ms_per_step * 1e-6, 1), "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f64",
            "data": "synthetic (seeded, shapes and distributions of the benchmark configurations)",
            "config": config_of(args, world, workloads, batches),
            "gflops": round(total_flops / ms_per_step * 1e-6, 1),
            "per_config": per_config,
            "per_config_note": "ms of each configuration from a second pass with an event on either side of it (median over the "
                               "steps); ms_per_step and value from the pass without events between the launches",
            "roofline": roof,
            "e2e": ({"value": round(total_bytes / e2e_ms * 1e-6, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d,
                     "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_ms, 2), "steps": e2e_steps,
                     "pinned": "all configurations at once, download overlapped with the next upload" if e2e_mode == "all"
                     else "one configuration at a time (host memory), upload and download serial"} if e2e_mode != "skip" else
                    {"value": None, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                     "skipped": "host memory: %.0f GB of pinned buffers needed on this node for one configuration, %.0f GB available"
                                % (need_one * 1e-9, (avail or 0) * 1e-9)}),
            "host_memory_available_gb": None if avail is None else round(avail * 1e-9, 1),
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "parity": parity,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(workloads, args)
        print(json.dumps(line))
    pool.shutdown()
    if world > 1:
        # orderly exit: nobody unmaps or frees a mailbox while a peer may still be running a kernel that writes to it
        barrier()
        for sess in sessions:
            sess.te.SetPeerGroup(None)
        peer_group = None
        barrier()
        dist.destroy_process_group()
    trace("done")


def contracted_parity(workloads, sessions, batches, world, rank, dev):
    """The configuration whose batch index is contracted, at any N (collective: every rank calls it).  Each rank sums
    its own slab with torch's fp64 tree reduction; the rank-ordered total of those sums is compared with the result
    the engine left on this rank, and all ranks must hold the same bits."""
    import torch
    import torch.distributed as dist
    found = {}
    for w, sess, b in zip(workloads, sessions, batches):
        if not w.batch_contracted:
            continue
        out = w.names("out")[0]
        got = sess.keep[out].reshape(-1).clone()
        mine = (sess.keep["A"].view(b, -1) * sess.keep["B"].view(b, 1)).sum(dim=0)
        if world > 1:
            sums = [torch.empty_like(mine) for _ in range(world)]
            results = [torch.empty_like(got) for _ in range(world)]
            dist.all_gather(sums, mine)
            dist.all_gather(results, got)
        else:
            sums, results = [mine], [got]
        total = torch.zeros_like(mine)
        for part in sums:          # rank order, as the exchange adds them
            total += part
        found[w.key] = float(((got - total).abs() / total.abs()).max().item())
        found[w.key + "_same_bits_on_every_rank"] = bool(all(torch.equal(r, results[0]) for r in results))
        found[w.key + "_ranks"] = world
    return found


def gram_rank_sum_check(peer_group, world, rank, dev):
    """N > 1, untimed: a Gram string over a sharded row index, run through the engine on every rank (its own
    family, followed by the all-reduce kernel), against the rank-ordered total of per-rank torch products."""
    import torch
    import torch.distributed as dist
    import acrotensor_b200 as ab
    rows, a = 1 << 16, 27
    gen = torch.Generator(device=dev)
    gen.manual_seed(4242 + rank)
    x = torch.rand((rows, a), generator=gen, device=dev, dtype=torch.float64) - 0.5
    y = torch.rand((rows, a), generator=gen, device=dev, dtype=torch.float64) - 0.5
    s = torch.zeros((a, a), device=dev, dtype=torch.float64)
    host = lambda t: torch.empty(tuple(t.shape), dtype=torch.float64).numpy()
    X, Y, S = (ab.Tensor(tuple(t.shape), hdata=host(t), ddata=t, ongpu=True) for t in (x, y, s))
    X.SetSharded(True)
    Y.SetSharded(True)
    te = ab.TensorEngine("Cuda")
    te.SetPeerGroup(peer_group)
    dist.barrier()
    te("S_a_b = X_n_a Y_n_b", S, X, Y)
    torch.cuda.synchronize()
    parts = [torch.empty_like(s) for _ in range(world)]
    mags = [torch.empty_like(s) for _ in range(world)]
    results = [torch.empty_like(s) for _ in range(world)]
    dist.all_gather(parts, x.t() @ y)
    dist.all_gather(mags, x.abs().t() @ y.abs())
    dist.all_gather(results, s)
    total, scale = torch.zeros_like(s), torch.zeros_like(s)
    for p_, m_ in zip(parts, mags):
        total += p_
        scale += m_
    family = te.GetImplementation("S_a_b = X_n_a Y_n_b", S, X, Y).split("family=")[1].split()[0]
    return {"string": "S_a_b = X_n_a Y_n_b", "rows_per_rank": rows, "family": family,
            "max_err_over_sum_abs_terms": float(((s - total).abs() / scale).max().item()),
            "same_bits_on_every_rank": bool(all(torch.equal(r, results[0]) for r in results))}


def cfg0_against_reference(workloads, sessions, batches):
    """N = 1, full size: the README reduction over all 2^26 rows that the GPU just summed, recomputed from the SAME
    inputs (downloaded from the device) by the reference CPU executor exactly as shipped (one thread, its own
    summation order) and by a long-double sum; reports the relative deviations, it gates nothing."""
    from oracle import oracle
    for w, sess, b in zip(workloads, sessions, batches):
        if not w.batch_contracted:
            continue
        t0 = time.perf_counter()
        a, wts = sess.keep["A"].cpu().numpy(), sess.keep["B"].cpu().numpy()
        got = sess.keep[w.names("out")[0]].cpu().numpy()
        ref = np.zeros_like(got)
        kind = "reference" if oracle.have("ref") else "port"
        if kind == "reference":
            oracle.run_ref_slabs([ref, a, wts], [(w.program[0][0], 0, [1, 2])], [False, True, True], b, 1)
        else:
            oracle.contract("port", w.program[0][0], ref, a, wts)
        exact = np.zeros(got.size, dtype=np.longdouble)
        flat = a.reshape(b, -1)
        for r0 in range(0, b, 1 << 22):
            r1 = min(b, r0 + (1 << 22))
            exact += (flat[r0:r1] * wts[r0:r1, None]).sum(axis=0, dtype=np.longdouble)
        exact = exact.reshape(got.shape)
        rel = lambda x, y: float(np.max(np.abs((x.astype(np.longdouble) - y) / y)))
        return {"rows": b, "checker": kind + " CPU executor, one thread, on the inputs downloaded from the device",
                "gpu_vs_reference_executor": float(np.max(np.abs(got - ref) / np.abs(ref))),
                "gpu_vs_long_double_sum": rel(got, exact), "reference_executor_vs_long_double_sum": rel(ref, exact),
                "seconds": round(time.perf_counter() - t0, 1)}
    return None


def spot_check(workloads, sessions, batches, world):
    """Compares a few batch units of every result with the C restatement (untimed)."""
    import torch
    from oracle import oracle
    worst = {}
    for w, sess, b in zip(workloads, sessions, batches):
        if w.batch_contracted:
            continue          # checked by contracted_parity (every rank takes part)
        take = sorted(set([0, b // 2, b - 1]))
        tensors = {}
        for name in w.tensors:
            t = sess.keep[name]
            tensors[name] = (t[take].cpu().numpy() if w.batched(name) else t.cpu().numpy()).copy()
        names = sorted(tensors)
        got = {n: tensors[n].copy() for n in w.names("out")}
        mags = [np.abs(tensors[n]) for n in names]
        prog = [(k, names.index(o), [names.index(i) for i in ins]) for k, o, ins in w.program]
        oracle.run("port", [tensors[n] for n in names], prog, multi=w.multi)
        oracle.run("port", mags, prog, multi=w.multi)
        worst[w.key] = max(oracle.parity_error(got[n], tensors[n], mags[names.index(n)]) for n in w.names("out"))
    return {"max_err_over_sum_abs_terms": worst, "tolerance": 1e-12,
            "note": "sampled batch units of this rank's slab against the oracle; cfg0 (and, for N > 1, the rank sum of a "
                    "Gram string) against the rank-ordered total of every rank's device-side fp64 sum"}


def run_ops(args):
    """Side measurements (not part of the suite), device resident, through the engine API: the batched
    3x3 inverse + determinant that produces cfg 3's inputs on [2^20, 64, 3, 3] (the headline of this
    line), the flat-indexed scatter / sum-gather either side of an operator chain, the mass-operator
    chain at its other compiled geometries, and two finite-element assembly strings of the reference's
    own tests that run on the generic kernel."""
    import torch
    import acrotensor_b200 as ab
    torch.cuda.set_device(0)
    hbm_peak, kind = measured_peaks()
    te = ab.TensorEngine("Cuda")

    def dev_tensor(shape, lo=0.0, hi=1.0, seed=7):
        gen = torch.Generator(device="cuda")
        gen.manual_seed(seed)
        return torch.rand(shape, generator=gen, device="cuda", dtype=torch.float64) * (hi - lo) + lo

    def bind(t):
        return ab.Tensor(tuple(t.shape), hdata=torch.empty(tuple(t.shape), dtype=torch.float64).numpy(), ddata=t, ongpu=True)

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            fn()
        t1.record()
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / args.steps

    def entry(ms, nbytes, note):
        return {"ms": round(ms, 4), "GBps": round(nbytes / ms * 1e-6, 1), "frac_hbm": round(nbytes / ms * 1e-6 / hbm_peak, 4), "what": note}

    per_op = {}
    E = max(1, int((1 << 20) * args.scale))

    # batched inverse + determinant
    J = dev_tensor((E, 64, 3, 3), -0.2, 0.2)
    for d in range(3):
        J[..., d, d] += 1.0
    inv, det = torch.empty_like(J), torch.empty((E, 64), device="cuda", dtype=torch.float64)
    TJ, TI, TD = bind(J), bind(inv), bind(det)
    ms = timed(lambda: te.BatchMatrixInvDet(TI, TD, TJ))
    nbytes = E * 64 * (72 + 72 + 8)
    ident = torch.einsum("ekij,eklj->ekil", J[:64], inv[:64])      # reference layout: inv holds the transposed inverse
    err = float((ident - torch.eye(3, device="cuda", dtype=torch.float64)).abs().max())
    headline = (ms, nbytes)
    del J, inv, det, TJ, TI, TD

    # scatter / sum-gather on a 3D triquadratic-like numbering: 27 entries per element on a (2n+1)^3 grid of
    # domain entries, faces / edges / corners shared by neighbouring elements
    n = max(2, int(round(E ** (1.0 / 3.0))))
    side = 2 * n + 1
    ex, ey, ez = torch.meshgrid(torch.arange(n), torch.arange(n), torch.arange(n), indexing="ij")
    corner = ((2 * ex) * side + 2 * ey) * side + 2 * ez
    offs = torch.tensor([(a * side + b) * side + c for a in (0, 1, 2) for b in (0, 1, 2) for c in (0, 1, 2)])
    mapping = (corner.reshape(-1, 1) + offs.reshape(1, -1)).to(torch.int32).reshape(-1).numpy()
    domain, rng_size = side ** 3, mapping.size
    M = ab.IndexMapping(domain, rng_size, mapping)
    M.ComputeInverse()
    x, u = dev_tensor((domain,)), torch.empty((rng_size,), device="cuda", dtype=torch.float64)
    TX, TU = bind(x), bind(u)
    per_op["flat_indexed_scatter"] = entry(timed(lambda: te.FlatIndexedScatter(TU, TX, M)), rng_size * 12 + domain * 8,
                                           "%d elements x 27 entries from %d domain entries; bytes = map + output + domain once" % (n ** 3, domain))
    per_op["flat_indexed_sum_gather"] = entry(timed(lambda: te.FlatIndexedSumGather(TX, TU, M)), rng_size * 12 + domain * 12,
                                              "same mapping; bytes = input + inverse map + offsets + output")
    del x, u, TX, TU, M

    # the mass-operator chain at its other geometries (cfg 2 is (4,5))
    chain = [("T1_e_i1_i2_k3 = B_k3_i3 U_e_i1_i2_i3", "T1", ["B", "U"]), ("T2_e_i1_k2_k3 = B_k2_i2 T1_e_i1_i2_k3", "T2", ["B", "T1"]),
             ("X_e_k1_k2_k3 = B_k1_i1 T2_e_i1_k2_k3 W_e_k1_k2_k3", "X", ["B", "T2", "W"]), ("Y1_e_i1_k2_k3 = B_k1_i1 X_e_k1_k2_k3", "Y1", ["B", "X"]),
             ("Y2_e_i1_i2_k3 = B_k2_i2 Y1_e_i1_k2_k3", "Y2", ["B", "Y1"]), ("V_e_i1_i2_i3 = B_k3_i3 Y2_e_i1_i2_k3", "V", ["B", "Y2"])]
    for p, q in ((2, 3), (2, 4), (3, 4), (3, 5), (4, 6), (5, 6)):
        Ec = max(1, int((1 << (19 if q >= 6 else 20)) * args.scale))
        shapes = {"B": (q, p), "U": (Ec, p, p, p), "W": (Ec, q, q, q), "T1": (Ec, p, p, q), "T2": (Ec, p, q, q), "X": (Ec, q, q, q),
                  "Y1": (Ec, p, q, q), "Y2": (Ec, p, p, q), "V": (Ec, p, p, p)}
        # the transient intermediates are elided by the fused kernel; to bind they only need storage
        # of the right size, so all five share one device buffer
        spare = torch.empty((Ec * q * q * q,), device="cuda", dtype=torch.float64)
        t = {}
        for k, shape in shapes.items():
            if k in ("B", "U", "W", "V"):
                t[k] = bind(dev_tensor(shape, 0.5, 1.5))
            else:
                t[k] = ab.Tensor(shape, hdata=torch.empty(shape, dtype=torch.float64).numpy(),
                                 ddata=spare[: int(np.prod(shape))].view(shape), ongpu=True)
                t[k].SetTransient(True)

        def step():
            te.BeginMultiKernelLaunch()
            for kernel, out, ins in chain:
                te(kernel, t[out], *[t[i] for i in ins])
            te.EndMultiKernelLaunch()

        per_op["sumfact_mass_p%d_q%d" % (p, q)] = entry(timed(step), Ec * 8 * (2 * p ** 3 + q ** 3), "%d elements, six stages fused" % Ec)
        del t, spare

    # finite-element assembly strings of the reference's tests: one batched input times batch-invariant factors,
    # planned as "multiply the invariant factors out, then one tensor-core GEMM"
    assembly = [
        ("assembly_mass2d", "M_e_i1_i2_j1_j2=B_k1_i1 B_k1_j1 B_k2_i2 B_k2_j2 D_e_k1_k2", ["M", "B", "B", "B", "B", "D"],
         lambda n: {"M": (n, 4, 4, 4, 4), "B": (4, 4), "D": (n, 4, 4)}, 65536),
        ("assembly_stiffness3d", "S_e_i1_i2_i3_j1_j2_j3 = Bt1_i1_j1_k1_m_n Bt2_i2_j2_k2_m_n Bt3_i3_j3_k3_m_n D_e_k1_k2_k3_m_n",
         ["S", "Bt1", "Bt2", "Bt3", "D"],
         lambda n: {"S": (n, 5, 5, 5, 5, 5, 5), "Bt1": (5, 5, 5, 3, 3), "Bt2": (5, 5, 5, 3, 3), "Bt3": (5, 5, 5, 3, 3), "D": (n, 5, 5, 5, 3, 3)}, 256),
        ("assembly_mass_q125", "M_e_i_j = W_e_q B_q_i B_q_j", ["M", "W", "B", "B"],
         lambda n: {"M": (n, 64, 64), "W": (n, 125), "B": (125, 64)}, 32768),
    ]
    for key, kernel, names, shapes_of, full in assembly:
        n = max(64, int(full * args.scale))
        dev = {k: dev_tensor(v, -1, 1) for k, v in shapes_of(n).items()}
        t = {k: bind(v) for k, v in dev.items()}
        operands = [t[k] for k in names]
        plan_line = [l for l in te.GetImplementation(kernel, *operands).splitlines() if l.startswith("step 0")][0]
        ms_a = timed(lambda: te(kernel, *operands))
        flops = float(plan_line.split("flops=")[1].split()[0])
        e = entry(ms_a, float(plan_line.split("bytes=")[1].split()[0]), "%d elements; %s" % (n, plan_line.split("family=")[1].split()[0]))
        e["TFLOPps"] = round(flops / ms_a * 1e-9, 2)
        per_op[key] = e
        del dev, t, operands

    # element matrices: products of small matrices, and their action on element vectors
    for key, kernel, shapes_of, full in [
            ("batched_gemm_8", "C_e_i_j = A_e_i_k B_e_k_j", lambda n: [(n, 8, 8), (n, 8, 8), (n, 8, 8)], 1 << 21),
            ("batched_gemm_27", "C_e_i_j = A_e_i_k B_e_k_j", lambda n: [(n, 27, 27), (n, 27, 27), (n, 27, 27)], 1 << 17),
            ("batched_gemm_8_transposed", "C_e_i_j = A_e_k_i B_e_j_k", lambda n: [(n, 8, 8), (n, 8, 8), (n, 8, 8)], 1 << 21),
            ("batched_gemm_27_transposed", "C_e_i_j = A_e_k_i B_e_j_k", lambda n: [(n, 27, 27), (n, 27, 27), (n, 27, 27)], 1 << 17),
            ("batched_gemm_64", "C_e_i_j = A_e_i_k B_e_k_j", lambda n: [(n, 64, 64), (n, 64, 64), (n, 64, 64)], 1 << 14),
            ("batched_gemm_64_transposed", "C_e_i_j = A_e_k_i B_e_j_k", lambda n: [(n, 64, 64), (n, 64, 64), (n, 64, 64)], 1 << 14),
            ("gram_8", "S_a_b = X_n_a Y_n_b", lambda n: [(8, 8), (n, 8), (n, 8)], 1 << 23),
            ("gram_27", "S_a_b = X_n_a Y_n_b", lambda n: [(27, 27), (n, 27), (n, 27)], 1 << 21),
            ("gram_64", "S_a_b = X_n_a Y_n_b", lambda n: [(64, 64), (n, 64), (n, 64)], 1 << 20),
            ("batched_matvec_27", "Y_e_i = M_e_i_j X_e_j", lambda n: [(n, 27), (n, 27, 27), (n, 27)], 1 << 18),
            ("batched_matvec_64", "Y_e_i = M_e_i_j X_e_j", lambda n: [(n, 64), (n, 64, 64), (n, 64)], 1 << 15)]:
        n = max(64, int(full * args.scale))
        dev = [dev_tensor(shape, -1, 1) for shape in shapes_of(n)]
        operands = [bind(t) for t in dev]
        plan_line = [l for l in te.GetImplementation(kernel, *operands).splitlines() if l.startswith("step 0")][0]
        per_op[key] = entry(timed(lambda: te(kernel, *operands)), float(plan_line.split("bytes=")[1].split()[0]),
                            "%d elements; %s" % (n, plan_line.split("|")[1].strip()[:90]))
        del dev, operands

    ms, nbytes = headline
    print(json.dumps({"metric": "batch_inv_det_throughput", "value": round(nbytes / ms * 1e-6, 1), "unit": "GB/s", "n_gpus": 1,
                      "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4), "dtype": "f64",
                      "config": {"workload": "BatchMatrixInvDet on [%d,64,3,3]" % E},
                      "roofline": {"bound": "hbm", "achieved": round(nbytes / ms * 1e-6, 1), "peak": hbm_peak, "unit": "GB/s",
                                   "frac": round(nbytes / ms * 1e-6 / hbm_peak, 4), "traffic": None},
                      "identity_error": err, "per_op": per_op}))


# ----------------------------------------------------------------------------- CPU arms

class CpuSample:
    """A bounded sample of every selected workload for the reference CPU executor: seeded host
    inputs for a leading slab of the batch, generated once and reused by every pass."""

    def __init__(self, workloads, args, sample_scale):
        from acrotensor_b200.runner import alloc_host
        self.items = []
        for w in workloads:
            full = max(1, int(round(w.batch * args.scale)))
            sample = max(1, min(full, int(CPU_SAMPLE[w.key] * sample_scale)))
            host = alloc_host(w, sample, w.make_inputs(sample, seed=args.seed))
            names = sorted(host)
            prog = [(k, names.index(o), [names.index(i) for i in ins]) for k, o, ins in w.program]
            self.items.append((w, full, sample, [host[n] for n in names], prog, [w.batched(n) for n in names]))

    def run(self, threads):
        """One pass.  Returns (suite GB/s extrapolated to the full batches, extrapolated seconds,
        per-configuration detail, 'reference' | 'port')."""
        from oracle import oracle
        full_seconds, detail, total_bytes = 0.0, {}, 0
        kind = "reference" if oracle.have("ref") else "port"
        for w, full, sample, arrays, prog, batched in self.items:
            t0 = time.perf_counter()
            if kind == "reference":
                oracle.run_ref_slabs(arrays, prog, batched, sample, threads, multi=w.multi)
            else:
                oracle.run("port", arrays, prog, multi=w.multi)
            sec = time.perf_counter() - t0
            # the interpreted executor's cost is linear in the batch
            full_s = sec * (full / sample)
            full_seconds += full_s
            total_bytes += w.bytes(full)
            detail[w.key] = {"sample_batch": sample, "sample_s": round(sec, 3), "full_s_extrapolated": round(full_s, 2)}
        return total_bytes / full_seconds * 1e-9, full_seconds, detail, kind


def cpu_sample_for_seconds(workloads, args, threads, seconds_per_pass):
    """Calibrates on a small sample, then sizes the sample so that one pass takes about
    `seconds_per_pass` on this machine."""
    small = CpuSample(workloads, args, 0.25)
    t0 = time.perf_counter()
    small.run(threads)
    took = max(time.perf_counter() - t0, 1e-3)
    scale = 0.25 * seconds_per_pass / took
    return CpuSample(workloads, args, max(0.05, scale))


def host_threads():
    from oracle import oracle
    try:
        return min(oracle.hardware_threads(), len(os.sched_getaffinity(0)))
    except Exception:
        return os.cpu_count() or 1


def cpu_baseline(workloads, args):
    from oracle import oracle
    threads = host_threads() if oracle.have("ref") else 1
    sample = cpu_sample_for_seconds(workloads, args, threads, 10.0)
    gbs, full_s, detail, kind = sample.run(threads)
    return {"value": round(gbs, 4), "unit": "GB/s", "cores": threads, "kind": kind,
            "sample": "per configuration a leading slab of the batch (sizes in detail), time scaled linearly to the full batch",
            "full_suite_seconds_extrapolated": round(full_s, 1), "detail": detail}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle
    if not oracle.have("port"):
        oracle.build()
    workloads = selected(args.workload)
    world = max(1, int(os.environ.get("WORLD_SIZE", str(args.gpus))))
    threads = host_threads() if oracle.have("ref") else 1
    # every pass is a bounded sample; the whole run stays within a few minutes
    per_pass = max(0.5, min(8.0, 150.0 / (args.steps + args.warmup)))
    sample = cpu_sample_for_seconds(workloads, args, threads, per_pass)
    for _ in range(args.warmup):
        sample.run(threads)
    vals, secs = [], []
    t0 = time.perf_counter()
    for _ in range(args.steps):
        gbs, full_s, detail, kind = sample.run(threads)
        vals.append(gbs)
        secs.append(full_s)
    wall = time.perf_counter() - t0
    value = float(np.median(vals))
    base = {"value": round(value, 4), "unit": "GB/s", "cores": threads, "kind": kind,
            "sample": "per configuration a leading slab of the batch, time scaled linearly to the full batch",
            "detail": detail}
    print(json.dumps({
        "impl": "reference", "metric": "contraction_throughput", "value": round(value, 4), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(float(np.median(secs)) * 1e3, 1), "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": "f64", "data": "synthetic (seeded)",
        "config": config_of(args, world, workloads, [local_batch(w, args, 0, world) for w in workloads]),
        "reference_note": "reference CPUInterpreted executor on the host cores, the whole job (all slabs) on one host; "
                          "ms_per_step is the full-size suite extrapolated from the sample",
        "wall_s": round(wall, 1),
        "cpu_baseline": base,
        "e2e": {"value": round(value, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="suite", choices=["suite", "cfg0", "cfg1", "cfg2", "cfg3", "cfg4", "ops"])
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"],
                    help="N > 1: strong = the benchmark sizes cut into N slabs (default), weak = a full-size slab per rank")
    ap.add_argument("--scale", type=float, default=1.0, help="multiplies every batch size (debugging; 1.0 = benchmark sizes)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--e2e-mode", default="auto", choices=["auto", "all", "one", "skip"],
                    help="pinned host buffers for the end-to-end leg: all configurations at once, one at a time, or none")
    ap.add_argument("--allreduce", default="fused", choices=["fused", "nccl"],
                    help="N > 1: how the contracted batch index of the README reduction is summed over ranks")
    ap.add_argument("--streams", default="one", choices=["one", "per-config"],
                    help="per-config: every configuration's engine launches on a stream of its own in the timed pass")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.workload == "ops":
        run_ops(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
