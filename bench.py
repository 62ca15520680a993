"""Benchmark of the data-parallel optimizer path: gradient mean over ranks + 1/world scaling + AdamW, fused.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference-gpu] [--model 124M|medium]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --fabric --gpus N          # what the NVLink fabric itself delivers (one process, all GPUs)
    python bench.py --sweep --gpus N           # bucket sizes 4 KB .. 1 GB, one-shot against two-shot

Workload: the GPT-2 124M parameter set (148 tensors, 124,439,808 fp32 parameters; soliton_b200/workload.py),
parameters seeded as the reference's example initialises them, per-rank gradients N(0, 1e-3) seeded by rank,
m = v = 0, lr 3e-4, betas (0.9, 0.999), eps 1e-8, weight decay 0.1 on matrices. A step is one pass of the path over
all tensors through the Soliton-shaped Python interface: distributed.all_reduce_grads(params); optimizer.step().
Inputs (2 GB per rank) are far larger than L2, so nothing is flushed between iterations.

Prints ONE JSON line on rank 0. `value` is GB/s of algorithmic HBM traffic (28 bytes per parameter per rank: read
g, p, m, v; write p, m, v) summed over all ranks, inputs resident in HBM; the timed region of K steps is repeated
and the median reported, with the spread beside it. `e2e` is the same metric for a host-fed step: inside the timed
region every step uploads its gradients from pinned host memory and reads the updated parameters back, bucket by
bucket over the library's copy streams, and ends when the parameters are on the host. `parity` is one checked run of
the same kernels on a small tensor set, against the CPU oracle bit for bit and across ranks by hash. `gpu_baseline`
is the reference's own GPU path (grouped ncclAllReduce(avg) + one k_adamw launch per tensor, built unmodified into
oracle/_ref/) timed in the same job. `--impl reference` times the reference's host path (CPU restatement of
core/soliton/cpu.d: axpy per rank, scale, adamw; the D core cannot be built here) on the host cores.
"""
import argparse
import ctypes
import hashlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "fused_allreduce_adamw_algorithmic_GBps"
BYTES_PER_PARAM = 28            # algorithmic HBM bytes per parameter per rank
NVLINK_NOMINAL_GBS = 900.0      # per direction per GPU
NVLINK_ONE_WAY_GBS = 770.0      # this pool's peer-copy figure with the links loaded one way (the fabric probe of this file
                                # gives 718-753 to a pulling kernel and up to 792 to the copy engines in that case)
# What `bench.py --fabric` measured on this pool's 8 x B200 boxes when every GPU exchanges with every other at once, so
# that every link carries data both ways as in an all-reduce: GB/s per GPU, the slowest GPU of the group, by a kernel
# pulling with 256-bit loads (what the two-shot exchange does), by a kernel pushing with 256-bit stores, and with
# every link loaded one way only.
FABRIC_MEASURED_GBS = {2: {"sm_pull": 615.6, "sm_push": 657.3, "sm_pull_one_direction": 718.4},
                       4: {"sm_pull": 631.4, "sm_push": 677.5, "sm_pull_one_direction": 730.0},
                       8: {"sm_pull": 641.1, "sm_push": 684.9, "sm_pull_one_direction": 737.8}}
FALLBACK_HBM_GBS = 6650.0       # used only when MEASURED_PEAKS.json is absent
# DRAM bytes per parameter of the dominant kernel from an ncu capture, per world size; None = not captured
NCU_DRAM_BYTES_PER_PARAM = {1: 27.31}
# A small tensor set for the checked run: 1.6 M floats, above the one-shot staging slot at every world size
PARITY_SHAPES = [(1000, 1200), (1200,), (300, 1000), (1000,), (3,), (2048 * 50,)]


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"])
    ap.add_argument("--model", default="124M", choices=["124M", "medium", "tiny"])
    ap.add_argument("--flat", type=int, default=0, help="one flat buffer of this many bytes instead of a model")
    ap.add_argument("--regions", type=int, default=5, help="how often the timed region of --steps steps is repeated")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--bucket-mb", type=int, default=32, help="bucket size of the host-fed step")
    ap.add_argument("--wc", action="store_true", help="write-combined pinned memory for the upload sources")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gpu-baseline", action="store_true")
    ap.add_argument("--mode", type=int, default=0, help="0 auto, 1 one-shot, 2 two-shot")
    ap.add_argument("--blocks-per-sm", type=int, default=0)
    ap.add_argument("--cyclic", type=int, default=-1)
    ap.add_argument("--stamps", action="store_true", help="device times at the phase borders of the last launch")
    ap.add_argument("--sweep", action="store_true", help="bucket-size sweep 4 KB .. 1 GB, one-shot vs two-shot (N >= 2)")
    ap.add_argument("--fabric", action="store_true", help="NVLink fabric ceiling: copy engines and kernels, one and both directions")
    ap.add_argument("--bare", action="store_true", help="gradient mean only, no optimizer update (link-bound floor)")
    ap.add_argument("--attention", action="store_true", help="fused causal attention against the reference's TF32 path")
    ap.add_argument("--xent", action="store_true", help="cross entropy forward and backward against the reference's kernels")
    ap.add_argument("--elementwise", action="store_true", help="binary ops and embedding backward against the reference's kernels")
    ap.add_argument("--layernorm", action="store_true", help="layer normalisation forward and backward against the reference's kernels")
    return ap.parse_args()


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and clock-event (throttle) reasons of one GPU every few milliseconds while the timed region
    runs: NVML in a thread of this process (read-only queries), nvidia-smi as a fallback."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        self.index, self.sm, self.mask, self.max_mhz = index, [], 0, None
        self.stop_flag, self.thread, self.nvml, self.proc = threading.Event(), None, None, None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[self.index]) if visible and visible.split(",")[self.index].isdigit() else self.index
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
        except Exception:
            self.nvml = None
            self._start_smi()

    def _poll(self):
        n = self.nvml
        while not self.stop_flag.is_set():
            try:
                self.sm.append(float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)))
                reasons = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
                self.mask |= int(reasons(self.handle))
            except Exception:
                pass
            time.sleep(0.004)

    def _start_smi(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", "--query-gpu=clocks.sm,clocks.max.sm,"
                                          "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                                          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.rows = []
            self.thread = threading.Thread(target=lambda: self.rows.extend(l.split(",") for l in self.proc.stdout), daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def stop(self):
        if self.nvml:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            sm = sorted(self.sm)
            return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_mhz,
                    "reasons": [name for bit, name in self.REASONS.items() if self.mask & bit], "samples": len(sm),
                    "source": "nvml"}
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock source available"], "samples": 0}
        time.sleep(0.1)
        self.proc.terminate()  # the exact process started above
        self.proc.wait()
        self.thread.join(timeout=2)
        rows = [[x.strip() for x in r] for r in self.rows if len(r) >= 6]
        sm = sorted(float(r[0]) for r in rows if r[0].replace(".", "").isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        mx = [float(r[1]) for r in rows if r[1].replace(".", "").isdigit()]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx[0] if mx else None, "reasons": reasons,
                "samples": len(sm), "source": "nvidia-smi"}


def workload_name(args):
    if args.flat:
        return f"flat fp32 buffer, {args.flat} bytes"
    from soliton_b200 import workload
    return f"GPT-2 {args.model} parameter set, {len(workload.param_shapes(args.model))} tensors"


def make_workload(args):
    """Shapes and per-rank host arrays (params identical on all ranks, gradients seeded by rank). A flat buffer is
    given the shape (1, n): a matrix, so that it takes weight decay as BASELINE's flat configurations say."""
    from soliton_b200 import workload
    if args.flat:
        n = args.flat // 4
        shapes = [(1, n)]
        make_p = lambda: [workload.flat_case(n)[0].reshape(1, n)]                        # noqa: E731
        make_g = lambda rank: [workload.flat_case(n, rank=rank)[1].reshape(1, n)]        # noqa: E731
    else:
        shapes = [s for _, s, _ in workload.param_shapes(args.model)]
        make_p = lambda: workload.init_params(args.model, seed=0)                        # noqa: E731
        make_g = lambda rank: workload.rank_grads(args.model, rank=rank)                 # noqa: E731
    return shapes, make_p, make_g


def total_params(args):
    from soliton_b200 import workload
    return args.flat // 4 if args.flat else workload.total_params(args.model)


def host_path_seconds(args, world, steps, threads):
    """Seconds for `steps` steps of the reference's host path over the WHOLE workload on each of `threads` threads
    (one thread stands for one rank's process: the reference's host kernels are single-threaded loops)."""
    import numpy as np
    from oracle import pyoracle
    n = total_params(args)
    p0 = np.random.default_rng(0).standard_normal(n, dtype=np.float32) * np.float32(0.02)
    grads = [np.random.default_rng(1 + r).standard_normal(n, dtype=np.float32) * np.float32(1e-3) for r in range(world)]
    return pyoracle.bench(p0, grads, steps, threads), n


def run_reference(args, rank, world):
    """The reference's host path (restated; core/soliton/cpu.d:85-101,362-373) on the host cores, over the same
    parameter set as the GPU arm: every one of `world` threads, standing for one rank's process, sums the ranks'
    gradients, scales and runs AdamW."""
    if rank != 0:
        return
    cores = min(world, os.cpu_count() or 1)
    host_path_seconds(args, world, max(args.warmup, 1), cores)
    t, n = host_path_seconds(args, world, args.steps, cores)
    ms = 1e3 * t / args.steps
    value = cores * BYTES_PER_PARAM * n / (t / args.steps) / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args), "params_per_rank": n, "world": world},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": f"all {n} parameters per step, {args.steps} steps, one thread per rank "
                                   f"(the reference's host kernels are single-threaded loops)"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def cpu_baseline(args):
    """Rank 0, N = 1: the host path on one core over the whole parameter set, about ten seconds of CPU work."""
    t1, n = host_path_seconds(args, 1, 2, 1)
    reps = max(3, min(50, int(10.0 / max(t1 / 2, 1e-4))))
    t, n = host_path_seconds(args, 1, reps, 1)
    return {"value": BYTES_PER_PARAM * n * reps / t / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
            "sample": f"all {n} parameters, {reps} steps, single thread as in core/soliton/cpu.d",
            "ms_per_step": 1e3 * t / reps, "host_cores_available": os.cpu_count()}


def bind_near_gpu(lib, ordinal):
    """Keeps this process (and the pages of the pinned buffers it allocates next) on the NUMA node the GPU hangs on,
    so that eight ranks feeding eight GPUs do not pull each other's host memory across the socket link."""
    try:
        buf = ctypes.create_string_buffer(32)
        if lib.slb_device_pci_bus_id(ordinal, buf, 32) != 0:
            return None
        node = int(open(f"/sys/bus/pci/devices/{buf.value.decode().lower()}/numa_node").read())
        if node < 0:
            return None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0) & cpus
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except Exception:
        return None


class Pinned:
    """float32 buffer in page-locked host memory from the library."""

    def __init__(self, lib, n, write_combined=False):
        import numpy as np
        self.lib, self.ptr = lib, (lib.slb_pinned_alloc_wc if write_combined else lib.slb_pinned_alloc)(4 * n)
        if not self.ptr:
            raise MemoryError("pinned host allocation failed")
        self.array = np.ctypeslib.as_array(ctypes.cast(self.ptr, ctypes.POINTER(ctypes.c_float)), shape=(n,))

    def data_ptr(self):
        return self.ptr


def reference_gpu_lib():
    from oracle import build as obuild
    if not os.path.exists(obuild.REF_SO):
        return None
    C = ctypes
    R = C.CDLL(obuild.REF_SO)
    R.sl_cuda_malloc.restype = C.c_void_p
    R.sl_cuda_malloc.argtypes = [C.c_size_t]
    R.sl_cuda_free.argtypes = [C.c_void_p]
    R.sl_cuda_h2d.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
    R.sl_cuda_adamw.argtypes = [C.c_void_p] * 4 + [C.c_int64] + [C.c_float] * 5 + [C.c_int]
    R.sl_cuda_nccl_allreduce_mean.argtypes = [C.c_void_p, C.c_int64]
    R.sl_cuda_fill.argtypes = [C.c_void_p, C.c_int64, C.c_float]
    return R


def time_reference_gpu(args, R, rank, local_rank, world, dist, steps, warmup):
    """ms per step (max over ranks) of the reference's own GPU path on this box: grouped ncclAllReduce(avg) per tensor,
    then one k_adamw launch per tensor (core/cuda/kernels.cu:242-254,772-775)."""
    import numpy as np
    import torch
    from soliton_b200 import workload
    C = ctypes
    assert R.sl_cuda_set_device(local_rank) == 0
    if world > 1:
        idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            buf = C.create_string_buffer(128)
            assert R.sl_cuda_nccl_unique_id(buf) == 0
            idt.copy_(torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8))
        dist.broadcast(idt, 0)
        assert R.sl_cuda_nccl_init(rank, world, C.create_string_buffer(bytes(idt.cpu().numpy().tobytes()), 128)) == 0
    shapes, make_p, make_g = make_workload(args)
    H = workload.HYPER
    bufs = []
    for a, gr in zip(make_p(), make_g(rank)):
        n = int(a.size)
        ptrs = [R.sl_cuda_malloc(4 * n) for _ in range(4)]
        R.sl_cuda_h2d(ptrs[0], np.ascontiguousarray(a).ctypes.data, 4 * n)
        R.sl_cuda_h2d(ptrs[1], np.ascontiguousarray(gr).ctypes.data, 4 * n)
        R.sl_cuda_fill(ptrs[2], n, 0.0)
        R.sl_cuda_fill(ptrs[3], n, 0.0)
        bufs.append((ptrs, n, H["wd"] if len(a.shape) >= 2 else 0.0))
    t = [0]

    def step():
        t[0] += 1
        if world > 1:
            R.sl_cuda_nccl_group(1)
            for ptrs, n, _ in bufs:
                R.sl_cuda_nccl_allreduce_mean(ptrs[1], n)
            R.sl_cuda_nccl_group(0)
        for ptrs, n, wd in bufs:
            R.sl_cuda_adamw(ptrs[0], ptrs[1], ptrs[2], ptrs[3], n, H["lr"], H["b1"], H["b2"], H["eps"], wd, t[0])

    for _ in range(max(warmup, 3)):
        step()
    R.sl_cuda_sync()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    R.sl_cuda_sync()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    assert R.sl_cuda_check() == 0
    if world > 1:
        R.sl_cuda_nccl_destroy()
    for ptrs, _, _ in bufs:
        for p in ptrs:
            R.sl_cuda_free(p)
    return float(ms.item()), len(bufs) + (1 if world > 1 else 0)


def nccl_version():
    try:
        import torch
        return ".".join(str(x) for x in torch.cuda.nccl.version())
    except Exception:
        return None


def parity_check(rank, world, dist):
    """One checked run of the path on a small tensor set: two steps through the same calls as the timed region, then
    every rank compares parameters, moments and gradients with the CPU oracle bit for bit, and the ranks compare a
    hash of their parameters."""
    import numpy as np
    from oracle import pyoracle
    from soliton_b200 import distributed, tensor as T, workload
    from soliton_b200._C import counter
    from soliton_b200.optim import AdamW
    H = workload.HYPER
    shapes = PARITY_SHAPES
    p0 = [(np.random.default_rng(100 + i).standard_normal(s) * 0.02).astype(np.float32) for i, s in enumerate(shapes)]
    grads = lambda r, step: [(np.random.default_rng(1000 * step + 10 * r + i).standard_normal(s) * 1e-3).astype(np.float32)  # noqa: E731
                             for i, s in enumerate(shapes)]
    params = [T.tensor(a, "cuda") for a in p0]
    opt = AdamW(params, lr=H["lr"], betas=(H["b1"], H["b2"]), eps=H["eps"], weight_decay=H["wd"])
    ref = [[a.ravel().copy(), np.zeros(a.size, np.float32), np.zeros(a.size, np.float32)] for a in p0]
    ok = True
    for step in (1, 2):
        for p, g in zip(params, grads(rank, step)):
            p.grad = T.tensor(g, "cuda")
        distributed.all_reduce_grads(opt.params)
        opt.step()
        T.synchronize()
        mode = counter("last_mode")
        per_rank = [grads(r, step) for r in range(world)]
        for i, s in enumerate(shapes):
            mean = pyoracle.mean_ranks([per_rank[r][i].ravel() for r in range(world)])
            pyoracle.adamw(ref[i][0], mean, ref[i][1], ref[i][2], H["lr"], H["b1"], H["b2"], H["eps"],
                           H["wd"] if len(s) >= 2 else 0.0, step, fma=True)
            ok = ok and np.array_equal(params[i].grad.numpy().ravel(), mean)
            ok = ok and np.array_equal(params[i].numpy().ravel(), ref[i][0])
            ok = ok and np.array_equal(opt.state[i][0].numpy().ravel(), ref[i][1])
            ok = ok and np.array_equal(opt.state[i][1].numpy().ravel(), ref[i][2])
        opt.zero_grad()
    digest = hashlib.sha256(b"".join(p.numpy().tobytes() for p in params)).hexdigest()
    all_ok, digests = [ok], [digest]
    if world > 1:
        all_ok, digests = [None] * world, [None] * world
        dist.all_gather_object(all_ok, ok)
        dist.all_gather_object(digests, digest)
    return {"vs_oracle_bits": bool(all(all_ok)), "cross_rank_hash_equal": len(set(digests)) == 1, "world": world,
            "kernel": {0: "k_twoshot<1,adam>", 1: f"k_oneshot<{world},adam>", 2: f"k_twoshot<{world},adam>"}[mode],
            "tensors": len(shapes), "params": int(sum(a.size for a in p0)), "steps": 2, "sha256_p": digest[:16]}


def run_ours(args, rank, local_rank, world):
    import numpy as np
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    from soliton_b200 import distributed, tensor as T, workload
    from soliton_b200._C import counter, lib, set_option
    from soliton_b200.bucketed import BucketedAdamW
    from soliton_b200.optim import AdamW
    H = workload.HYPER
    numa = bind_near_gpu(lib, local_rank)

    T.set_device(local_rank)
    T._dev(T.CUDA)
    for name, value in (("mode", args.mode), ("blocks_per_sm", args.blocks_per_sm)):
        if value:
            set_option(name, value)
    if args.cyclic >= 0:
        set_option("cyclic", args.cyclic)
    if args.stamps:
        set_option("stamps", 1)

    # the same-box GPU baseline first: the reference's own NCCL + k_adamw path, in this job, on this workload
    gpu_baseline = None
    if not args.no_gpu_baseline and not args.bare:
        R = reference_gpu_lib()
        if R is None:
            gpu_baseline = {"unavailable": "oracle/_ref/ not built (no reference checkout at build time)"}
        else:
            ms_ref, launches_ref = time_reference_gpu(args, R, rank, local_rank, world, dist, 10, 3)
            gpu_baseline = {"kind": "reference ncclAllReduce(avg) grouped + one k_adamw per tensor, oracle/_ref",
                            "ms_per_step": ms_ref, "launches_per_step": launches_ref, "nccl": nccl_version(), "steps": 10}

    if world > 1:
        idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            idt.copy_(torch.frombuffer(bytearray(distributed.unique_id()), dtype=torch.uint8))
        dist.broadcast(idt, 0)
        distributed.init_with_id(rank, world, bytes(idt.cpu().numpy().tobytes()))

    parity = parity_check(rank, world, dist)

    # device state through the library's allocator; host copies of the gradients in pinned memory for the e2e leg
    shapes, make_p, make_g = make_workload(args)
    host_p = make_p()
    host_g = make_g(rank)
    P = sum(int(a.size) for a in host_p)
    params = [T.tensor(a, "cuda") for a in host_p]
    pinned_g = [Pinned(lib, int(a.size), write_combined=args.wc) for a in host_g]
    for buf, a in zip(pinned_g, host_g):
        buf.array[:] = a.ravel()
    pinned_out = [Pinned(lib, int(a.size)) for a in host_p]
    for p, a in zip(params, host_g):
        p.grad = T.tensor(a, "cuda")
    del host_p, host_g

    opt = BucketedAdamW(params, bucket_bytes=args.bucket_mb << 20, lr=H["lr"], betas=(H["b1"], H["b2"]), eps=H["eps"],
                        weight_decay=H["wd"])

    def step():
        distributed.all_reduce_grads(opt.params)
        if args.bare:
            lib.slb_flush()
        else:
            AdamW.step(opt)   # the whole step as one launch

    def fence():
        lib.slb_flush()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(nsteps, body):
        fence()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(nsteps):
            body()
        lib.slb_flush()  # the last step's launch goes out before the closing event
        e1.record()
        fence()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(max(args.warmup, 3)):
        step()
    fence()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = counter("launches")
    region_ms = [timed(args.steps, step) / args.steps for _ in range(max(args.regions, 1))]
    launches = (counter("launches") - launches0) // max(args.regions, 1)
    clocks = sampler.stop() if rank == 0 else None
    err = lib.sl_check(T.CUDA)
    if err:
        raise RuntimeError(f"soliton_b200: sticky error {err} after the timed region")
    mode, blocks = counter("last_mode"), counter("last_blocks")
    stamps = None
    if args.stamps and world > 1:
        raw = (ctypes.c_uint64 * 5)()
        if lib.slb_read_stamps(raw) == 0:
            t = [int(x) for x in raw]
            stamps = {"us_wait_for_peers": (t[1] - t[0]) / 1e3, "us_reduce_own_chunk": (t[2] - t[1]) / 1e3,
                      "us_gather_other_chunks": (t[3] - t[2]) / 1e3, "us_wait_peers_done": (t[4] - t[3]) / 1e3,
                      "us_total_block0": (t[4] - t[0]) / 1e3}

    # host-fed step: gradients up, parameters down, bucket by bucket over the copy streams
    # gradients differ per rank: every rank uploads its own; parameters come out identical on all ranks: each rank
    # reads back its 1 / world share, so that the job has them on the host once
    opt.bind_host(pinned_g, pinned_out, share=(rank, world))
    e2e_ms, breakdown = None, None
    if not args.bare:
        opt.host_step()
        e2e_ms = timed(args.e2e_steps, opt.host_step) / args.e2e_steps

        def uploads():
            for b in range(len(opt.buckets)):
                opt.upload(b)
            lib.slb_wait_copies()

        def downloads():
            for b in range(len(opt.buckets)):
                opt.download(b)
            lib.slb_wait_copies()

        breakdown = {"h2d_ms": timed(2, uploads) / 2, "d2h_ms": timed(2, downloads) / 2, "kernel_ms": statistics.median(region_ms),
                     "buckets": len(opt.buckets), "numa_node": numa}
        if world > 1:
            per_rank = [None] * world
            dist.all_gather_object(per_rank, {"rank": rank, "numa_node": numa})
            breakdown["ranks"] = per_rank
    err = lib.sl_check(T.CUDA)
    if err:
        raise RuntimeError(f"soliton_b200: sticky error {err} after the host-fed steps")

    if rank != 0:
        if world > 1:
            distributed.destroy()
            dist.destroy_process_group()
        return
    ms = statistics.median(region_ms)
    value = world * BYTES_PER_PARAM * P / (ms * 1e-3) / 1e9
    hbm, hbm_kind = hbm_peak()
    hbm_per_rank = BYTES_PER_PARAM * P / (ms * 1e-3) / 1e9
    t_hbm = BYTES_PER_PARAM * P / (hbm * 1e9)
    nvl_bytes = 8.0 * P * (world - 1) / world
    fabric = FABRIC_MEASURED_GBS.get(world)
    t_nvl = nvl_bytes / (NVLINK_ONE_WAY_GBS * 1e9)
    kernel = {0: "k_twoshot<1,adam>", 1: f"k_oneshot<{world},adam>", 2: f"k_twoshot<{world},adam>"}[mode]
    if args.bare:
        kernel = kernel.replace(",adam>", ",mean only>")
    traffic = NCU_DRAM_BYTES_PER_PARAM.get(world)
    if t_hbm >= t_nvl:
        roof = {"bound": "hbm", "achieved": hbm_per_rank, "peak": hbm, "unit": "GB/s", "frac": hbm_per_rank / hbm,
                "traffic": traffic * P if traffic else None, "peak_source": f"{hbm_kind} HBM copy"}
    else:
        nvl = nvl_bytes / (ms * 1e-3) / 1e9
        roof = {"bound": "nvlink", "achieved": nvl, "peak": NVLINK_ONE_WAY_GBS, "unit": "GB/s", "frac": nvl / NVLINK_ONE_WAY_GBS,
                "traffic": traffic * P if traffic else None,
                "peak_source": "peer copy per direction per GPU with the links loaded one way (nominal 900)",
                "frac_of_nominal_900": nvl / NVLINK_NOMINAL_GBS,
                "fabric_measured_two_way": fabric, "frac_of_fabric_measured_two_way": nvl / fabric["sm_pull"] if fabric else None,
                "hbm_achieved": hbm_per_rank, "hbm_peak": hbm, "hbm_frac": hbm_per_rank / hbm}
    roof.update({"kernel": kernel, "ms_per_launch": ms / max(launches / args.steps, 1), "roofline_ms": 1e3 * max(t_hbm, t_nvl),
                 "frac_of_roofline_time": max(t_hbm, t_nvl) / (ms * 1e-3)})
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args), "params_per_rank": P, "world": world,
                   "l2": "inputs larger than L2, no flush",
                   "exchange": {0: "none", 1: "one-shot", 2: "two-shot"}[mode], "blocks_per_rank": blocks,
                   "optimizer": "none (--bare)" if args.bare else "AdamW",
                   "arithmetic": "gradient mean, m, v in f32; parameter update in f64, rounded to f32 once",
                   "e2e_copies": "h2d: this rank's gradients from pinned memory; d2h: updated parameters, each rank its "
                                 "1/world share (all ranks hold the same bits, checked in `parity`); "
                                 f"buckets of {args.bucket_mb} MiB over two copy streams beside the kernels"},
        "regions": {"n": len(region_ms), "steps_each": args.steps, "ms_per_step_median": ms,
                    "ms_per_step_min": min(region_ms), "ms_per_step_max": max(region_ms)},
        "roofline": roof, "parity": parity, "gpu_baseline": gpu_baseline,
        "gpu_launches": int(launches), "clocks": clocks,
    }
    if e2e_ms is not None:
        line["e2e"] = {"value": world * BYTES_PER_PARAM * P / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                       "h2d_bytes_per_step": opt.upload_bytes, "d2h_bytes_per_step": opt.download_bytes,
                       "bytes_are": "per rank; the job moves world x h2d up and, over all ranks together, every parameter down once",
                       "ms_per_step": e2e_ms,
                       "steps": args.e2e_steps, "breakdown": breakdown}
    if stamps:
        line["phases_block0_last_launch"] = stamps
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args)
    print(json.dumps(line), flush=True)
    if world > 1:
        distributed.destroy()
        dist.destroy_process_group()


def run_sweep(args, rank, local_rank, world):
    """Flat fp32 buffers of 4^k bytes, k = 6..15, through the fused path with the exchange forced to one-shot (where the
    buffer fits a staging slot) and to two-shot; one JSON line with a row per (size, exchange)."""
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    from soliton_b200 import distributed, tensor as T, workload
    from soliton_b200._C import counter, lib, set_option
    H = workload.HYPER
    T.set_device(local_rank)
    T._dev(T.CUDA)
    idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
    if rank == 0:
        idt.copy_(torch.frombuffer(bytearray(distributed.unique_id()), dtype=torch.uint8))
    dist.broadcast(idt, 0)
    distributed.init_with_id(rank, world, bytes(idt.cpu().numpy().tobytes()))
    rows = []
    for k in range(6, 16):
        nbytes = 4 ** k
        n = nbytes // 4
        p0, g0 = workload.flat_case(n, rank=rank)
        p, g, m, v = T.tensor(p0, "cuda"), T.tensor(g0, "cuda"), T.zeros((n,), "cuda"), T.zeros((n,), "cuda")
        steps = 200 if nbytes <= (1 << 24) else 30
        for mode in (1, 2):
            if mode == 1 and nbytes > (16 << 20) // (2 * world):
                continue
            set_option("mode", mode)

            def step(t=[0]):
                t[0] += 1
                lib.sl_dist_group(T.CUDA, 1)
                lib.sl_dist_allreduce_mean(T.CUDA, g.ptr, n)
                lib.sl_dist_group(T.CUDA, 0)
                lib.sl_adamw(T.CUDA, p.ptr, g.ptr, m.ptr, v.ptr, n, H["lr"], H["b1"], H["b2"], H["eps"], H["wd"], t[0])

            for _ in range(5):
                step()
            lib.slb_flush()
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                step()
            lib.slb_flush()
            e1.record()
            torch.cuda.synchronize()
            ms = torch.tensor([e0.elapsed_time(e1) / steps], device="cuda")
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            us = float(ms.item()) * 1e3
            rows.append({"bytes": nbytes, "exchange": "one-shot" if mode == 1 else "two-shot", "us_per_step": round(us, 2),
                         "hbm_GBps_per_rank": round(BYTES_PER_PARAM * n / us / 1e3, 1),
                         "nvlink_GBps_per_dir": round(8.0 * n * (world - 1) / world / us / 1e3, 1),
                         "kernel_mode": counter("last_mode"), "blocks": counter("last_blocks")})
        set_option("mode", 0)
        del p, g, m, v
    err = lib.sl_check(T.CUDA)
    if rank == 0:
        print(json.dumps({"metric": "bucket_sweep_fused_allreduce_adamw", "n_gpus": world, "sticky_error": err,
                          "rows": rows}), flush=True)
    distributed.destroy()
    dist.destroy_process_group()


def run_fabric(args):
    """One process, all GPUs: GB/s per GPU that the fabric delivers to copy engines and to kernels, with every link
    carrying data one way and both ways. The slowest GPU's figure is the ceiling a collective can be held against."""
    from soliton_b200._C import lib
    have = lib.sl_cuda_count()
    rows = []
    nbytes = 64 << 20
    for w in (2, 4, 8):
        if w > min(have, args.gpus):
            continue
        for mode, name in ((0, "copy engines"), (1, "kernel, 256-bit loads (pull)"), (2, "kernel, 256-bit stores (push)")):
            for both in (0, 1):
                gbs = (ctypes.c_double * 8)()
                ms = (ctypes.c_double * 8)()
                rc = lib.slb_fabric_probe(w, nbytes, mode, both, 20, gbs, ms)
                active = [round(g, 1) for g in list(gbs)[:w] if g > 0]
                rows.append({"gpus": w, "by": name, "links": "both directions at once" if both else "one direction",
                             "rc": rc, "GBps_per_gpu_min": min(active) if active else None,
                             "GBps_per_gpu_max": max(active) if active else None,
                             "ms": round(max(list(ms)[:w]), 2), "bytes_per_pair": nbytes, "repeats": 20})
    print(json.dumps({"metric": "nvlink_fabric_GBps_per_direction_per_gpu", "gpus_visible": have, "rows": rows}), flush=True)


def run_layernorm(args):
    """Layer normalisation, forward and backward, this library's kernels and the reference's (core/cuda/kernels.cu
    :385-449 from oracle/_ref/) on the same buffers: 65,536 rows of 768 and of 1024 floats (201 / 268 MB per tensor,
    larger than L2), CUDA events, median of 20. GB/s are algorithmic: 8 bytes per element forward (read x, write y),
    12 backward (read dy and x, write dx)."""
    import numpy as np
    import torch
    from soliton_b200 import tensor as T
    from soliton_b200._C import lib
    T._dev(T.CUDA)
    R = reference_gpu_lib()
    C = ctypes
    if R is not None:
        assert R.sl_cuda_set_device(0) == 0
        R.sl_cuda_layernorm.argtypes = [C.c_void_p] * 6 + [C.c_int64, C.c_int64, C.c_float, C.c_void_p]
        R.sl_cuda_layernorm_bwd.argtypes = [C.c_void_p] * 8 + [C.c_int64, C.c_int64] + [C.c_void_p] * 5
    hbm, hbm_kind = hbm_peak()

    def timed(fn, reps=20):
        out = []
        for i in range(reps + 3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= 3:
                out.append(e0.elapsed_time(e1))
        return statistics.median(out)

    rows_out = []
    for rows, c in ((65536, 768), (65536, 1024), (8192, 768)):
        rng = np.random.default_rng(0)
        x = T.tensor(rng.standard_normal((rows, c), dtype=np.float32), "cuda")
        dy = T.tensor(rng.standard_normal((rows, c), dtype=np.float32), "cuda")
        w, b = T.tensor(np.ones(c, np.float32), "cuda"), T.zeros((c,), "cuda")
        y, dx, tmp = T.empty((rows, c), "cuda"), T.empty((rows, c), "cuda"), T.empty((rows, c), "cuda")
        mean, invstd, sg, sgx, ones_r = (T.empty((rows,), "cuda") for _ in range(5))
        dw, db, ones_c = (T.empty((c,), "cuda") for _ in range(3))
        T.synchronize()
        for name, L in (("this library", lib), ("reference", R)):
            if L is None:
                continue
            fwd = lambda: L.sl_cuda_layernorm(x.ptr, w.ptr, b.ptr, y.ptr, mean.ptr, invstd.ptr, rows, c, 1e-5, ones_c.ptr)  # noqa: E731
            bwd = lambda: L.sl_cuda_layernorm_bwd(dy.ptr, x.ptr, w.ptr, mean.ptr, invstd.ptr, dx.ptr, dw.ptr, db.ptr, rows, c,  # noqa: E731
                                                  tmp.ptr, sg.ptr, sgx.ptr, ones_c.ptr, ones_r.ptr)
            tf, tb = timed(fwd), timed(bwd)
            n = rows * c
            rows_out.append({"rows": rows, "c": c, "by": name, "fwd_ms": round(tf, 4), "bwd_ms": round(tb, 4),
                             "fwd_GBps": round(8 * n / tf / 1e6, 1), "bwd_GBps": round(12 * n / tb / 1e6, 1),
                             "fwd_frac_of_hbm": round(8 * n / tf / 1e6 / hbm, 3), "bwd_frac_of_hbm": round(12 * n / tb / 1e6 / hbm, 3)})
        assert lib.sl_check(T.CUDA) == 0
    print(json.dumps({"metric": "layernorm_algorithmic_GBps", "hbm_peak": hbm, "hbm_peak_kind": hbm_kind, "rows": rows_out}), flush=True)


def run_attention(args):
    """Causal attention, forward and backward, this library's fused kernels and the reference's path
    (core/cuda/kernels.cu:536-692 from oracle/_ref/) on the same buffers, in both matmul precisions (fp32, and TF32
    as after sl_set_tf32(1)), at GPT-2's shapes (batch 8, context 1024, head size 64; 12 and 16 heads), CUDA events,
    median of 20. TFLOP/s count the causal half of the products only: forward 2 products, backward 5, each
    2 * T * T / 2 * 64 flops per head."""
    import numpy as np
    import torch
    from soliton_b200 import tensor as T
    from soliton_b200._C import lib
    T._dev(T.CUDA)
    R = reference_gpu_lib()
    C = ctypes
    if R is not None:
        assert R.sl_cuda_set_device(0) == 0
        R.sl_cuda_attention.argtypes = [C.c_void_p] * 3 + [C.c_int64] * 4 + [C.c_float, C.c_int64] + [C.c_void_p] * 8
        R.sl_cuda_attention_bwd.argtypes = [C.c_void_p] * 5 + [C.c_int64] * 4 + [C.c_float, C.c_int64] + [C.c_void_p] * 9
        R.sl_cuda_set_tf32.argtypes = [C.c_int]

    def timed(fn, reps=20):
        out = []
        for i in range(reps + 3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= 3:
                out.append(e0.elapsed_time(e1))
        return statistics.median(out)

    rows_out = []
    hs, tile = 64, 256
    for B, Tn, H in ((8, 1024, 12), (8, 1024, 16), (8, 512, 12)):
        rng = np.random.default_rng(0)
        bh = B * H
        rows = bh * tile
        qkv = T.tensor(rng.standard_normal((B, Tn, 3, H, hs), dtype=np.float32), "cuda")
        dout = T.tensor(rng.standard_normal((B, Tn, H, hs), dtype=np.float32), "cuda")
        out, dqkv, Lb = T.empty((B, Tn, H, hs), "cuda"), T.empty((B, Tn, 3, H, hs), "cuda"), T.empty((bh, Tn), "cuda")
        s, dp = T.empty((rows, tile), "cuda"), T.empty((rows, tile), "cuda")
        acc, oc = T.empty((rows, hs), "cuda"), T.empty((rows, hs), "cuda")
        m, l, c = (T.empty((rows,), "cuda") for _ in range(3))
        rowbuf, ones, ptrs = T.empty((rows, 17), "cuda"), T.empty((tile,), "cuda"), T.empty((18 * bh,), "cuda")
        T.synchronize()
        scale = 0.125
        for tf32, name, Lib in ((1, "this library", lib), (1, "reference", R), (0, "this library", lib), (0, "reference", R)):
            if Lib is None:
                continue
            lib.sl_cuda_attention_set_tf32(tf32)
            if R is not None:
                R.sl_cuda_set_tf32(tf32)
            fwd = lambda: Lib.sl_cuda_attention(qkv.ptr, out.ptr, Lb.ptr, B, Tn, H, hs, scale, tile, s.ptr, acc.ptr, m.ptr, l.ptr,  # noqa: E731
                                                c.ptr, rowbuf.ptr, ones.ptr, ptrs.ptr)
            bwd = lambda: Lib.sl_cuda_attention_bwd(qkv.ptr, out.ptr, Lb.ptr, dout.ptr, dqkv.ptr, B, Tn, H, hs, scale, tile, s.ptr,  # noqa: E731
                                                    dp.ptr, acc.ptr, oc.ptr, m.ptr, l.ptr, rowbuf.ptr, ones.ptr, ptrs.ptr)
            tf, tb = timed(fwd), timed(bwd)
            flop = bh * Tn * Tn * hs  # one causal product: 2 * T * T / 2 * hs per head
            rows_out.append({"B": B, "T": Tn, "H": H, "precision": "tf32" if tf32 else "fp32", "by": name, "fwd_ms": round(tf, 4), "bwd_ms": round(tb, 4),
                             "fwd_causal_TFLOPs": round(2 * flop / tf / 1e9, 1), "bwd_causal_TFLOPs": round(5 * flop / tb / 1e9, 1)})
        assert lib.sl_check(T.CUDA) == 0
    lib.sl_cuda_attention_set_tf32(0)
    if R is not None:
        R.sl_cuda_set_tf32(0)
    print(json.dumps({"metric": "attention_ms", "rows": rows_out}), flush=True)


def run_xent(args):
    """Cross entropy forward (including its blocking read of the mean) and backward, this library's kernels and the
    reference's (core/cuda/kernels.cu:488-534 from oracle/_ref/) on the same buffers: GPT-2's 8,192 rows of 50,257
    logits (1.65 GB, larger than L2), CUDA events, median of 20. GB/s are algorithmic: 4 bytes per logit forward,
    8 backward (read the logits, write the gradient)."""
    import numpy as np
    import torch
    from soliton_b200 import tensor as T
    from soliton_b200._C import lib
    T._dev(T.CUDA)
    R = reference_gpu_lib()
    C = ctypes
    if R is not None:
        assert R.sl_cuda_set_device(0) == 0
        R.sl_cuda_cross_entropy.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
        R.sl_cuda_cross_entropy.restype = C.c_double
        R.sl_cuda_cross_entropy_bwd.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_float]
    hbm, hbm_kind = hbm_peak()

    def timed(fn, reps=20):
        out = []
        for i in range(reps + 3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= 3:
                out.append(e0.elapsed_time(e1))
        return statistics.median(out)

    rows_out = []
    for n, v in ((8192, 50257), (8192, 50304)):
        rng = np.random.default_rng(0)
        logits = T.tensor(rng.standard_normal((n, v), dtype=np.float32), "cuda")
        t = T.tensor(rng.integers(0, v, n).astype(np.int32).view(np.float32), "cuda")
        dl, rowloss = T.empty((n, v), "cuda"), T.empty((n,), "cuda")
        T.synchronize()
        for name, Lib in (("this library", lib), ("reference", R)):
            if Lib is None:
                continue
            loss = []
            fwd = lambda: loss.append(Lib.sl_cuda_cross_entropy(logits.ptr, t.ptr, n, v, rowloss.ptr))  # noqa: E731
            bwd = lambda: Lib.sl_cuda_cross_entropy_bwd(logits.ptr, t.ptr, dl.ptr, n, v, 1.0)  # noqa: E731
            tf, tb = timed(fwd), timed(bwd)
            rows_out.append({"rows": n, "v": v, "by": name, "loss": loss[-1], "fwd_ms": round(tf, 4), "bwd_ms": round(tb, 4),
                             "fwd_GBps": round(4 * n * v / tf / 1e6, 1), "bwd_GBps": round(8 * n * v / tb / 1e6, 1),
                             "fwd_frac_of_hbm": round(4 * n * v / tf / 1e6 / hbm, 3), "bwd_frac_of_hbm": round(8 * n * v / tb / 1e6 / hbm, 3)})
        assert lib.sl_check(T.CUDA) == 0
    print(json.dumps({"metric": "cross_entropy_algorithmic_GBps", "hbm_peak": hbm, "hbm_peak_kind": hbm_kind, "rows": rows_out}), flush=True)


def run_elementwise(args):
    """Binary ops in the two shapes a GPT-2 step uses (residual add, bias add, 8,192 x 3,072 floats) and the
    embedding's backward at GPT-2's sizes (8,192 tokens, 50,257 x 768 table), this library's kernels and the
    reference's (core/cuda/kernels.cu:139-181, 459-487 from oracle/_ref/) on the same buffers, CUDA events, median of
    20; GELU forward and backward on the same 8,192 x 3,072 floats. GB/s are algorithmic: 12 bytes per element for
    the residual add and GELU's backward, 8 for the bias add and GELU; for the embedding the table written once plus
    the rows of dy read once."""
    import numpy as np
    import torch
    from soliton_b200 import tensor as T
    from soliton_b200._C import lib
    T._dev(T.CUDA)
    R = reference_gpu_lib()
    C = ctypes
    if R is not None:
        assert R.sl_cuda_set_device(0) == 0
        R.sl_cuda_binary.argtypes = [C.c_int] + [C.c_void_p] * 3 + [C.c_int] + [C.c_void_p] * 3
        R.sl_cuda_embedding_bwd.argtypes = [C.c_void_p] * 3 + [C.c_int64] * 3 + [C.c_void_p] * 4 + [C.c_size_t]
        R.sl_cuda_gelu.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        R.sl_cuda_gelu_bwd.argtypes = [C.c_void_p] * 3 + [C.c_int64]
    hbm, hbm_kind = hbm_peak()

    def timed(fn, reps=20):
        out = []
        for i in range(reps + 3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= 3:
                out.append(e0.elapsed_time(e1))
        return statistics.median(out)

    longs = lambda v: (C.c_int64 * len(v))(*v)  # noqa: E731
    rows_out = []
    rows, c = 8192, 3072
    rng = np.random.default_rng(0)
    a = T.tensor(rng.standard_normal((rows, c), dtype=np.float32), "cuda")
    b = T.tensor(rng.standard_normal((rows, c), dtype=np.float32), "cuda")
    bias = T.tensor(rng.standard_normal((c,), dtype=np.float32), "cuda")
    o = T.empty((rows, c), "cuda")
    n, vocab, width = 8192, 50257, 768
    dy = T.tensor(rng.standard_normal((n, width), dtype=np.float32), "cuda")
    idx = T.tensor(rng.integers(0, vocab, n).astype(np.int32).view(np.float32), "cuda")
    dw = T.empty((vocab, width), "cuda")
    keys, perm, perm_out = (T.empty((n,), "cuda") for _ in range(3))
    temp_bytes = n * 16 + (1 << 20)
    temp = T.empty((temp_bytes // 4,), "cuda")
    T.synchronize()
    shape, dense, suffix = longs((rows, c)), longs((c, 1)), longs((0, 1))
    for name, Lib in (("this library", lib), ("reference", R)):
        if Lib is None:
            continue
        t_res = timed(lambda: Lib.sl_cuda_binary(0, a.ptr, b.ptr, o.ptr, 2, shape, dense, dense))
        t_bias = timed(lambda: Lib.sl_cuda_binary(0, a.ptr, bias.ptr, o.ptr, 2, shape, dense, suffix))
        t_emb = timed(lambda: Lib.sl_cuda_embedding_bwd(dy.ptr, idx.ptr, dw.ptr, vocab, n, width, keys.ptr, perm.ptr, perm_out.ptr,
                                                        temp.ptr, temp_bytes))
        t_gelu = timed(lambda: Lib.sl_cuda_gelu(a.ptr, o.ptr, rows * c))
        t_gelu_bwd = timed(lambda: Lib.sl_cuda_gelu_bwd(a.ptr, b.ptr, o.ptr, rows * c))
        e = rows * c
        emb_bytes = 4 * (vocab * width + n * width)
        rows_out.append({"by": name, "residual_add_ms": round(t_res, 4), "residual_add_GBps": round(12 * e / t_res / 1e6, 1),
                         "residual_add_frac_of_hbm": round(12 * e / t_res / 1e6 / hbm, 3),
                         "bias_add_ms": round(t_bias, 4), "bias_add_GBps": round(8 * e / t_bias / 1e6, 1),
                         "bias_add_frac_of_hbm": round(8 * e / t_bias / 1e6 / hbm, 3),
                         "gelu_ms": round(t_gelu, 4), "gelu_frac_of_hbm": round(8 * e / t_gelu / 1e6 / hbm, 3),
                         "gelu_bwd_ms": round(t_gelu_bwd, 4), "gelu_bwd_frac_of_hbm": round(12 * e / t_gelu_bwd / 1e6 / hbm, 3),
                         "embedding_bwd_ms": round(t_emb, 4), "embedding_bwd_GBps": round(emb_bytes / t_emb / 1e6, 1),
                         "embedding_bwd_frac_of_hbm": round(emb_bytes / t_emb / 1e6 / hbm, 3)})
    assert lib.sl_check(T.CUDA) == 0
    print(json.dumps({"metric": "elementwise_algorithmic_GBps", "hbm_peak": hbm, "hbm_peak_kind": hbm_kind, "rows": rows_out}), flush=True)


def run_reference_gpu(args, rank, local_rank, world):
    """The reference's own GPU path as an arm of its own (the product arm also carries it as `gpu_baseline`)."""
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    R = reference_gpu_lib()
    if R is None:
        if rank == 0:
            print(json.dumps({"impl": "reference-gpu", "unavailable": "oracle/_ref/ not built (no reference checkout at build time)"}))
        return
    ms, launches = time_reference_gpu(args, R, rank, local_rank, world, dist, args.steps, args.warmup)
    P = total_params(args)
    if rank == 0:
        print(json.dumps({"impl": "reference-gpu", "metric": METRIC,
                          "value": world * BYTES_PER_PARAM * P / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world,
                          "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
                          "config": {"workload": workload_name(args), "params_per_rank": P, "world": world,
                                     "path": "reference core/cuda/kernels.cu: grouped ncclAllReduce(avg) + k_adamw per tensor"},
                          "nccl": nccl_version(), "gpu_launches_per_step": launches}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.fabric:
        return run_fabric(args)
    if args.layernorm:
        return run_layernorm(args)
    if args.attention:
        return run_attention(args)
    if args.xent:
        return run_xent(args)
    if args.elementwise:
        return run_elementwise(args)
    if world == 1 and args.gpus > 1:
        # launched without torchrun: start one process per GPU ourselves
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 2000), os.path.abspath(__file__)]
        sys.exit(subprocess.call(cmd + sys.argv[1:]))
    if args.impl == "reference":
        run_reference(args, rank, world)
    elif args.impl == "reference-gpu":
        run_reference_gpu(args, rank, local_rank, world)
    elif args.sweep:
        run_sweep(args, rank, local_rank, world)
    else:
        run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
