"""Benchmark of the data-parallel optimizer path: gradient mean over ranks + 1/world scaling + AdamW, fused.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--model 124M|medium] [--flat BYTES]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Workload: the GPT-2 124M parameter set (148 tensors, 124,439,808 fp32 parameters; soliton_b200/workload.py),
parameters seeded as the reference's example initialises them, per-rank gradients N(0, 1e-3) seeded by rank,
m = v = 0, lr 3e-4, betas (0.9, 0.999), eps 1e-8, weight decay 0.1 on matrices. A step is one pass of the path over
all tensors through the Soliton-shaped Python interface: distributed.all_reduce_grads(params); optimizer.step().
Inputs (2 GB per rank) are far larger than L2, so nothing is flushed between iterations.

Prints ONE JSON line on rank 0. `value` is GB/s of algorithmic HBM traffic (28 bytes per parameter per rank: read
g, p, m, v; write p, m, v) summed over all ranks, inputs resident in HBM. `e2e` is the same metric with, inside the
timed region of every step, the host->device copy of the step's gradients from pinned memory and the device->host
read of the updated parameters. `--impl reference` times the reference's host path (CPU restatement of
core/soliton/cpu.d: axpy per rank, scale, adamw; the D core cannot be built here) on the host cores.
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

BYTES_PER_PARAM = 28            # algorithmic HBM bytes per parameter per rank
NVLINK_GBS = 770.0              # measured peer copy bandwidth per direction on this pool (nominal 900)
FALLBACK_HBM_GBS = 6650.0       # used only when MEASURED_PEAKS.json is absent
# DRAM bytes per parameter of the dominant kernel from an ncu capture (profiles/), per world size; None = not captured
NCU_DRAM_BYTES_PER_PARAM = {1: 27.22}  # profiles/k_twoshot_w1_flat256MiB_ncu.md


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"])
    ap.add_argument("--model", default="124M", choices=["124M", "medium", "tiny"])
    ap.add_argument("--flat", type=int, default=0, help="one flat buffer of this many bytes instead of a model")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--mode", type=int, default=0, help="0 auto, 1 one-shot, 2 two-shot")
    ap.add_argument("--blocks-per-sm", type=int, default=0)
    ap.add_argument("--cyclic", type=int, default=-1)
    ap.add_argument("--sweep", action="store_true", help="bucket-size sweep 4 KB .. 1 GB, one-shot vs two-shot (N >= 2)")
    ap.add_argument("--bare", action="store_true", help="gradient mean only, no optimizer update (link-bound floor)")
    ap.add_argument("--pipeline", type=int, default=-1, help="-1 auto, 1 k_step (shared-memory ring), 0 k_twoshot")
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


def make_workload(args):
    """[(name, shape)] and per-rank host arrays (params identical on all ranks, gradients seeded by rank)."""
    import numpy as np
    from soliton_b200 import workload
    if args.flat:
        n = args.flat // 4
        shapes = [("flat", (n,))]
        make_p = lambda: [workload.flat_case(n)[0]]                                  # noqa: E731
        make_g = lambda rank: [workload.flat_case(n, rank=rank)[1]]                  # noqa: E731
        wds = [workload.HYPER["wd"]]
        name = f"flat fp32 buffer, {args.flat} bytes"
    else:
        ps = workload.param_shapes(args.model)
        shapes = [(nm, s) for nm, s, _ in ps]
        make_p = lambda: workload.init_params(args.model, seed=0)                    # noqa: E731
        make_g = lambda rank: workload.rank_grads(args.model, rank=rank)             # noqa: E731
        wds = [workload.HYPER["wd"] if len(s) >= 2 else 0.0 for _, s in shapes]
        name = f"GPT-2 {args.model} parameter set, {len(shapes)} tensors"
    return shapes, make_p, make_g, wds, name, np


def run_reference(args, rank, world):
    """The reference's host path (restated; core/soliton/cpu.d:85-101,362-373) on the host cores: every one of
    `world` threads, standing for one rank's process, sums the ranks' gradients, scales and runs AdamW."""
    if rank != 0:
        return
    import numpy as np
    from oracle import pyoracle
    from soliton_b200 import workload
    total = args.flat // 4 if args.flat else workload.total_params(args.model)
    n = min(total, 4 << 20)  # bounded sample of the workload: its first 4 Mi parameters
    p0 = np.random.default_rng(0).standard_normal(n, dtype=np.float32) * np.float32(0.02)
    grads = [np.random.default_rng(1 + r).standard_normal(n, dtype=np.float32) * np.float32(1e-3) for r in range(world)]
    cores = min(world, os.cpu_count() or 1)
    pyoracle.bench(p0, grads, max(args.warmup, 1), cores)
    t = pyoracle.bench(p0, grads, args.steps, cores)
    ms = 1e3 * t / args.steps
    value = cores * BYTES_PER_PARAM * n / (t / args.steps) / 1e9
    name = f"flat fp32 buffer, {args.flat} bytes" if args.flat else f"GPT-2 {args.model} parameter set"
    line = {
        "impl": "reference", "metric": "fused_allreduce_adamw_algorithmic_GBps", "value": value, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "params_per_rank": total, "world": world},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": f"first {n} parameters per step, {args.steps} steps, one thread per rank "
                                   f"(the reference's host kernels are single-threaded loops)"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def cpu_baseline(world):
    """Rank 0, N = 1: the host path on one core over a bounded sample, about ten seconds of CPU work."""
    import numpy as np
    from oracle import pyoracle
    n = 4 << 20
    p0 = np.random.default_rng(0).standard_normal(n, dtype=np.float32) * np.float32(0.02)
    grads = [np.random.default_rng(1 + r).standard_normal(n, dtype=np.float32) * np.float32(1e-3) for r in range(world)]
    t1 = pyoracle.bench(p0, grads, 2, 1)
    reps = max(3, min(400, int(10.0 / max(t1 / 2, 1e-4))))
    t = pyoracle.bench(p0, grads, reps, 1)
    return {"value": BYTES_PER_PARAM * n * reps / t / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
            "sample": f"first {n} parameters, {reps} steps, single thread as in core/soliton/cpu.d",
            "host_cores_available": os.cpu_count()}


def run_ours(args, rank, local_rank, world):
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    from soliton_b200 import distributed, tensor as T
    from soliton_b200._C import counter, lib, set_option
    from soliton_b200.optim import AdamW
    from soliton_b200 import workload
    shapes, make_p, make_g, wds, name, np = make_workload(args)
    H = workload.HYPER

    T.set_device(local_rank)
    T._dev(T.CUDA)
    if args.mode:
        set_option("mode", args.mode)
    if args.blocks_per_sm:
        set_option("blocks_per_sm", args.blocks_per_sm)
    if args.pipeline >= 0:
        set_option("pipeline", args.pipeline)
    if args.cyclic >= 0:
        set_option("cyclic", args.cyclic)
    if world > 1:
        idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            idt.copy_(torch.frombuffer(bytearray(distributed.unique_id()), dtype=torch.uint8))
        dist.broadcast(idt, 0)
        distributed.init_with_id(rank, world, bytes(idt.cpu().numpy().tobytes()))

    # device state through the library's allocator; host copies of the gradients in pinned memory for the e2e leg
    host_p = make_p()
    host_g = make_g(rank)
    P = sum(int(a.size) for a in host_p)
    params = [T.tensor(a, "cuda") for a in host_p]
    pinned_g = [torch.empty(a.size, dtype=torch.float32).pin_memory() for a in host_g]
    for t, a in zip(pinned_g, host_g):
        t.numpy()[:] = a.ravel()
    pinned_out = [torch.empty(a.size, dtype=torch.float32).pin_memory() for a in host_p]
    for p, a in zip(params, host_g):
        p.grad = T.tensor(a, "cuda")
    del host_p, host_g

    class Opt(AdamW):  # weight decay per tensor as the workload defines it (flat buffers decay although 1-D)
        def step(self):
            self.t += 1
            b1, b2 = self.betas
            for (p, (m, v)), wd in zip(zip(self.params, self.state), wds):
                lib.sl_adamw(p.dev, p.ptr, p.grad.ptr, m.ptr, v.ptr, p.numel, self.lr, b1, b2, self.eps, wd, self.t)

    opt = Opt(params, lr=H["lr"], betas=(H["b1"], H["b2"]), eps=H["eps"], weight_decay=H["wd"])

    def step():
        distributed.all_reduce_grads(opt.params)
        if args.bare:
            lib.slb_flush()
        else:
            opt.step()

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
    total_ms = timed(args.steps, step)
    launches = counter("launches") - launches0
    clocks = sampler.stop() if rank == 0 else None
    err = lib.sl_check(T.CUDA)
    if err:
        raise RuntimeError(f"soliton_b200: sticky error {err} after the timed region")
    mode, blocks = counter("last_mode"), counter("last_blocks")

    def e2e_step():
        for p, src in zip(params, pinned_g):
            lib.sl_from_host(T.CUDA, p.grad.ptr, src.data_ptr(), p.numel * 4)
        step()
        for p, dst in zip(params, pinned_out):
            lib.sl_to_host(T.CUDA, dst.data_ptr(), p.ptr, p.numel * 4)

    e2e_step()
    e2e_ms = timed(args.e2e_steps, e2e_step)

    if rank != 0:
        if world > 1:
            distributed.destroy()
            dist.destroy_process_group()
        return
    ms = total_ms / args.steps
    value = world * BYTES_PER_PARAM * P / (ms * 1e-3) / 1e9
    e2e_value = world * BYTES_PER_PARAM * P / (e2e_ms / args.e2e_steps * 1e-3) / 1e9
    hbm, hbm_kind = hbm_peak()
    hbm_per_rank = BYTES_PER_PARAM * P / (ms * 1e-3) / 1e9
    t_hbm = BYTES_PER_PARAM * P / (hbm * 1e9)
    nvl_bytes = 8.0 * P * (world - 1) / world
    t_nvl = nvl_bytes / (NVLINK_GBS * 1e9)
    per_launch_ms = total_ms / max(launches, 1)
    use_step = args.pipeline == 1
    base = "k_step" if use_step else "k_twoshot"
    kernel = {0: f"{base}<1,adam>", 1: f"k_oneshot<{world},adam>", 2: f"{base}<{world},adam>"}[mode]
    traffic = NCU_DRAM_BYTES_PER_PARAM.get(world)
    if t_hbm >= t_nvl:
        roof = {"bound": "hbm", "achieved": hbm_per_rank, "peak": hbm, "unit": "GB/s", "frac": hbm_per_rank / hbm,
                "traffic": traffic * P if traffic else None}
    else:
        nvl = nvl_bytes / (ms * 1e-3) / 1e9
        roof = {"bound": "nvlink", "achieved": nvl, "peak": NVLINK_GBS, "unit": "GB/s", "frac": nvl / NVLINK_GBS,
                "traffic": traffic * P if traffic else None, "hbm_achieved": hbm_per_rank, "hbm_peak": hbm,
                "hbm_frac": hbm_per_rank / hbm}
    roof.update({"kernel": kernel, "peak_source": f"{hbm_kind} HBM copy; NVLink 770 GB/s measured peer copy",
                 "ms_per_launch": per_launch_ms, "roofline_ms": 1e3 * max(t_hbm, t_nvl),
                 "frac_of_roofline_time": max(t_hbm, t_nvl) / (ms * 1e-3)})
    line = {
        "metric": "fused_allreduce_adamw_algorithmic_GBps", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "params_per_rank": P, "world": world, "l2": "inputs larger than L2, no flush",
                   "exchange": {0: "none", 1: "one-shot", 2: "two-shot"}[mode], "blocks_per_rank": blocks,
                   "optimizer": "none (--bare)" if args.bare else "AdamW",
                   "arithmetic": "gradient mean, m, v in f32; parameter update in f64, rounded to f32 once",
                   "e2e_copies": "h2d: this step's gradients from pinned memory; d2h: updated parameters"},
        "roofline": roof,
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": 4 * P, "d2h_bytes_per_step": 4 * P,
                "ms_per_step": e2e_ms / args.e2e_steps, "steps": args.e2e_steps},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(1)
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


def run_reference_gpu(args, rank, local_rank, world):
    """The reference's own GPU path on this box: grouped ncclAllReduce(avg) per tensor, then one k_adamw launch per
    tensor (core/cuda/kernels.cu:242-254,772-775), from the unmodified backend built into oracle/_ref/."""
    import ctypes as C
    import torch
    import torch.distributed as dist
    from oracle import build as obuild
    if not os.path.exists(obuild.REF_SO):
        if rank == 0:
            print(json.dumps({"impl": "reference-gpu", "unavailable": "oracle/_ref/ not built (no reference checkout at build time)"}))
        return
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("gloo")
    R = C.CDLL(obuild.REF_SO)
    assert R.sl_cuda_set_device(local_rank) == 0
    R.sl_cuda_malloc.restype = C.c_void_p
    R.sl_cuda_malloc.argtypes = [C.c_size_t]
    R.sl_cuda_h2d.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
    R.sl_cuda_adamw.argtypes = [C.c_void_p] * 4 + [C.c_int64] + [C.c_float] * 5 + [C.c_int]
    R.sl_cuda_nccl_allreduce_mean.argtypes = [C.c_void_p, C.c_int64]
    R.sl_cuda_fill.argtypes = [C.c_void_p, C.c_int64, C.c_float]
    if world > 1:
        idt = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            buf = C.create_string_buffer(128)
            assert R.sl_cuda_nccl_unique_id(buf) == 0
            idt = torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8).clone()
        dist.broadcast(idt, 0)
        assert R.sl_cuda_nccl_init(rank, world, C.create_string_buffer(bytes(idt.numpy().tobytes()), 128)) == 0
    shapes, make_p, make_g, wds, name, np = make_workload(args)
    from soliton_b200 import workload
    H = workload.HYPER
    bufs = []
    for a, gr in zip(make_p(), make_g(rank)):
        n = int(a.size)
        ptrs = [R.sl_cuda_malloc(4 * n) for _ in range(4)]
        R.sl_cuda_h2d(ptrs[0], np.ascontiguousarray(a).ctypes.data, 4 * n)
        R.sl_cuda_h2d(ptrs[1], np.ascontiguousarray(gr).ctypes.data, 4 * n)
        R.sl_cuda_fill(ptrs[2], n, 0.0)
        R.sl_cuda_fill(ptrs[3], n, 0.0)
        bufs.append((ptrs, n))
    P = sum(n for _, n in bufs)
    t = [0]

    def step():
        t[0] += 1
        if world > 1:
            R.sl_cuda_nccl_group(1)
            for ptrs, n in bufs:
                R.sl_cuda_nccl_allreduce_mean(ptrs[1], n)
            R.sl_cuda_nccl_group(0)
        for (ptrs, n), wd in zip(bufs, wds):
            R.sl_cuda_adamw(ptrs[0], ptrs[1], ptrs[2], ptrs[3], n, H["lr"], H["b1"], H["b2"], H["eps"], wd, t[0])

    for _ in range(max(args.warmup, 3)):
        step()
    R.sl_cuda_sync()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    R.sl_cuda_sync()
    ms = torch.tensor([e0.elapsed_time(e1) / args.steps])
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    assert R.sl_cuda_check() == 0
    if rank == 0:
        m = float(ms.item())
        print(json.dumps({"impl": "reference-gpu", "metric": "fused_allreduce_adamw_algorithmic_GBps",
                          "value": world * BYTES_PER_PARAM * P / (m * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world,
                          "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": m, "higher_is_better": True,
                          "config": {"workload": name, "params_per_rank": P, "world": world,
                                     "path": "reference core/cuda/kernels.cu: grouped ncclAllReduce(avg) + k_adamw per tensor"},
                          "gpu_launches_per_step": len(bufs) + (1 if world > 1 else 0)}), flush=True)
    if world > 1:
        R.sl_cuda_nccl_destroy()
        dist.destroy_process_group()


def main():
    args = parse()
    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
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
