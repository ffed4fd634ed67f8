#!/usr/bin/env python
"""Benchmark of the raised-contraction hot path (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl pgb200|reference]
                    [--workload NAME] [--kernel-only] [--no-per-config]

Default workload: BASELINE.json configs[4]b, the largest configuration that
fits one GPU - fp32 GEMM C = alpha*A*B + beta*C, M=N=K=32768, inputs uniform
[0,1) from a seed, alpha=1.5, beta=1.2, on the 3xTF32 tensor path.  With N>1
ranks (torchrun) the rows of A and C are partitioned across the ranks (strong
scaling: total work fixed) and the shared operand B is broadcast from rank 0
inside every step, in K-slices, so that the transfer overlaps the product: by
the copy engines over peer-mapped memory (no SMs; `broadcast` in the line says
which route ran), else by NCCL.

`value`   device-resident throughput, CUDA events on the launching stream.
`e2e`     same metric through the reference-facing drop-in (pgb200_kernel_gemm
          on host arrays), H2D and D2H copies inside the timed region: the
          headline figure uses pageable host arrays (what the PolyBench nests
          get from posix_memalign, utilities/polybench.c:519-525); the same
          call on page-locked arrays and on arrays registered with pgb200Pin
          (device-resident across repeated calls) are reported beside it.
`roofline` dominant kernel: algorithmic flop (or bytes) per launch / CUDA-event
          time, against a measured peak (MEASURED_PEAKS.json for HBM; this
          library's own issue-rate probes for the fp64 and TF32 tensor rates).
`per_config` the other BASELINE configs ([0], [1], [2], [3], [4]a), measured in
          the same process after the headline (1 GPU runs only): value,
          roofline and clocks each.
`cpu_baseline` the reference's compiled loop nest on the host cores, a bounded
          sample: all cores and one core, each 5 runs with the fastest and the
          slowest dropped (utilities/time_benchmark.sh:27-32).
`--impl reference` times the reference's own compiled kernel (oracle/_ref) on
the host cores, on the same workload and config.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEED = 20261125
ALPHA, BETA = 1.5, 1.2
DEFAULT_WORKLOAD = "sgemm32768"
# The other BASELINE configs, measured after the headline on a 1-GPU run.
PER_CONFIG = [("configs[0]", "sgemm1024"), ("configs[1]", "dgemm4096"), ("configs[2]", "mvt32768"),
              ("configs[3]", "chain2mm"), ("configs[4]a", "ssyrk16384"), ("configs[4]b", "sgemm32768")]

# DRAM bytes (read + write) per launch of the dominant kernel from the ncu
# captures summarised under profiles/ (mvt32768: the N=16384 capture x 4;
# sgemm32768: the 16384^3 capture, 45.07 GB, x 8 - with the producers meeting
# between rounds of tiles the traffic is rounds x panels x panel bytes, i.e.
# proportional to tiles x K: 8192^3 5.94 GB, 16384^3 45.07 GB.  One-GPU launch
# only; the row-block launches of a multi-GPU run were not captured).
TRAFFIC = {"dgemm4096": 1.1345e9, "mvt16384": 2.156e9, "mvt32768": 8.624e9, "sgemm4096": 8.31e8,
           "sgemm8192": 5.94e9, "sgemm32768": 3.606e11}

WORKLOADS = {
    "dgemm4096": dict(dtype="f64", M=4096, N=4096, K=4096, lo=-1.0, hi=1.0,
                      desc="configs[1]: fp64 GEMM 4096^3, uniform [-1,1), alpha=1.5 beta=1.2"),
    "sgemm1024": dict(dtype="f32", M=1024, N=1024, K=1024, lo=0.0, hi=1.0,
                      desc="configs[0]: fp32 GEMM 1024^3, uniform [0,1), alpha=1.5 beta=1.2"),
    "sgemm4096": dict(dtype="f32", M=4096, N=4096, K=4096, lo=0.0, hi=1.0,
                      desc="fp32 GEMM 4096^3 (3xTF32), uniform [0,1); profiling-size case"),
    "sgemm8192": dict(dtype="f32", M=8192, N=8192, K=8192, lo=0.0, hi=1.0,
                      desc="fp32 GEMM 8192^3 (3xTF32), uniform [0,1)"),
    "sgemm32768": dict(dtype="f32", M=32768, N=32768, K=32768, lo=0.0, hi=1.0, strong=True,
                       desc="configs[4]b: fp32 GEMM 32768^3 (3xTF32), uniform [0,1), alpha=1.5 beta=1.2; "
                            "rows partitioned across the GPUs, B broadcast from rank 0 in every step"),
    "ssyrk16384": dict(dtype="f32", N=16384, K=8192, lo=0.0, hi=1.0, strong=True,
                       desc="configs[4]a: fp32 SYRK N=16384 K=8192 lower (3xTF32), uniform [0,1), rows "
                            "partitioned by equal triangular area, A broadcast from rank 0 in every step"),
    "mvt16384": dict(dtype="f64", N=16384, lo=0.0, hi=1.0,
                     desc="fp64 mat-vec pair, N=16384 (2.1 GB; the profiling-size case of configs[2])"),
    "mvt32768": dict(dtype="f64", N=32768, lo=0.0, hi=1.0,
                     desc="configs[2]: fp64 mat-vec pair x1+=A*y1, x2+=A^T*y2, N=32768, fused single pass"),
    "chain2mm": dict(dtype="f64", ni=4096, nk=6144, nj=5120, nl=8192, lo=-1.0, hi=1.0,
                     desc="configs[3]: fp64 chained GEMM tmp=alpha*A*B; D=tmp*C+beta*D"),
}

L2_BYTES = 128 << 20


# ----------------------------------------------------------------------------- clocks
class NvmlSampler:
    """SM clock and throttle reasons polled from NVML (what nvidia-smi reads)
    every few milliseconds on a thread, during the timed region only."""

    def __init__(self, index, period_s=0.004):
        import threading
        self.index, self.period = index, period_s
        self.sm, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self.ok = False
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if vis:
                ids = [v for v in vis.split(",") if v != ""]
                if index < len(ids) and ids[index].isdigit():
                    phys = int(ids[index])
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.ok = False

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        while not self._stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for n, bit in names.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self.ok:
            self._thread.start()

    def stop(self):
        if not self.ok:
            return None
        self._stop.set()
        self._thread.join(timeout=2)
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None,
                "sm_max_mhz": self.max_mhz, "samples": len(self.sm),
                "reasons": sorted(self.reasons), "source": "nvml"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples (fallback when NVML's Python
    binding is unusable)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms",
                 "100", "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


def start_sampler(local):
    if os.environ.get("PGB_BENCH_NO_CLOCKS"):
        return None
    s = NvmlSampler(local)
    if not s.ok:
        s = ClockSampler(local)
    s.start()
    return s


# ----------------------------------------------------------------------------- workload arithmetic
def operand_bytes(name, w):
    """Bytes of the arrays one step reads and writes on one GPU."""
    esz = 8 if w["dtype"] == "f64" else 4
    if name.startswith("mvt"):
        return w["N"] * w["N"] * esz
    if name == "chain2mm":
        return esz * (w["ni"] * w["nk"] + w["nk"] * w["nj"] + w["nj"] * w["nl"] + 2 * w["ni"] * w["nl"])
    if name.startswith("ssyrk"):
        return esz * (w["N"] * w["K"] + w["N"] * w["N"])
    return esz * (w["M"] * w["K"] + w["K"] * w["N"] + w["M"] * w["N"])


def algorithmic_work(name, w):
    """Units per step for `value`: flop for contractions, bytes for mat-vec."""
    if name.startswith("mvt"):
        n = w["N"]
        return n * n * 8 + 6 * n * 8
    if name == "chain2mm":
        return 2 * w["ni"] * w["nj"] * w["nk"] + 2 * w["ni"] * w["nl"] * w["nj"]
    if name.startswith("ssyrk"):
        return w["N"] * (w["N"] + 1) * w["K"]
    return 2 * w["M"] * w["N"] * w["K"]


def metric_of(name):
    if name.startswith("mvt"):
        return "HBM GB/s of the raised mat-vec pair", "GB/s", 1e9
    return "GFLOP/s per raised op", "GFLOP/s", 1e9


def l2_note(name, w):
    if operand_bytes(name, w) < 2 * L2_BYTES:
        return "L2 flushed (256 MiB write) before every step; steps timed one by one"
    return "operands exceed the 126 MB L2; no flush between steps"


def config_of(name, w, world):
    """The `config` object of the JSON line; both arms print the same one."""
    return {"workload": w["desc"], "l2": l2_note(name, w),
            "parallelism": ("single GPU" if world == 1 else
                            f"{world} row blocks, shared operand broadcast from rank 0 each step")}


def measured_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        return {}


# ----------------------------------------------------------------------------- CPU legs
def trimmed(times):
    """5 runs, the fastest and the slowest dropped, mean of the other three,
    and the largest deviation of those three from their mean in percent - the
    protocol of the reference's utilities/time_benchmark.sh:27-32."""
    mid = sorted(times)[1:-1] if len(times) >= 3 else sorted(times)
    mean = sum(mid) / len(mid)
    dev = max(abs(t - mean) for t in mid) / mean * 100.0
    return mean, dev


def cpu_sample(w, name, threads, host_b=None):
    """A bounded sample of the workload for `threads` host threads.  Returns
    (units_per_step, step_fn, threads_used, description, kind).

    The kernels are the reference's own compiled kernel_* functions
    (oracle/_ref, kind "reference") when present, else this repository's C
    restatement (kind "port").  The loop nests are sequential; with several
    threads every thread runs the unmodified kernel on its own contiguous block
    of rows, which is what `#pragma omp parallel for` (static schedule) on the
    outer i loop does (gemm, 2mm: rows are independent), or on its own problem
    instance (syrk: the j<=i bound ties a block to its absolute rows)."""
    import concurrent.futures as cf

    import numpy as np

    from oracle import pbo, ref
    have_ref = ref.available()
    kind = "reference" if have_ref else "port"
    np_dt = np.float64 if w["dtype"] == "f64" else np.float32
    lo, hi = w["lo"], w["hi"]
    if name.startswith("mvt"):
        n = 4096
        A = pbo.fill(n, n, np_dt, SEED, 1, lo, hi)
        v = [pbo.fill_vec(n, np_dt, SEED, 2 + k, lo, hi) for k in range(4)]

        def step():
            if have_ref:
                ref.kernel_mvt(n, v[0], v[1], v[2], v[3], A)
            else:
                pbo.mvt(v[0], v[1], v[2], v[3], A)
        return n * n * 8 + 6 * n * 8, step, 1, f"kernel_mvt at N={n}, one thread (sequential nests)", kind
    pool = cf.ThreadPoolExecutor(max_workers=threads)
    if name.startswith("ssyrk"):
        n, m = 512, w["K"]
        As = [pbo.fill(n, m, np_dt, SEED, 1, lo, hi, row0=t * n) for t in range(threads)]
        Cs = [pbo.fill(n, n, np_dt, SEED, 3, lo, hi, row0=t * n) for t in range(threads)]

        def one(t):
            if have_ref:
                ref.kernel_syrk(n, m, ALPHA, BETA, Cs[t], As[t])
            else:
                pbo.syrk(ALPHA, BETA, Cs[t], As[t])

        def step():
            list(pool.map(one, range(threads)))
        return (threads * n * (n + 1) * m, step, threads,
                f"{threads} independent kernel_syrk instances of n={n}, m={m}, one thread each", kind)
    if name == "chain2mm":
        K, N = w["nk"], w["nj"]
    else:
        K, N = w["K"], w["N"]
    rows_per = 2 if name == "sgemm32768" else 16
    B = host_b if host_b is not None else pbo.fill(K, N, np_dt, SEED, 2, lo, hi)
    As = [pbo.fill(rows_per, K, np_dt, SEED, 1, lo, hi, row0=t * rows_per) for t in range(threads)]
    Cs = [pbo.fill(rows_per, N, np_dt, SEED, 3, lo, hi, row0=t * rows_per) for t in range(threads)]

    def one(t):
        if have_ref:
            ref.kernel_gemm(rows_per, N, K, ALPHA, BETA, Cs[t], As[t], B)
        else:
            pbo.gemm(ALPHA, BETA, Cs[t], As[t], B)

    def step():
        list(pool.map(one, range(threads)))
    return (2 * rows_per * threads * N * K, step, threads,
            f"kernel_gemm on {threads} block(s) of {rows_per} rows of the {K}x{N} problem, one "
            f"thread per block (the i loop split statically across threads)", kind)


def run_reference(args, w, name):
    """`--impl reference`: the reference's CPU implementation of the path on
    all host cores; each step is the bounded sample of cpu_sample()."""
    cores = os.cpu_count() or 1
    units, step, used, sample, kind = cpu_sample(w, name, cores)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    metric, unit, scale = metric_of(name)
    val = units / dt / scale
    print(json.dumps({
        "impl": "reference", "metric": metric, "value": val, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong" if w.get("strong") else "weak",
        "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": config_of(name, w, args.gpus),
        "cpu_baseline": {"value": val, "unit": unit, "cores": used, "kind": kind,
                         "sample": sample},
        "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def cpu_baseline(w, name, host_b=None):
    """The same sample beside the GPU number: all host cores, and one core (the
    nest as the reference's own test times it, one thread), each run 5 times
    after a warm-up with the fastest and slowest dropped."""
    _, unit, scale = metric_of(name)
    out = None
    for threads in (os.cpu_count() or 1, 1):
        units, step, used, sample, kind = cpu_sample(w, name, threads, host_b)
        step()
        times = []
        for _ in range(5):
            t0 = time.perf_counter()
            step()
            times.append(time.perf_counter() - t0)
        mean, dev = trimmed(times)
        rec = {"value": units / mean / scale, "unit": unit, "cores": used, "kind": kind,
               "sample": sample,
               "protocol": "5 runs, fastest and slowest dropped, mean of 3 "
                           "(utilities/time_benchmark.sh:27-32)",
               "max_deviation_pct": dev}
        if out is None:
            out = rec
            if used == 1:       # a sequential sample (mvt): one figure is all there is
                break
        else:
            out["one_core"] = rec
    return out


class _OneRank:
    """Stand-in for torch.distributed when there is a single rank."""

    @staticmethod
    def get_world_size(group=None):
        return 1

    @staticmethod
    def get_rank(group=None):
        return 0


# ----------------------------------------------------------------------------- pgb200 arm
class Bench:
    """Shared state of one process of the GPU arm."""

    def __init__(self):
        import torch
        import torch.distributed as dist

        import polygeist_b200 as pgb
        from polygeist_b200 import partition, polybench
        self.torch, self.dist, self.pgb = torch, dist, pgb
        self.partition, self.polybench = partition, polybench
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py: no CUDA device; libpgb200 has no CPU fallback")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.flush = None
        self.broadcast = None        # route of the shared operand in a multi-GPU strong run
        self.broadcast_note = None   # why the copy-engine route was not taken, if so
        self.peaks = measured_peaks()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def tdt(self, w):
        return self.torch.float64 if w["dtype"] == "f64" else self.torch.float32

    def peer_broadcast(self, w, K, N):
        """The shared operand in symmetric memory (every rank's copy mapped into
        every process) and a PeerPullBroadcast over it, or None when that cannot
        be set up here (the step then uses the NCCL broadcast).  All ranks take
        the same branch: the outcome is agreed on with an all-reduce."""
        torch, dist, partition = self.torch, self.dist, self.partition
        self.broadcast_note = None
        if os.environ.get("PGB_BENCH_BCAST", "peer") == "nccl":
            return None
        peer, err = None, None
        try:
            import torch.distributed._symmetric_memory as symm_mem
            dt = self.tdt(w)
            buf = symm_mem.empty((K, N), dtype=dt, device=self.dev)
            hb = symm_mem.rendezvous(buf, dist.group.WORLD)
            views = [hb.get_buffer(r, (K, N), dt) for r in range(self.world)]
            flags, memops, fl, hf = None, None, None, None
            if self.world > 2:
                slots = 64
                fl = symm_mem.empty((self.world, slots), dtype=torch.int32, device=self.dev)
                fl.zero_()
                hf = symm_mem.rendezvous(fl, dist.group.WORLD)
                flags = [hf.get_buffer(r, (self.world, slots), torch.int32) for r in range(self.world)]
                memops = partition.stream_memops()
            peer = partition.PeerPullBroadcast(torch, dist, views, src=0, flags=flags, memops=memops)
            self._symm = (buf, hb, fl, hf)   # the allocations must outlive the mapped views
        except Exception as e:          # noqa: BLE001 - any failure means "use NCCL"
            err = repr(e)
        ok = torch.tensor([0 if peer is None else 1], dtype=torch.int32, device=self.dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        torch.cuda.synchronize()
        if int(ok.item()) == 0:
            self.broadcast_note = err or "a peer could not map the operand"
            return None
        return peer

    def check_broadcast(self, plan, A, B, Cm):
        """One untimed step on poisoned receive buffers: afterwards every rank's
        copy of the shared operand must equal the source's bit for bit (sum of
        the words as integers, compared across ranks); C is restored.  Returns
        whether that held on every rank."""
        torch, dist = self.torch, self.dist
        keep = Cm.clone()
        if self.rank != 0:
            B.fill_(float("nan"))
        self.barrier()
        plan.run(ALPHA, A, B, BETA, Cm)
        torch.cuda.synchronize()
        words = B.view(torch.int32)
        sums = torch.stack([words[i::8].sum(dtype=torch.int64) for i in range(8)])
        lo, hi = sums.clone(), sums.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        same = bool(torch.equal(lo, hi))
        Cm.copy_(keep)
        self.barrier()
        return same

    def filled(self, w, rows, cols, aid, row0=0):
        t = self.torch.empty((rows, cols), dtype=self.tdt(w), device=self.dev)
        self.pgb.fill_uniform(t, SEED, aid, w["lo"], w["hi"], row0=row0)
        return t

    # ---- operands resident in HBM, and the step that runs on them ----
    def build(self, name, w):
        """Returns (step, operands) for this rank; `operands` keeps the tensors
        alive and hands A, B, C to the end-to-end leg of the GEMM workloads."""
        torch, dist, pgb, partition = self.torch, self.dist, self.pgb, self.partition
        rank, world = self.rank, self.world
        ops = {}
        if name.startswith("mvt"):
            n = w["N"]
            A = self.filled(w, n, n, 1)
            vec = [self.filled(w, 1, n, 2 + k).reshape(n) for k in range(4)]
            ops.update(A=A, vec=vec)

            def step():
                pgb.mvt(A, vec[2], vec[3], vec[0], vec[1])
        elif name == "chain2mm":
            A = self.filled(w, w["ni"], w["nk"], 1)
            B = self.filled(w, w["nk"], w["nj"], 2)
            Cc = self.filled(w, w["nj"], w["nl"], 3)
            D = self.filled(w, w["ni"], w["nl"], 4)
            tmp = torch.empty((w["ni"], w["nj"]), dtype=self.tdt(w), device=self.dev)
            ops.update(A=A, B=B, Cc=Cc, D=D, tmp=tmp)

            def step():
                pgb.gemm(ALPHA, A, B, 0.0, tmp)
                pgb.gemm(1.0, tmp, Cc, BETA, D)
        elif name.startswith("ssyrk"):
            n, K = w["N"], w["K"]
            sp = partition.PartitionedSyrk(
                dist if world > 1 else _OneRank(), lambda al, Ar, be, Cb, rows: pgb.syrk_rows(
                    al, Ar, be, Cb, rows[0], rows[1]), src=0,
                kchunk=int(os.environ.get("PGB_BENCH_KCHUNK", 2048)))
            b = sp.blocks(n)
            r0, r1 = b[rank], b[rank + 1]
            A = self.filled(w, n, K, 1) if rank == 0 else torch.empty((n, K), dtype=self.tdt(w),
                                                                      device=self.dev)
            Cm = self.filled(w, r1 - r0, n, 3, row0=r0)
            ops.update(A=A, C=Cm)

            def step():
                sp.run(ALPHA, A, BETA, Cm)
        else:
            M, N, K = w["M"], w["N"], w["K"]
            strong = bool(w.get("strong"))
            if strong:
                b = partition.row_blocks(M, world)
                r0, r1 = b[rank], b[rank + 1]
            else:                       # weak scaling: every rank owns a full-height block
                r0, r1 = rank * M, (rank + 1) * M
            A = self.filled(w, r1 - r0, K, 1, row0=r0)
            Cm = self.filled(w, r1 - r0, N, 3, row0=r0)
            peer = self.peer_broadcast(w, K, N) if (world > 1 and strong) else None
            if peer is not None:
                B = peer.views[rank]
                if rank == 0:
                    pgb.fill_uniform(B, SEED, 2, w["lo"], w["hi"])
            else:
                B = self.filled(w, K, N, 2) if rank == 0 else torch.empty(
                    (K, N), dtype=self.tdt(w), device=self.dev)
            ops.update(A=A, B=B, C=Cm)
            if world > 1:
                # Large shared operand: K-chunks that overlap the chunk products.
                # Small one (128 MiB against 4 ms of compute): a single broadcast.
                # (measured at 8 GPUs, 32768^3: 46.6 ms with K/8 slices, 44.4 ms with
                # K/16 - the first, exposed slice is half as long.)
                dflt = K // 16 if strong else K
                plan = partition.PartitionedGemm(
                    dist, pgb.gemm, src=0, chunk=int(os.environ.get("PGB_BENCH_KCHUNK", dflt)),
                    first_chunk=int(os.environ.get("PGB_BENCH_KFIRST", 0)),
                    grow=os.environ.get("PGB_BENCH_KGROW", "1") != "0", peer_broadcast=peer)
                self.broadcast = ("copy engines over peer-mapped memory, stream-ordered signals"
                                  if peer is not None else "nccl")
                if strong and not self.check_broadcast(plan, A, B, Cm):
                    if peer is None:
                        raise RuntimeError("the broadcast operand differs between the ranks")
                    # The copy-engine route failed its check: the step uses NCCL.
                    plan.peer_broadcast = None
                    self.broadcast = "nccl"
                    self.broadcast_note = "the copy-engine route failed its check"
                    if not self.check_broadcast(plan, A, B, Cm):
                        raise RuntimeError("the broadcast operand differs between the ranks")

                def step():
                    plan.run(ALPHA, A, B, BETA, Cm)
            else:
                def step():
                    pgb.gemm(ALPHA, A, B, BETA, Cm)
        return step, ops

    # ---- timed region ----
    def time_steps(self, name, w, step, steps, warmup):
        torch, pgb = self.torch, self.pgb
        for _ in range(warmup):
            step()
        self.barrier()
        sampler = start_sampler(self.local) if self.rank == 0 else None
        stream = torch.cuda.current_stream()
        # Operands smaller than L2 (only the 1024^3 case) would be served from L2
        # on every step after the first: those steps are timed one by one, each
        # after a write larger than L2; everything else streams more than L2.
        small = operand_bytes(name, w) < 2 * L2_BYTES
        l0 = pgb.launch_count()
        if small:
            if self.flush is None:
                self.flush = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=self.dev)
            pairs = []
            for _ in range(steps):
                self.flush.fill_(1)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                step()
                b.record(stream)
                pairs.append((a, b))
            self.barrier()
            ms = sum(a.elapsed_time(b) for a, b in pairs)
        else:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                step()
            e1.record(stream)
            self.barrier()
            ms = e0.elapsed_time(e1)
        launches = pgb.launch_count() - l0
        clocks = sampler.stop() if sampler else None
        pgb.poll_device_status()
        if self.world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=self.dev)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps, int(launches), clocks

    # ---- dominant-kernel roofline ----
    def roofline(self, name, w, ms_per_step, clocks, peak_cold):
        pgb, world = self.pgb, self.world
        units = algorithmic_work(name, w)
        strong = bool(w.get("strong"))
        mhz = (clocks or {}).get("sm_mhz")
        extra = {"ms_x_sm_mhz": ms_per_step * mhz if mhz else None}
        if name.startswith("mvt"):
            peak = self.peaks.get("hbm_gbs", 6650.0)
            src = "of measured (MEASURED_PEAKS.json hbm_gbs)" if self.peaks else "of fallback"
            ach = units / (ms_per_step * 1e-3) / 1e9
            return {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s",
                    "frac": ach / peak, "traffic": TRAFFIC.get(name), "peak_source": src, **extra}
        if w["dtype"] == "f64":
            peak_hot = pgb.probe_peak(pgb.PEAK_DMMA) / 1e3
            peak = max(peak_cold or 0.0, peak_hot)
            # chained GEMM: two launches per step, both on this kernel
            ach = units / (ms_per_step * 1e-3) / 1e12
            return {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s",
                    "frac": ach / peak, "traffic": TRAFFIC.get(name),
                    "peak_burst": peak_cold, "peak_after_run": peak_hot,
                    "peak_source": "fp64 tensor (mma.sync .f64) issue-rate probe of this library, "
                                   "max of before/after the timed region (MEASURED_PEAKS.json has "
                                   "no fp64 figure)", **extra}
        # 3xTF32: every useful FMA costs three tensor-core FMAs, so the tensor
        # pipe does 3 * 2MNK flop per step; compare with dense TF32.
        peak_hot = pgb.probe_peak(pgb.PEAK_TF32) / 1e3
        burst = max(peak_cold or 0.0, peak_hot)
        # A kernel timed alone is compared with the burst figure.  A timed region
        # that sat at the 1 kW power cap (sw_power_cap seen by the clock sampler,
        # or a step of >= 100 ms) is compared with the sustained one:
        # MEASURED_PEAKS.json has the driver's burst and sustained numbers for a
        # tensor-core GEMM (bf16), and their ratio is applied to the TF32 burst
        # probe.  (The issue-loop probe run right after a long step is NOT an
        # upper bound: the two-CTA GEMM is more power-efficient than the probe.)
        capped = ms_per_step >= 100.0 or "sw_power_cap" in ((clocks or {}).get("reasons") or [])
        derate = 1.0
        if capped:
            try:
                derate = self.peaks["bf16_tflops_sustained"] / self.peaks["bf16_tflops"]
            except KeyError:
                derate = 1.4 / 1.59  # fallback ratio of the profiling recipe
        peak = burst * derate
        ach = 3 * (units / world if strong else units) / (ms_per_step * 1e-3) / 1e12
        # Context: the vendor library's dense TF32 GEMM on this GPU, measured in
        # this process with MEASURED_PEAKS.json's protocol (once; 1-GPU runs only).
        lib = self.library_tf32() if world == 1 else None
        lib_peak = None
        if lib and "burst_tflops" in lib:
            lib_peak = lib["sustained_tflops"] if capped else lib["burst_tflops"]
        return {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s",
                "frac": ach / peak, "frac_of_burst": ach / burst,
                "traffic": TRAFFIC.get(name) if world == 1 else None,
                "peak_burst": burst, "peak_after_run": peak_hot,
                "peak_source": "dense TF32 tcgen05.mma issue-rate probe of this library "
                               "(MEASURED_PEAKS.json has no TF32 figure): "
                               + (f"burst x {derate:.3f} (sustained/burst ratio of the measured "
                                  "bf16 GEMM) because the timed region ran at the power cap" if capped
                                  else "burst (max of before/after the timed region)")
                               + "; achieved counts the 3 tensor products per useful product",
                "library_tf32": lib,
                "frac_of_library": (ach / lib_peak) if lib_peak else None, **extra}

    def library_tf32(self):
        """Context for the power-capped fp32 figures: the vendor library's dense
        TF32 GEMM (torch.matmul with TF32 allowed, 8192^3) on this GPU, best of 10
        and back to back for 3 s - the same protocol MEASURED_PEAKS.json used for
        bf16.  Not a kernel of this library and not on its path; it only shows
        what a dense TF32 GEMM sustains under the same 1 kW cap."""
        torch = self.torch
        if getattr(self, "_lib_tf32", None) is not None:
            return self._lib_tf32
        try:
            old = torch.backends.cuda.matmul.allow_tf32
            torch.backends.cuda.matmul.allow_tf32 = True
            n = 8192
            a = torch.rand((n, n), dtype=torch.float32, device=self.dev)
            b = torch.rand((n, n), dtype=torch.float32, device=self.dev)
            c = torch.empty((n, n), dtype=torch.float32, device=self.dev)
            torch.cuda.synchronize()
            time.sleep(2.0)                      # from an idle GPU, like a burst probe
            best = 1e9
            for _ in range(10):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                torch.matmul(a, b, out=c)
                e1.record()
                torch.cuda.synchronize()
                best = min(best, e0.elapsed_time(e1))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = max(10, int(3000.0 / best))
            e0.record()
            for _ in range(reps):
                torch.matmul(a, b, out=c)
            e1.record()
            torch.cuda.synchronize()
            sus = e0.elapsed_time(e1) / reps
            torch.backends.cuda.matmul.allow_tf32 = old
            flop = 2.0 * n ** 3
            del a, b, c
            self._lib_tf32 = {"burst_tflops": flop / (best * 1e-3) / 1e12,
                              "sustained_tflops": flop / (sus * 1e-3) / 1e12,
                              "how": "torch.matmul, TF32 allowed, 8192^3: best of 10 / back to "
                                     "back for 3 s"}
        except Exception as ex:               # context only: never fails the bench
            self._lib_tf32 = {"error": repr(ex)}
        return self._lib_tf32

    def cold_peak(self, name, w):
        if self.rank != 0 or name.startswith("mvt"):
            return None
        pgb = self.pgb
        return pgb.probe_peak(pgb.PEAK_DMMA if w["dtype"] == "f64" else pgb.PEAK_TF32) / 1e3

    # ---- end to end through the reference-facing drop-in, host arrays ----
    def e2e_gemm(self, name, w, ops, total_units, scale, unit, steps):
        """pgb200_kernel_gemm on host copies of this rank's operands, three ways:
        pageable arrays (headline), page-locked arrays, and pageable arrays
        registered with pgb200Pin across repeated calls.  Returns (e2e, host B)."""
        import numpy as np
        torch, pgb, polybench = self.torch, self.pgb, self.polybench
        A, B, Cm = ops["A"], ops["B"], ops["C"]
        M, N, K = A.shape[0], w["N"], w["K"]
        if self.world > 1:
            self.dist.broadcast(B, src=0)  # every rank's host copy of the shared operand
        isz = 8 if w["dtype"] == "f64" else 4
        h2d, d2h = (M * K + K * N + M * N) * isz, M * N * isz
        big = name == "sgemm32768"
        reps = 1 if big else max(3, min(steps, 10))

        def timed(hA, hB, hC, n):
            polybench.kernel_gemm(M, N, K, ALPHA, BETA, hC, hA, hB)   # warm: buffers, pool
            self.barrier()
            sampler = start_sampler(self.local) if self.rank == 0 else None
            t0 = time.perf_counter()
            for _ in range(n):
                polybench.kernel_gemm(M, N, K, ALPHA, BETA, hC, hA, hB)
            torch.cuda.synchronize()
            dt = (time.perf_counter() - t0) / n
            ck = sampler.stop() if sampler else None
            if self.world > 1:
                t = torch.tensor([dt], dtype=torch.float64, device=self.dev)
                self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
                dt = float(t.item())
            return dt, (ck or {}).get("sm_mhz")
        # pageable: what malloc / posix_memalign give the nests
        pA, pB, pC = (t.cpu().numpy() for t in (A, B, Cm))
        dt_page, mhz = timed(pA, pB, pC, reps)
        e2e = {"value": total_units / dt_page / scale, "unit": unit, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "host_memory": "pageable", "ms_per_call": dt_page * 1e3,
               "sm_mhz": mhz}
        # the same arrays registered with pgb200Pin: resident across repeated calls
        nrep = 3 if big else 10
        t0 = time.perf_counter()
        for a in (pA, pB, pC):
            pgb.pin(a)
        t_pin = time.perf_counter() - t0
        polybench.kernel_gemm(M, N, K, ALPHA, BETA, pC, pA, pB)
        self.barrier()
        sampler = start_sampler(self.local) if self.rank == 0 else None
        t0 = time.perf_counter()
        for _ in range(nrep):
            polybench.kernel_gemm(M, N, K, ALPHA, BETA, pC, pA, pB)
        torch.cuda.synchronize()
        dt_res = (time.perf_counter() - t0) / nrep
        ck_res = sampler.stop() if sampler else None
        t0 = time.perf_counter()
        for a in (pA, pB, pC):
            pgb.unpin(a)
        t_unpin = time.perf_counter() - t0
        if self.world > 1:
            t = torch.tensor([dt_res], dtype=torch.float64, device=self.dev)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            dt_res = float(t.item())
        e2e["registered"] = {"value": total_units / dt_res / scale, "unit": unit,
                             "ms_per_call": dt_res * 1e3, "calls": nrep,
                             "sm_mhz": (ck_res or {}).get("sm_mhz"),
                             "pin_ms_once": t_pin * 1e3, "unpin_ms_once": t_unpin * 1e3,
                             "note": "host arrays registered with pgb200Pin: uploaded once, "
                                     "downloaded once at pgb200Unpin; per-call time excludes both"}
        host_b = pB
        del pA, pC
        # page-locked host arrays
        def pinned(t):
            h = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
            h.copy_(t)
            return h.numpy()
        hA, hB, hC = pinned(A), pinned(B), pinned(Cm)
        dt_pin, mhz = timed(hA, hB, hC, reps)
        e2e["page_locked"] = {"value": total_units / dt_pin / scale, "unit": unit,
                              "ms_per_call": dt_pin * 1e3, "sm_mhz": mhz}
        return e2e, host_b

    def e2e_mvt(self, w, ops, scale, unit):
        torch, polybench = self.torch, self.polybench
        n = min(8192, w["N"])  # host-array drop-in on a bounded sample (0.5 GB): PCIe-bound
        hAn = ops["A"][:n, :n].cpu().numpy().copy()
        hv = [v[:n].cpu().numpy().copy() for v in ops["vec"]]
        polybench.kernel_mvt(n, hv[0], hv[1], hv[2], hv[3], hAn)
        t0 = time.perf_counter()
        for _ in range(3):
            polybench.kernel_mvt(n, hv[0], hv[1], hv[2], hv[3], hAn)
        dt = (time.perf_counter() - t0) / 3
        return {"value": (n * n * 8 + 6 * n * 8) / dt / scale, "unit": unit,
                "h2d_bytes_per_step": n * n * 8 + 4 * n * 8, "d2h_bytes_per_step": 2 * n * 8,
                "host_memory": "pageable", "note": f"kernel_mvt drop-in at N={n}"}

    def measure(self, name, w, steps, warmup):
        """One workload on this process: (ms_per_step, launches, clocks, roofline, ops)."""
        step, ops = self.build(name, w)
        peak_cold = self.cold_peak(name, w)
        ms, launches, clocks = self.time_steps(name, w, step, steps, warmup)
        roof = self.roofline(name, w, ms, clocks, peak_cold) if self.rank == 0 else None
        return ms, launches, clocks, roof, ops


def run_pgb200(args, w, name):
    bench = Bench()
    torch, pgb = bench.torch, bench.pgb
    rank, world = bench.rank, bench.world
    strong_mg = world > 1 and bool(w.get("strong"))
    # The broadcast of the next operand chunk runs beside the GEMM of the
    # current one: optionally leave it some SMs.
    pgb.init(reserve_sms=int(os.environ.get("PGB_BENCH_RESERVE_SMS", "0")) if strong_mg else 0)
    metric, unit, scale = metric_of(name)
    units = algorithmic_work(name, w)
    strong = bool(w.get("strong"))
    total_units = units if strong else units * world

    ms_per_step, launches, clocks, roof, ops = bench.measure(name, w, args.steps, args.warmup)
    value = total_units / (ms_per_step * 1e-3) / scale

    e2e, host_b = None, None
    if not args.kernel_only:
        if name.startswith(("dgemm", "sgemm")):
            e2e, host_b = bench.e2e_gemm(name, w, ops, total_units, scale, unit, args.steps)
        elif name.startswith("mvt") and rank == 0:
            e2e = bench.e2e_mvt(w, ops, scale, unit)
    del ops
    torch.cuda.empty_cache()

    per_config = None
    if world == 1 and not args.kernel_only and not args.no_per_config:
        per_config = []
        for label, wn in PER_CONFIG:
            if wn == name:
                continue
            ww = WORKLOADS[wn]
            # The headline step runs at the power cap; let the clocks recover so
            # that each config is measured from an idle GPU, as a caller sees it.
            torch.cuda.synchronize()
            time.sleep(2.0)
            k = min(args.steps, 20 if wn != "sgemm32768" else 5)
            ms, ln, ck, rf, o = bench.measure(wn, ww, k, max(3, min(args.warmup, 5)))
            m2, u2, s2 = metric_of(wn)
            # end to end through the host-array drop-in where one call is short
            pe = None
            if wn.startswith(("dgemm", "sgemm")) and wn != "sgemm32768":
                pe, _ = bench.e2e_gemm(wn, ww, o, algorithmic_work(wn, ww), s2, u2, 5)
            elif wn.startswith("mvt"):
                pe = bench.e2e_mvt(ww, o, s2, u2)
            per_config.append({"config": label, "workload": ww["desc"], "metric": m2,
                               "value": algorithmic_work(wn, ww) / (ms * 1e-3) / s2, "unit": u2,
                               "dtype": ww["dtype"], "steps": k, "ms_per_step": ms,
                               "gpu_launches": ln, "l2": l2_note(wn, ww), "roofline": rf,
                               "clocks": ck, "e2e": pe})
            del o
            torch.cuda.empty_cache()

    if rank == 0:
        cpu = cpu_baseline(w, name, host_b) if (world == 1 and not args.kernel_only) else None
        line = {
            "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": w["dtype"],
            "data": "synthetic", "config": config_of(name, w, world),
            "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "roofline": roof,
            "cpu_baseline": cpu,
        }
        if per_config is not None:
            line["per_config"] = per_config
        if bench.broadcast is not None:
            line["broadcast"] = bench.broadcast
            if bench.broadcast_note:
                line["broadcast_note"] = bench.broadcast_note
        print(json.dumps(line))
    if world > 1:
        bench.dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="pgb200", choices=["pgb200", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the end-to-end, per-config and CPU-baseline legs (profiling runs)")
    ap.add_argument("--no-per-config", action="store_true",
                    help="skip the measurements of the other BASELINE configs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "pgb200" else args.warmup
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return
        run_reference(args, w, args.workload)
    else:
        run_pgb200(args, w, args.workload)


if __name__ == "__main__":
    main()
