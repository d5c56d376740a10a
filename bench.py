"""Benchmark of the brute.bit1 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--gemm-impl auto|popc|b1|i8|i8x2]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Headline workload: the large square binary GEMM, M = N = K = 16384 bit1 operands
(uint64-packed, uniform random bits from a seeded generator), int32 output
C = K - 2*popcount(a ^ b). One step = one pass of the GEMM. With N GPUs the rows
of B (output features) are split into N equal blocks, one per rank, with no
data-path collective (total work fixed: strong scaling). One JSON line is printed
by rank 0. Besides the contract keys it carries `roofline`, `cpu_baseline`,
`e2e`, `clocks`, `gpu_launches`, and an `extra` object with the bandwidth ops
(pack / unpack / popcount / bitwise GB/s), the binarised MLP and binary attention.

`--impl reference` times the CPU implementation of the same GEMM (the C
restatement of the reference's Highway path in oracle/, all host threads) on a
bounded sample of the workload; the reference's own extension cannot be built
offline (its Highway submodule is empty).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M = N = K = 16384
METRIC = "binary_gemm_tops"
UNIT = "TOPS (1 bit-MAC = 1 op)"
WORKLOAD = "xnor-popcount GEMM M=N=K=16384 bit1, uint64-packed, int32 out (BASELINE config 3)"


# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the pair kernel at 16384^3, from an ncu
# capture of `bench.py --size 16384 --steps 1` (the kernel re-reads operand tiles through L2, not DRAM)
NCU_DRAM_BYTES_16384 = 1.313e9
ALG_BYTES_16384 = 8 * 256 * (16384 + 16384) + 4 * 16384 * 16384


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--gemm-impl", default="auto", choices=["auto", "popc", "b1", "i8", "i8x2"])
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary workloads")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sustained-s", type=float, default=2.0,
                    help="seconds of back-to-back GEMM launches for the sustained figure (0 = skip)")
    ap.add_argument("--size", type=int, default=16384, help="M=N=K (profiling runs use smaller sizes)")
    ap.add_argument("--op", default="gemm",
                    help="time ONE op alone (for profiler captures): gemm | pack_sign | pack_bool | unpack_bool | "
                         "unpack_pm1 | popcount_total | hamming_total | word_popcount | xor | not | attention | mlp | "
                         "pack_bool_4097 | unpack_bool_4097 | memset | transpose_bits | any_dim0 | flip | roll | signed_bundle | "
                         "gather_sweep (under torchrun: the replicated result over peer memory, parameter sweep)")
    ap.add_argument("--log2-bits", type=int, default=28, help="size of the bandwidth ops under --op")
    ap.add_argument("--att", default="2,8,4096,128", help="B,H,S,D of --op attention")
    return ap.parse_args()


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ---------------------------------------------------------------------------
# CPU arm (oracle port of the reference's CPU path)
# ---------------------------------------------------------------------------
def cpu_gemm_sample(size: int, target_s: float = 10.0):
    """Time the CPU GEMM on rows [0:r) x [0:r) of the workload, full K."""
    import numpy as np
    from oracle import c_oracle as co
    co.build()
    # torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU arm uses every core it may run on
    co.set_num_threads(len(os.sched_getaffinity(0)))
    rng = np.random.default_rng(1234)
    kp = size // 64
    probe = min(1024, size)
    A = rng.integers(-2 ** 63, 2 ** 63 - 1, size=(probe, kp), dtype=np.int64)
    B = rng.integers(-2 ** 63, 2 ** 63 - 1, size=(probe, kp), dtype=np.int64)
    co.xnor_gemm(A[:64], B[:64], size)                      # warm the thread pool
    t0 = time.perf_counter()
    co.xnor_gemm(A, B, size)
    t_probe = max(time.perf_counter() - t0, 1e-6)
    rate = probe * probe * size / t_probe
    rows = int(min(size, max(probe, (target_s * rate / size) ** 0.5)))
    rows = max(256, rows // 256 * 256)
    return co, rng, rows, kp


def run_reference_arm(args):
    import numpy as np
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    size = args.size
    # each step is a bounded sample sized so that steps + warmup end within a few minutes
    total_calls = max(1, args.steps + args.warmup)
    co, rng, rows, kp = cpu_gemm_sample(size, target_s=min(10.0, 120.0 / total_calls))
    A = rng.integers(-2 ** 63, 2 ** 63 - 1, size=(rows, kp), dtype=np.int64)
    B = rng.integers(-2 ** 63, 2 ** 63 - 1, size=(rows, kp), dtype=np.int64)
    for _ in range(args.warmup):
        co.xnor_gemm(A, B, size)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        co.xnor_gemm(A, B, size)
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    tops = rows * rows * size / dt / 1e12
    sample = f"rows [0:{rows}) of A against rows [0:{rows}) of B, full K={size} ({rows}x{rows}x{size} bit-MACs per step)"
    line = {
        "impl": "reference", "metric": METRIC, "value": tops, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "u64", "data": "synthetic",
        "config": {"workload": WORKLOAD if size == 16384 else f"xnor-popcount GEMM M=N=K={size}",
                   "sharding": "none (the CPU arm runs on rank 0's host cores only)", "gemm_impl": "cpu port of the reference's Highway path",
                   "l2": "n/a (host)", "timing": "wall clock around the steps", "sample": sample},
        "cpu_baseline": {"value": tops, "unit": UNIT, "cores": co.num_threads(), "kind": "port", "sample": sample,
                         "host_cpus": os.cpu_count(), "vpopcntdq": co.has_vpopcntdq()},
        "e2e": {"value": tops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
class ClockSampler:
    """Reads (never sets) SM clocks and throttle reasons of one GPU through NVML."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz, self.power = [], set(), None, []
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
                get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
                mask = int(get(self.h))
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.005)

    def start(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()

    def stop(self):
        self._stop.set()
        if self._thr is not None:
            self._thr.join(timeout=2)
        med = int(statistics.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples),
                "power_w_median": round(statistics.median(self.power), 1) if self.power else None,
                "power_w_max": round(max(self.power), 1) if self.power else None}


def pin_to_gpu_numa_node(index: int) -> None:
    """Run this rank on the CPUs next to its GPU (a setting of this process only), so that the pinned
    host buffers of the end-to-end leg are allocated on the GPU's own NUMA node and the ranks do not
    all pull their results through one socket."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * i + b for i, w in enumerate(mask) for b in range(64) if (int(w) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
    except Exception:
        pass


def time_steps(fn, steps, warmup, flush, stream_sync):
    """Per-step CUDA events on the launching stream, L2 flushed between steps
    (outside the timed spans). Returns the list of step times in ms."""
    import torch
    for _ in range(warmup):
        flush()
        fn()
    stream_sync()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for s, e in evs:
        flush()
        s.record()
        fn()
        e.record()
    stream_sync()
    return [s.elapsed_time(e) for s, e in evs]


def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        pin_to_gpu_numa_node(local_rank)
        dist.init_process_group("nccl", device_id=dev)

    import brute_b200 as brute  # fails loudly if the CUDA library is missing
    from brute_b200 import _lib as L
    from brute_b200.kernels import shard_bounds
    ops = torch.ops.brute
    impl = {"auto": L.GEMM_AUTO, "popc": L.GEMM_POPC, "b1": L.GEMM_MMA_B1, "i8": L.GEMM_TCGEN05, "i8x2": L.GEMM_TCGEN05_PAIR}[args.gemm_impl]
    size = args.size
    m = n = k = size
    kp = k // 64
    peaks = measured_peaks()

    # identical operands on every rank from the seed; each rank keeps its block of B's rows
    g = torch.Generator(device=dev).manual_seed(1234)
    A = torch.randint(-2 ** 63, 2 ** 63 - 1, (m, kp), generator=g, dtype=torch.int64, device=dev)
    Bfull = torch.randint(-2 ** 63, 2 ** 63 - 1, (n, kp), generator=g, dtype=torch.int64, device=dev)
    lo, hi = shard_bounds(n, world, rank)
    B = Bfull[lo:hi].contiguous()
    if world == 1:
        del Bfull
    n_loc = hi - lo

    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)      # 2x the 126 MB L2

    def flush():
        flush_buf.zero_()

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    holder = {}

    def step():
        # the reference's own schema (cbrute/ext.cpp:50); the variant with an explicit kernel choice
        # only when --gemm-impl asks for one
        if args.gemm_impl == "auto":
            holder["C"] = ops.xnor_popcount_matmul(A, B, k)
        else:
            holder["C"] = ops.xnor_popcount_matmul_impl(A, B, k, impl)

    sampler = ClockSampler(local_rank)
    sync()
    sampler.start()
    times = time_steps(step, args.steps, args.warmup, flush, sync)
    clocks = sampler.stop()
    status = L.load().brute_b200_device_status()
    if status != 0:
        raise SystemExit(f"GEMM kernel reported status {status}: {L.strerror(status)}")
    total_ms = sum(times)
    t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    macs_all = float(m) * n * k
    value = macs_all / (ms_per_step * 1e-3) / 1e12

    # roofline of the dominant kernel (this rank's launch)
    my_ms = sum(times) / args.steps
    my_macs = float(m) * n_loc * k
    if args.gemm_impl in ("auto", "i8", "i8x2"):
        # tcgen05 kind::i8: 2 int8 ops per bit-MAC; int8 dense runs at twice the bf16 rate on B200
        achieved = 2 * my_macs / (my_ms * 1e-3) / 1e12
        peak = 2 * peaks["bf16_tflops"]
        # DRAM bytes of one 16384^3 launch from the committed ncu capture of this kernel
        # (dram__bytes_read.sum + dram__bytes_write.sum), scaled by the outputs this launch writes
        alg_bytes = 8 * kp * (m + n_loc) + 4 * m * n_loc          # this rank's launch: A replicated, its block of B and C
        traffic = NCU_DRAM_BYTES_16384 * alg_bytes / ALG_BYTES_16384 if size == 16384 else None
        pipe = 148 * 8192 * 2 * 1.965e9 / 1e12     # int8 MACs/clk/SM x 2 ops x SMs x max SM clock
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TOP/s (int8, 2 per bit-MAC)",
                "frac": achieved / peak, "traffic": traffic,
                "peak_source": f"DERIVED: 2 x bf16_tflops (burst) of {peaks['source']} MEASURED_PEAKS.json (the file has no int8 "
                               "figure; int8 dense runs at twice the bf16 rate; a cuBLAS bf16 GEMM does not saturate its pipe, "
                               "so a fraction above 1 is possible)",
                "traffic_source": "ncu dram bytes of one 16384^3 launch x this launch's share of the algorithmic bytes "
                                  "(A replicated, B and C split by rank)" if traffic is not None else None,
                "frac_of_pipe_rate": achieved / pipe,
                "algorithmic_bytes_per_launch": 8 * kp * (m + n_loc) + 4 * m * n_loc}
    else:
        alg = 8 * kp * (m + n_loc) + 4 * m * n_loc
        achieved = alg / (my_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                "note": "CUDA-core / mma.sync paths are instruction bound; HBM figure shown for reference"}

    # ---- sustained: >= 2 s of back-to-back launches, no flush (the 1 GiB result does not fit L2),
    #      clocks / power / throttle reasons sampled during the span
    sustained = None
    if args.sustained_s > 0 and args.gemm_impl in ("auto", "i8", "i8x2"):
        n_launch = max(10, int(args.sustained_s * 1e3 / max(my_ms, 1e-3)))
        s_sampler = ClockSampler(local_rank)
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s_sampler.start()
        e0.record()
        for _ in range(n_launch):
            step()
        e1.record()
        torch.cuda.synchronize()
        s_clk = s_sampler.stop()
        s_ms = e0.elapsed_time(e1) / n_launch
        ts_ = torch.tensor([s_ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ts_, op=dist.ReduceOp.MAX)
        s_ms_all = float(ts_.item())
        s_ach = 2 * my_macs / (s_ms * 1e-3) / 1e12
        sustained = {"launches": n_launch, "ms_per_launch": s_ms_all, "tops": macs_all / (s_ms_all * 1e-3) / 1e12,
                     "int8_top_s_this_rank": s_ach, "peak": 2 * peaks["bf16_tflops_sustained"],
                     "frac": s_ach / (2 * peaks["bf16_tflops_sustained"]),
                     "peak_source": "DERIVED: 2 x bf16_tflops_sustained of " + peaks["source"] + " MEASURED_PEAKS.json",
                     "clocks": s_clk,
                     "ms_x_median_mhz": (s_ms * s_clk["sm_mhz"]) if s_clk.get("sm_mhz") else None,
                     "burst_ms_x_median_mhz": (my_ms * clocks["sm_mhz"]) if clocks.get("sm_mhz") else None}
        if L.load().brute_b200_device_status() != 0:
            raise SystemExit("GEMM kernel reported a bounded-wait timeout in the sustained leg")

    # ---- end to end through the public op with HOST buffers (pinned), every step:
    #      H2D of both operands, the op, D2H of the int32 result
    e2e = None
    if rank == 0 or world > 1:
        from brute_b200.kernels import host_matmul
        hA = A.cpu().pin_memory()
        hB = B.cpu().pin_memory()
        hC = torch.empty((m, n_loc), dtype=torch.int32).pin_memory()

        def e2e_step():
            # the public host-buffer call: H2D of B and of A block by block, the GEMM of each
            # block, D2H of that block of C, overlapped on three streams
            host_matmul(hA, hB, k, out=hC, device=dev, impl=impl)

        e_steps = max(3, min(args.steps, 5))
        e_times = time_steps(e2e_step, e_steps, 1, flush, sync)
        te = torch.tensor([sum(e_times)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e_ms = float(te.item()) / e_steps
        e2e = {"value": macs_all / (e_ms * 1e-3) / 1e12, "unit": UNIT,
               "h2d_bytes_per_step": int(hA.numel() * 8 + hB.numel() * 8),
               "d2h_bytes_per_step": int(hC.numel() * 4), "ms_per_step": e_ms, "steps": e_steps,
               "d2h_GB/s_per_rank": hC.numel() * 4 / (e_ms * 1e-3) / 1e9,
               "note": "bytes are this rank's; every rank moves its own block of C over its own PCIe link"}
        # the copied-back result is the device result
        assert torch.equal(hC[:8], holder["C"][:8].cpu())

    extra = {"all_gather_C_ms": None, "tops_with_gather": None, "replicated_result_ms": None}
    if world > 1:
        # The replicated result (optional in the workload): every rank ends with the full int32 C.
        # (a) the plain NCCL all-gather of the int32 blocks, timed apart from the GEMM, for reference;
        c_loc = holder["C"]
        gathered = torch.empty((world * m, n_loc), dtype=torch.int32, device=dev)
        g_times = time_steps(lambda: dist.all_gather_into_tensor(gathered, c_loc), 3, 1, lambda: None, sync)
        tg = torch.tensor([sum(g_times) / 3], dtype=torch.float64, device=dev)
        dist.all_reduce(tg, op=dist.ReduceOp.MAX)
        extra["all_gather_C_ms"] = float(tg.item())
        del gathered
        # (b) the public call, sharded_matmul(gather=True): GEMM by row blocks, int16 blocks, each block's
        #     exchange under the next block's GEMM. Default: one kernel per row block pulls the peers'
        #     blocks over NVLink (peer memory) and widens them into place; where no peer mapping is to
        #     be had, NCCL all-gather + a widening pass (timed here as well, for comparison)
        from brute_b200 import kernels as bk
        from brute_b200.kernels import sharded_matmul
        rep = {}

        def rep_step():
            rep["C"] = sharded_matmul(A, Bfull, k, gather=True)

        def timed_rep():
            ts = time_steps(rep_step, 5, 2, flush, sync)
            t = torch.tensor([sum(ts) / 5], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        os.environ["BRUTE_B200_GATHER"] = "nccl"
        extra["replicated_result_nccl_ms"] = timed_rep()
        assert torch.equal(rep["C"][:, lo:hi], holder["C"]), "replicated result (NCCL path) differs from the local block"
        os.environ["BRUTE_B200_GATHER"] = "peer"
        tr = torch.tensor([timed_rep()], dtype=torch.float64, device=dev)
        peer_used = torch.tensor([1 if bk._peer_ws and all(bool(v) for v in bk._peer_ws.values()) else 0], device=dev)
        dist.all_reduce(peer_used, op=dist.ReduceOp.MIN)
        extra["replicated_result_path"] = "peer memory (own kernel, plain peer loads by bulk copy)" if int(peer_used.item()) else "NCCL all-gather + widening pass"
        extra["peer_wait_status"] = bk.peer_gather_status()
        extra["replicated_result_ms"] = float(tr.item())
        # what has to cross NVLink into every rank: the other ranks' int16 blocks; 770 GB/s per direction is
        # the measured peer-copy rate of this pool (900 nominal)
        inbound = (world - 1) * m * n_loc * 2
        extra["replicated_result_link"] = {"inbound_bytes_per_rank": inbound, "floor_ms_at_770GB/s": inbound / 770e9 * 1e3,
                                           "achieved_GB/s_over_whole_call": inbound / (float(tr.item()) * 1e-3) / 1e9}
        extra["tops_with_gather"] = macs_all / (float(tr.item()) * 1e-3) / 1e12
        extra["tops_with_plain_int32_gather"] = macs_all / ((ms_per_step + float(tg.item())) * 1e-3) / 1e12
        # this rank's columns of the replicated result are its own GEMM block, bit for bit
        assert torch.equal(rep["C"][:, lo:hi], holder["C"]), "replicated result differs from the local block"
        del rep

    if world > 1 and not args.no_extra and size == 16384:
        # binary attention B=8 H=32 S=4096 D=128 causal, the 256 heads split across the ranks
        # (no collective on the path); time = max over ranks, rate = all heads / that time
        Bq, H, S, D = 8, 32, 4096, 128
        ga = torch.Generator(device=dev).manual_seed(77)      # same operands on every rank
        qb = brute.pack_sign(torch.randn((Bq, H, S, D), generator=ga, device=dev), ge0=True)
        kb = brute.pack_sign(torch.randn((Bq, H, S, D), generator=ga, device=dev), ge0=True)
        vb = torch.randn((Bq, H, S, D), generator=ga, device=dev).to(torch.bfloat16)
        a_times = time_steps(lambda: brute.sharded_attention(qb, kb, vb, causal=True), 5, 3, flush, sync)
        ta = torch.tensor([sum(a_times) / 5], dtype=torch.float64, device=dev)
        dist.all_reduce(ta, op=dist.ReduceOp.MAX)
        a_ms = float(ta.item())
        pairs = Bq * H * S * (S + 1) / 2
        extra["attention_8x32x4096x128_causal_sharded"] = {
            "ms": a_ms, "heads_per_rank": Bq * H // world, "score_bitmac_tops": pairs * D / (a_ms * 1e-3) / 1e12,
            "pv_tflops": 2 * pairs * D / (a_ms * 1e-3) / 1e12, "sharding": "batch x head, no collective"}
        del qb, kb, vb

    if rank == 0 and not args.no_extra and size == 16384:
        # rank 0 alone runs these: synchronise the device only, no collective
        extra.update(secondary_workloads(dev, peaks, flush, torch.cuda.synchronize))

    cpu_base = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import numpy as np
        co, rng, rows, _ = cpu_gemm_sample(size, target_s=10.0)
        a_np = rng.integers(-2 ** 63, 2 ** 63 - 1, size=(rows, kp), dtype=np.int64)
        b_np = rng.integers(-2 ** 63, 2 ** 63 - 1, size=(rows, kp), dtype=np.int64)
        t0 = time.perf_counter()
        c_np = co.xnor_gemm(a_np, b_np, k)
        dt = time.perf_counter() - t0
        # the same sample on the GPU must give the same integers
        c_gpu = ops.xnor_popcount_matmul_impl(torch.from_numpy(a_np).to(dev), torch.from_numpy(b_np).to(dev), k, impl)
        assert np.array_equal(c_gpu.cpu().numpy(), c_np), "GPU result differs from the CPU baseline's"
        # BASELINE config 2 on the host: float threshold + pack of 2^26 elements
        x_np = rng.standard_normal((1 << 10, 1 << 16), dtype=np.float32)     # rows are the oracle's unit of threading
        co.pack_sign_f32(x_np[:16], 1)
        t0 = time.perf_counter()
        co.pack_sign_f32(x_np, 1)
        dt_pack = time.perf_counter() - t0
        del x_np
        cpu_base = {"pack_sign_f32_2^26_GB/s": (4.125 * (1 << 26)) / dt_pack / 1e9,
                    "value": rows * rows * k / dt / 1e12, "unit": UNIT, "cores": co.num_threads(), "kind": "port",
                    "sample": f"{rows}x{rows} outputs, full K={k}, {dt:.2f} s", "host_cpus": os.cpu_count(),
                    "vpopcntdq": co.has_vpopcntdq()}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "u64", "data": "synthetic",
            "config": {"workload": WORKLOAD if size == 16384 else f"xnor-popcount GEMM M=N=K={size}",
                       "sharding": f"B rows (output features) split in {world} block(s), A replicated, no collective",
                       "gemm_impl": args.gemm_impl, "l2": "flushed between steps (256 MiB memset outside the timed spans)",
                       "timing": "per-step CUDA events on the launching stream, max over ranks of the sum",
                       "sample": "the whole workload, every step"},
            "roofline": roof, "cpu_baseline": cpu_base, "e2e": e2e, "clocks": clocks, "sustained": sustained,
            "gpu_launches": args.steps, "extra": extra,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def secondary_workloads(dev, peaks, flush, sync):
    """Bandwidth ops at 2^30 bits, the [4096, 4097] bool case, the binarised MLP and
    binary attention: algorithmic GB/s or rate, fraction of the measured HBM peak."""
    import torch
    import brute_b200 as brute
    ops = torch.ops.brute
    out = {}
    hbm = peaks["hbm_gbs"]

    def bw(name, fn, alg_bytes, steps=10):
        ts = time_steps(fn, steps, 3, flush, sync)
        ms = statistics.median(ts)
        gbs = alg_bytes / (ms * 1e-3) / 1e9
        out[name] = {"ms": ms, "GB/s": gbs, "frac_of_hbm": gbs / hbm, "algorithmic_bytes": alg_bytes}

    def rotating(name, fns, alg_bytes, steps=10):
        """A 30 us op bracketed by two events carries about 5 us of event and launch-gap time (ncu sees the
        same kernel at 25 us). Second figure for such ops: len(fns) launches on DISTINCT inputs, together
        several times the L2, inside one event pair with no flush in between (every input was evicted by the
        others before its turn comes again); per-op time = span / len(fns)."""
        for _ in range(2):
            for f in fns:
                f()
        ts = time_steps(lambda: [f() for f in fns], steps, 2, flush, sync)
        ms = statistics.median(ts) / len(fns)
        out[name]["rotating_inputs"] = {"launches_per_span": len(fns), "ms_per_op": ms,
                                        "frac_of_hbm": alg_bytes / (ms * 1e-3) / 1e9 / hbm}

    side = torch.cuda.Stream(dev)

    def graph_us(fn):
        """Median time of the replay of a CUDA graph that holds the op's launches (L2 flushed before
        every replay): the kernel time without the host's dispatch of the op."""
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                fn()
        torch.cuda.current_stream(dev).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            held = fn()
        us = statistics.median(time_steps(graph.replay, 9, 3, flush, sync)) * 1e3
        del graph, held
        return us

    n = 1 << 30
    g = torch.Generator(device=dev).manual_seed(1235)
    x = torch.randn(n, generator=g, device=dev)
    bw("pack_sign_f32_2^30", lambda: ops.pack_sign(x, 1), 4 * n + n // 8)
    p = ops.pack_sign(x, 1)

    # BASELINE config 2 sweep: fp32 [2^k], k = 10..30, threshold x >= 0. Small sizes are bound by
    # the dispatch of one op from Python, so each size is timed twice: as an eager call and as the
    # replay of a CUDA graph that holds the one kernel (L2 flushed before every timed launch).
    sweep = {"k": [], "eager_us": [], "graph_us": [], "graph_GB/s": []}
    for k in range(10, 31):
        xk = x[: 1 << k]
        eager = statistics.median(time_steps(lambda: ops.pack_sign(xk, 1), 7, 3, flush, sync))
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                ops.pack_sign(xk, 1)
        torch.cuda.current_stream(dev).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            held = ops.pack_sign(xk, 1)
        replay = statistics.median(time_steps(graph.replay, 7, 3, flush, sync))
        del graph, held
        sweep["k"].append(k)
        sweep["eager_us"].append(round(eager * 1e3, 2))
        sweep["graph_us"].append(round(replay * 1e3, 2))
        sweep["graph_GB/s"].append(round((4 * (1 << k) + (1 << k) // 8) / (replay * 1e-3) / 1e9, 1))
    out["pack_sign_f32_sweep"] = sweep
    del x
    q = torch.randint(-2 ** 63, 2 ** 63 - 1, (n // 64,), generator=g, dtype=torch.int64, device=dev)
    bw("unpack_bool_2^30", lambda: ops.unpack_bool(p, [n]), n // 8 + n)
    xb = ops.unpack_bool(p, [n])
    bw("pack_bool_2^30", lambda: ops.pack_bool(xb), n + n // 8)
    del xb
    bw("unpack_pm1_f32_2^30", lambda: ops.unpack_bits(p, [n]), n // 8 + 4 * n, steps=5)
    bw("popcount_total_2^30", lambda: ops.packed_popcount(p), n // 8)
    rot = [p, q] + [torch.randint(-2 ** 63, 2 ** 63 - 1, (n // 64,), generator=g, dtype=torch.int64, device=dev) for _ in range(2)]
    rotating("popcount_total_2^30", [(lambda t=t: ops.packed_popcount(t)) for t in rot], n // 8)
    bw("hamming_total_2^30", lambda: ops.bit1_hamming_total(p, q), 2 * n // 8)
    bw("word_popcount_2^30", lambda: ops.popcount(p), n // 8 + n // 16)
    bw("xor_2^30", lambda: ops.bitwise_packed(p, q, 2, n), 3 * n // 8)
    bw("not_2^30", lambda: ops.bit1_not_packed(p, n), 2 * n // 8)
    p2 = p.view(32768, 512)
    bw("transpose_bits_32768x32768", lambda: ops.transpose_packed(p2, 32768, 32768), 2 * n // 8)
    bw("any_dim0_4096x2^18", lambda: ops.reduce_rows_packed(p.view(4096, 4096), 0, True), n // 8 + (1 << 18) // 8)
    rotating("any_dim0_4096x2^18", [(lambda t=t: ops.reduce_rows_packed(t.view(4096, 4096), 0, True)) for t in rot], n // 8 + (1 << 18) // 8)
    del rot
    p3 = p.view(1024, -1)                  # 1024 rows of 2^20 bits; the -5 makes every row ragged
    nrow = (1 << 20) - 5
    bw("flip_last_axis_1024x(2^20-5)", lambda: ops.flip_packed(p3, nrow), 2 * n // 8)
    bw("roll_last_axis_1024x(2^20-5)", lambda: ops.roll_packed(p3, nrow, 12345), 2 * n // 8)
    del p3
    del p, q, p2
    xb = torch.rand((4096, 4097), generator=g, device=dev) < 0.3
    bw("pack_bool_4096x4097", lambda: ops.pack_bool(xb), 4096 * 4097 + 4096 * 65 * 8)
    pb = ops.pack_bool(xb)
    bw("unpack_bool_4096x4097", lambda: ops.unpack_bool(pb, [4096, 4097]), 4096 * 4097 + 4096 * 65 * 8)
    bw("not_4096x4097", lambda: ops.bit1_not_packed(pb, 4097), 2 * 4096 * 65 * 8)
    # the same three as graph replays (no host dispatch in the span), and the flat kernel at the same bytes
    for name, fn, alg in (("pack_bool_4096x4097", lambda: ops.pack_bool(xb), 4096 * 4097 + 4096 * 65 * 8),
                          ("unpack_bool_4096x4097", lambda: ops.unpack_bool(pb, [4096, 4097]), 4096 * 4097 + 4096 * 65 * 8),
                          ("not_4096x4097", lambda: ops.bit1_not_packed(pb, 4097), 2 * 4096 * 65 * 8)):
        us = graph_us(fn)
        out[name]["graph_us"] = round(us, 2)
        out[name]["graph_GB/s"] = round(alg / (us * 1e-6) / 1e9, 1)
        out[name]["graph_frac_of_hbm"] = round(alg / (us * 1e-6) / 1e9 / hbm, 3)
    xflat = xb.reshape(-1)[: 4096 * 4096].contiguous()
    out["pack_bool_flat_2^24"] = {"graph_us": round(graph_us(lambda: ops.pack_bool(xflat)), 2),
                                  "algorithmic_bytes": 4096 * 4096 + 4096 * 4096 // 8}
    pflat = ops.pack_bool(xflat)
    out["unpack_bool_flat_2^24"] = {"graph_us": round(graph_us(lambda: ops.unpack_bool(pflat, [4096 * 4096])), 2),
                                    "algorithmic_bytes": 4096 * 4096 + 4096 * 4096 // 8}
    del xb, pb, xflat, pflat
    # scatter through a tensor index on the packed axis: 4096 rows of 2^16 bits, 8192 positions per row
    ps = torch.randint(-2 ** 63, 2 ** 63 - 1, (4096, 1024), generator=g, dtype=torch.int64, device=dev)
    idx = torch.randperm(1 << 16, generator=g, device=dev)[:8192]
    srcp = torch.randint(-2 ** 63, 2 ** 63 - 1, (4096, 128), generator=g, dtype=torch.int64, device=dev)
    ts = time_steps(lambda: ops.scatter_packed_(ps, idx, srcp, False, 1 << 16), 10, 3, flush, sync)
    out["scatter_last_axis_4096x2^16_8192idx"] = {"ms": statistics.median(ts),
                                                  "bit_writes_per_s": 4096 * 8192 / (statistics.median(ts) * 1e-3)}
    del ps, idx, srcp

    # binarised MLP, batch 8192, 4096 -> 16384 -> 4096 (BASELINE config 4)
    xs = brute.pack_sign(torch.randn((8192, 4096), generator=g, device=dev), ge0=True)
    w1 = brute.pack_sign(torch.randn((16384, 4096), generator=g, device=dev), ge0=True)
    w2 = brute.pack_sign(torch.randn((4096, 16384), generator=g, device=dev), ge0=True)
    s1 = torch.rand(16384, generator=g, device=dev) + 0.5
    s2 = torch.rand(4096, generator=g, device=dev) + 0.5

    def mlp():
        return brute.binary_linear(brute.binary_linear(xs, w1, s1), w2, s2)
    ts = time_steps(mlp, 10, 3, flush, sync)
    ms = statistics.median(ts)
    macs = 2 * 8192.0 * 4096 * 16384
    out["mlp_8192x4096x16384x4096"] = {"ms": ms, "tops": macs / (ms * 1e-3) / 1e12}
    del xs, w1, w2

    # signed_bundle: int8 votes [256, 1024, 1024] x bit1 values [256, 1024, 128] -> bit1 [256, 1024, 128]
    Bb, Mb, Nb, Db = 256, 1024, 1024, 128
    wv = torch.randint(-3, 4, (Bb, Mb, Nb), generator=g, device=dev, dtype=torch.int8)
    vv = torch.randint(-2 ** 63, 2 ** 63 - 1, (Bb, Nb, Db // 64), generator=g, dtype=torch.int64, device=dev)
    ts = time_steps(lambda: ops.signed_bundle(wv, vv, Db), 5, 2, flush, sync)
    ms = statistics.median(ts)
    alg = Bb * Mb * Nb + Bb * Nb * Db // 8 + Bb * Mb * Db // 8
    out["signed_bundle_256x1024x1024x128"] = {
        "ms": ms, "int8_x_bit_tmacs": float(Bb) * Mb * Nb * Db / (ms * 1e-3) / 1e12,
        "algorithmic_bytes": alg, "GB/s": alg / (ms * 1e-3) / 1e9, "frac_of_hbm": alg / (ms * 1e-3) / 1e9 / hbm}
    # second figure as for the 30 us reductions: three launches on three distinct W (0.8 GB together) per event pair
    wrot = [wv] + [torch.randint(-3, 4, (Bb, Mb, Nb), generator=g, device=dev, dtype=torch.int8) for _ in range(2)]
    rotating("signed_bundle_256x1024x1024x128", [(lambda w=w: ops.signed_bundle(w, vv, Db)) for w in wrot], alg, steps=5)
    del wv, vv, wrot

    # binary attention B=8 H=32 S=4096 D=128 causal (BASELINE config 5)
    Bq, H, S, D = 8, 32, 4096, 128
    qb = brute.pack_sign(torch.randn((Bq, H, S, D), generator=g, device=dev), ge0=True)
    kb = brute.pack_sign(torch.randn((Bq, H, S, D), generator=g, device=dev), ge0=True)
    v = torch.randn((Bq, H, S, D), generator=g, device=dev).to(torch.bfloat16)
    ts = time_steps(lambda: brute.binary_attention(qb, kb, v, causal=True), 5, 2, flush, sync)
    ms = statistics.median(ts)
    pairs = Bq * H * S * (S + 1) / 2
    # observed error of one head of this very run against the CPU oracle (the tolerance is 2e-2)
    err = None
    try:
        import numpy as np
        from oracle import c_oracle as co
        o_gpu = brute.binary_attention(qb, kb, v, causal=True)[:1, :1].float().cpu().numpy()
        o_ref = co.binary_attention(qb._packed_buf[:1, :1].cpu().numpy(), kb._packed_buf[:1, :1].cpu().numpy(),
                                    v[:1, :1].float().cpu().numpy(), True, D ** -0.5)
        num = np.sqrt(((o_gpu - o_ref) ** 2).sum(-1))
        den = np.maximum(np.sqrt((o_ref ** 2).sum(-1)), 1e-6)
        err = {"max_norm": float(np.abs(o_gpu - o_ref).max() / np.abs(o_ref).max()), "worst_row_rel_l2": float((num / den).max()),
               "tolerance": 2e-2, "checked": "head (0, 0) of this run, S = 4096, against the CPU oracle"}
    except Exception as exc:                                  # the checker is optional here
        err = {"unavailable": repr(exc)}
    out["attention_8x32x4096x128_causal"] = {
        "ms": ms, "score_bitmac_tops": pairs * D / (ms * 1e-3) / 1e12,
        "pv_tflops": 2 * pairs * D / (ms * 1e-3) / 1e12,
        "algorithmic_bytes": 2 * Bq * H * S * 16 + 2 * Bq * H * S * D * 2, "observed_error": err}
    return out


def run_single_op(args):
    """One op alone, a few launches, one JSON line: the command that profiler captures use."""
    import torch
    import brute_b200 as brute
    ops = torch.ops.brute
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = measured_peaks()
    n = 1 << args.log2_bits
    g = torch.Generator(device=dev).manual_seed(1235)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    alg = None
    if args.op in ("pack_sign",):
        x = torch.randn(n, generator=g, device=dev)
        fn, alg = (lambda: ops.pack_sign(x, 1)), 4 * n + n // 8
    elif args.op == "attention":
        Bq, H, S, D = (int(v) for v in args.att.split(","))
        qb = brute.pack_sign(torch.randn((Bq, H, S, D), generator=g, device=dev), ge0=True)
        kb = brute.pack_sign(torch.randn((Bq, H, S, D), generator=g, device=dev), ge0=True)
        v = torch.randn((Bq, H, S, D), generator=g, device=dev).to(torch.bfloat16)
        fn, alg = (lambda: brute.binary_attention(qb, kb, v, causal=True)), 2 * Bq * H * S * (D // 4) + 2 * Bq * H * S * D * 2
    elif args.op == "signed_bundle":
        Bb, Mb, Nb, Db = 256, 1024, 1024, 128
        wv = torch.randint(-3, 4, (Bb, Mb, Nb), generator=g, device=dev, dtype=torch.int8)
        vv = torch.randint(-2 ** 63, 2 ** 63 - 1, (Bb, Nb, Db // 64), generator=g, dtype=torch.int64, device=dev)
        fn, alg = (lambda: ops.signed_bundle(wv, vv, Db)), Bb * Mb * Nb + Bb * Nb * Db // 8 + Bb * Mb * Db // 8
    elif args.op == "mlp":
        xs = brute.pack_sign(torch.randn((8192, 4096), generator=g, device=dev), ge0=True)
        w1 = brute.pack_sign(torch.randn((16384, 4096), generator=g, device=dev), ge0=True)
        w2 = brute.pack_sign(torch.randn((4096, 16384), generator=g, device=dev), ge0=True)
        s1 = torch.rand(16384, generator=g, device=dev) + 0.5
        s2 = torch.rand(4096, generator=g, device=dev) + 0.5
        fn = lambda: brute.binary_linear(brute.binary_linear(xs, w1, s1), w2, s2)
    else:
        p = torch.randint(-2 ** 63, 2 ** 63 - 1, (n // 64,), generator=g, dtype=torch.int64, device=dev)
        q = torch.randint(-2 ** 63, 2 ** 63 - 1, (n // 64,), generator=g, dtype=torch.int64, device=dev)
        table = {
            "unpack_bool": (lambda: ops.unpack_bool(p, [n]), n // 8 + n),
            "unpack_pm1": (lambda: ops.unpack_bits(p, [n]), n // 8 + 4 * n),
            "popcount_total": (lambda: ops.packed_popcount(p), n // 8),
            "hamming_total": (lambda: ops.bit1_hamming_total(p, q), 2 * n // 8),
            "word_popcount": (lambda: ops.popcount(p), n // 8 + n // 16),
            "xor": (lambda: ops.bitwise_packed(p, q, 2, n), 3 * n // 8),
            "not": (lambda: ops.bit1_not_packed(p, n), 2 * n // 8),
            "transpose_bits": (lambda: ops.transpose_packed(p.view(1 << (args.log2_bits // 2), -1), 1 << (args.log2_bits // 2),
                                                           64 * ((n // 64) >> (args.log2_bits // 2))), 2 * n // 8),
            "any_dim0": (lambda: ops.reduce_rows_packed(p.view(4096, -1), 0, True), n // 8 + n // 8 // 4096),
            "flip": (lambda: ops.flip_packed(p.view(1024, -1), n // 1024 - 5), 2 * n // 8),
            "roll": (lambda: ops.roll_packed(p.view(1024, -1), n // 1024 - 5, 12345), 2 * n // 8),
        }
        if args.op == "pack_bool":
            xb = ops.unpack_bool(p, [n])
            fn, alg = (lambda: ops.pack_bool(xb)), n + n // 8
        elif args.op in ("pack_bool_4097", "unpack_bool_4097"):
            # BASELINE config 2's ragged case: bool [4096, 4097], 65 words per row, 1 valid bit in the last
            xr = torch.rand((4096, 4097), generator=g, device=dev) < 0.3
            pr = ops.pack_bool(xr)
            alg = 4096 * 4097 + 4096 * 65 * 8
            fn = (lambda: ops.pack_bool(xr)) if args.op == "pack_bool_4097" else (lambda: ops.unpack_bool(pr, [4096, 4097]))
        elif args.op == "memset":
            # write-only reference: how fast this GPU stores, to read the unpack numbers against
            buf = torch.empty(n, dtype=torch.uint8, device=dev)
            fn, alg = buf.zero_, n
        else:
            fn, alg = table[args.op]
    ts = time_steps(fn, args.steps, args.warmup, flush_buf.zero_, torch.cuda.synchronize)
    ms = statistics.median(ts)
    line = {"op": args.op, "ms": ms, "steps": args.steps, "log2_bits": args.log2_bits}
    if alg is not None:
        line.update({"algorithmic_bytes": alg, "GB/s": alg / (ms * 1e-3) / 1e9,
                     "frac_of_hbm": alg / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]})
    print(json.dumps(line), flush=True)


def run_gather_sweep(args):
    """torchrun only (`--op gather_sweep`): the replicated result of the 16384^3 GEMM over peer memory, timed for
    row blocks x SMs the GEMM leaves free x gather CTAs per peer (CUDA events over 5 back-to-back calls, max
    over ranks), beside the NCCL form and its parts. One JSON line from rank 0."""
    import torch
    import torch.distributed as dist
    world, rank, local_rank = int(os.environ["WORLD_SIZE"]), int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    import brute_b200  # noqa: F401
    from brute_b200 import kernels as bk
    ops = torch.ops.brute
    size = args.size
    kp = size // 64
    g = torch.Generator(device=dev).manual_seed(1234)
    A = torch.randint(-2 ** 63, 2 ** 63 - 1, (size, kp), generator=g, dtype=torch.int64, device=dev)
    B = torch.randint(-2 ** 63, 2 ** 63 - 1, (size, kp), generator=g, dtype=torch.int64, device=dev)
    lo, hi = bk.shard_bounds(size, world, rank)
    Bl = B[lo:hi].contiguous()

    def timeit(fn, n=5, w=2):
        for _ in range(w):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return round(float(t), 4)

    res = {"world": world, "size": size}
    res["gemm_ms"] = timeit(lambda: ops.xnor_popcount_matmul(A, Bl, size))
    c = ops.xnor_popcount_matmul(A, Bl, size)
    s16 = ops.narrow_i32_i16(c)
    st16 = torch.empty((world, size, hi - lo), dtype=torch.int16, device=dev)
    res["narrow_ms"] = timeit(lambda: ops.narrow_i32_i16(c))
    res["nccl_all_gather_int16_ms"] = timeit(lambda: dist.all_gather_into_tensor(st16.view(world * size, hi - lo).view(torch.uint8), s16.view(torch.uint8)))
    out = torch.empty((size, size), dtype=torch.int32, device=dev)
    res["unstack_ms"] = timeit(lambda: ops.unstack_rank_blocks(st16, out, 0))
    del st16, out, s16, c
    ref = bk._gather_row_blocks(A, Bl, size, world, None, None)
    res["nccl_form_ms"] = timeit(lambda: bk._gather_row_blocks(A, Bl, size, world, None, None))
    got = bk._gather_peer_blocks(A, Bl, size, world, rank, None, None)
    if got is None:
        res["peer"] = "unavailable"
    else:
        res["peer_equals_nccl_form"] = bool(torch.equal(ref, got))
        res["peer_default_ms"] = timeit(lambda: bk._gather_peer_blocks(A, Bl, size, world, rank, None, None))
        sweep = {}
        leaves = (32, 48) if world == 2 else (24, 32, 40, 48, 56, 64)
        for nb in (2, 4, 8):
            for leave in leaves:
                # around one gather CTA per SM left free (2 GPUs: the one peer takes many more)
                for cpp in ((16, 32) if world == 2 else sorted({max(2, leave // world + d) for d in (-1, 0, 1)})):
                    sweep[f"blocks{nb}_leave{leave}_ctas{cpp}"] = timeit(
                        lambda nb=nb, leave=leave, cpp=cpp: bk._gather_peer_blocks(A, Bl, size, world, rank, None, nb, leave, cpp))
        res["peer_sweep_ms"] = sweep
        res["peer_wait_status"] = bk.peer_gather_status()
    if rank == 0:
        print(json.dumps(res), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.op == "gather_sweep":
        run_gather_sweep(args)
    elif args.op != "gemm":
        run_single_op(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
