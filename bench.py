"""Benchmark of the quantized-Linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N --steps K --warmup W

Workload (config.workload): benchmark configuration 5 -- the DiT Linears K/N = 5120/5120 (attention projection),
5120/13824 (FFN up) and 13824/5120 (FFN down) at M = 31x45x80 = 111600 token rows, each as NVFP4 (native fp4
activations) and as W4A8, the token rows SHARDED over the N ranks of the launch with replicated weights and no
collective on the data path (strong scaling: the total work is fixed). Weights ~N(0,0.02) packed by the library's own
packers, activations bf16 ~N(0,1) with 0.1 % outliers x20, seed 4. A step is one pass over the six Linears through
LinearRunner.forward on the rank's rows: quantizer + GEMM for NVFP4, weight expansion + quantizer + GEMM for W4A8
(15 launches).

value      whole-job TFLOP/s (2*M*N*K summed over the six Linears, M the full 111600) with inputs resident in HBM,
           K steps between CUDA events, max over ranks. Every operand is far larger than L2 (126 MB).
e2e        the same metric through the same calls with HOST buffers: pinned x -> device, forward, y -> host for every
           Linear of the step, the copies inside the timed region, three streams so that consecutive Linears overlap
           copy-in, compute and copy-out.
linears    per Linear: ms, TFLOP/s, and the fraction of the derived (2x / 4x the measured dense bf16 burst) and of the
           nominal (4.5 / 9 PFLOP/s) tensor peaks per GPU.
roofline   the dominant kernel -- the NVFP4 CTA-pair GEMM at the FFN-up shape -- timed alone; tensor-bound.
column_split   the FFN-up column split: every rank quantizes its rows, ONE all-gather of the quantized activation (run
           as pairwise steps on a communication stream, overlapped with the GEMMs of the blocks already here), each rank
           computes its output columns for all tokens. Reported beside the blocking form, with the collective's own time.
dit_block  (N=1) benchmark configuration 4: one NVFP4 DiT block at 75600 tokens, Linear-path and whole-block ms.
gpu_reference  (N=1) the reference's own LinearRunner (its kernels + cuBLAS, compiled unmodified for sm_100a as the
           test checker) timed on the same Linears on this GPU: reference leg only, never on the product path.
cpu_baseline / --impl reference   the reference's host path (decode to dense fp32, x * W^T) restated in oracle/ and timed
           on all host cores over a bounded row sample of each of the six Linears.
Other modes: --config2, --config3, --block-stack, --case NAME, --extra (see their help).
"""
from __future__ import annotations

import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

# ---- the headline workload: configuration 5
TOKENS = 31 * 45 * 80
SHAPES = (("attn_proj", 5120, 5120), ("ffn_up", 5120, 13824), ("ffn_down", 13824, 5120))  # name, K (in), N (out)
KINDS = ("nvfp4", "w4a8")
SEED5 = 4
WORKLOAD5 = ("config5: NVFP4 and W4A8 DiT Linears K/N 5120/5120, 5120/13824, 13824/5120 at M=111600 tokens, "
             "token-sharded over the ranks, weights replicated, bf16 in/out")
CPU_SAMPLE_ROWS5 = 128
NOMINAL_TFLOPS = {"nvfp4": 9000.0, "w4a8": 4500.0}
PEAK_MULT = {"nvfp4": 4.0, "w4a8": 2.0}  # derived peaks: multiples of the measured dense bf16 burst

# ---- configuration 2 (--config2)
M, N, K = 4096, 5120, 5120
SEED = 1
WORKLOAD = "config2: W4A8 attention projection M=4096 K=N=5120, bf16 in/out, fp32 bias"
METRIC = "quantized_linear_tflops"
UNIT = "TFLOP/s"
CPU_SAMPLE_ROWS = 256


def host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def make_inputs(np, rows, seed, rank=0):
    import oracle
    from helpers import pack_w4a8

    rng = np.random.default_rng(seed)
    w = (0.02 * rng.standard_normal((N, K))).astype(np.float32)
    packed, s_rel, s_ch, book = pack_w4a8(w)
    bias = (0.01 * rng.standard_normal(N)).astype(np.float32)
    if rank:
        rng = np.random.default_rng(seed + 1000 * rank)  # same weights on every rank, its own rows of tokens
    x = rng.standard_normal((rows, K)).astype(np.float32)
    x = np.where(rng.random((rows, K)) < 1e-3, x * 20.0, x).astype(np.float32)
    return dict(packed=packed, s_rel=s_rel, s_ch=s_ch, book=book, bias=bias, x=oracle.to_bf16(x))


class ClockSampler:
    """Samples the SM clock and the throttle reasons of one GPU while the timed region runs: NVML from a thread of this
    process every few milliseconds (a short multi-GPU step lasts tens of milliseconds), `nvidia-smi` as the fallback.
    Reading only: no setting of the GPU is touched."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int, period_ms: int = 5):
        self.index, self.rows, self.proc, self.period_ms = index, [], None, period_ms
        self.stop, self.thread, self.source = threading.Event(), None, None

    def _nvml_loop(self, nv, handle, mx):
        bits = [nv.nvmlClocksThrottleReasonHwSlowdown, nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                nv.nvmlClocksThrottleReasonSwThermalSlowdown, nv.nvmlClocksThrottleReasonSwPowerCap]
        while not self.stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)
                reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                self.rows.append([str(mhz), str(mx)] + ["Active" if reasons & b else "Not Active" for b in bits])
            except Exception:  # noqa: BLE001  (a failed sample is skipped, not fatal)
                pass
            self.stop.wait(self.period_ms / 1e3)

    def __enter__(self):
        try:
            import pynvml as nv

            nv.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[self.index]) if visible and all(v.strip().isdigit() for v in visible.split(",")) else self.index
            handle = nv.nvmlDeviceGetHandleByIndex(phys)
            mx = nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM)
            self.source = "nvml"
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, handle, mx), daemon=True)
            self.thread.start()
            return self
        except Exception:  # noqa: BLE001
            self.source = "nvidia-smi"
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", str(max(self.period_ms, 20))],
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
        self.stop.set()
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        elif self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self):
        mhz, mx, reasons = [], 0, set()
        for r in list(self.rows):
            try:
                mhz.append(float(r[0]))
                mx = max(mx, float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(self.NAMES, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = [m for m in mhz if m >= 0.5 * mx] or mhz
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz), "source": self.source}


def cpu_baseline(np, data, steps=1, warmup=0):
    """Reference host path on a bounded sample: decode W to dense fp32, rotate x, y = x W^T, all host threads."""
    import ctypes as C

    import oracle

    rows = CPU_SAMPLE_ROWS
    x = np.ascontiguousarray(data["x"][:rows])
    y = np.empty((rows, N), np.float32)
    P = lambda a: a.ctypes.data_as(C.c_void_p)  # noqa: E731

    def once():
        oracle.lib.orc_host_dequant_matmul(4, P(x), rows, P(data["packed"]), P(data["s_rel"]), P(data["s_ch"]),
                                           P(data["book"]), 1.0, 16, N, K, P(y))

    for _ in range(warmup):
        once()
    t0 = time.perf_counter()
    for _ in range(steps):
        once()
    dt = (time.perf_counter() - t0) / steps
    return {"value": 2.0 * rows * N * K / dt / 1e12, "unit": UNIT, "cores": oracle.lib.orc_num_threads(),
            "kind": "port", "sample": f"{rows} of {M} rows of the workload, weight decode included, per step",
            "ms_per_sample": dt * 1e3}


def run_reference_config2(args):
    import numpy as np

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    data = make_inputs(np, CPU_SAMPLE_ROWS, SEED)
    base = cpu_baseline(np, data, steps=max(1, args.steps), warmup=min(args.warmup, 2))
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_sample"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "seed": SEED}, "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))




def time_region(torch, fn, iters):
    """CUDA-event time of `iters` calls on the current stream, in milliseconds."""
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(iters):
        fn(i)
    b.record()
    b.synchronize()
    return a.elapsed_time(b)


def run_config2(args):
    import ctypes as C

    import numpy as np
    import torch
    import torch.distributed as dist

    import slopfab_b200 as sfq
    from helpers import bf16_tensor, dev

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peaks = load_peaks()
    data = make_inputs(np, M, SEED, rank)  # every rank owns M rows of the token axis; weights replicated

    # ---- device-resident inputs, rotated so that consecutive steps never find their operands in L2
    ROT = 4  # 4 x (42 MB activations + 13 MB packed weight + 42 MB output) >> 126 MB of L2
    xs = [bf16_tensor(np.roll(data["x"], i, axis=0)) for i in range(ROT)]
    ys = [torch.empty((M, N), dtype=torch.bfloat16, device="cuda") for _ in range(ROT)]
    weights, keep = [], []
    for i in range(ROT):
        t = [dev(data["packed"]), dev(data["s_rel"]), dev(data["s_ch"]), dev(data["book"]), dev(data["bias"])]
        keep.append(t)
        weights.append(sfq.new_weight(format=sfq.W4A8, data=sfq.ptr(t[0]), out_features=N, in_features=K,
                                      block_scale=sfq.ptr(t[1]), weight_scale=sfq.ptr(t[2]), w4_codebook=sfq.ptr(t[3]),
                                      packed_group_size=16, convrot=1, convrot_group=256, bias=sfq.ptr(t[4])))
    runner = sfq.LinearRunner()
    runner.reserve(runner.workspace_bytes(weights[0], M))

    def step(i):
        runner.forward(weights[i % ROT], xs[i % ROT], ys[i % ROT])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()
    with ClockSampler(local) as clocks:
        barrier()
        ms = time_region(torch, step, args.steps)
        barrier()
        # ---- end to end: host buffers, copies inside the timed region
        hx = [torch.from_numpy(np.roll(data["x"], i, axis=0).view(np.int16)).view(torch.bfloat16).pin_memory()
              for i in range(2)]
        hy = [torch.empty((M, N), dtype=torch.bfloat16).pin_memory() for _ in range(2)]

        # Three streams, as a serving loop would run it: copy-in, compute and copy-out of consecutive steps
        # overlap (PCIe is full duplex); every step still moves its own input and its own result.
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        s_comp = torch.cuda.current_stream()
        ev_in = [torch.cuda.Event() for _ in range(ROT)]
        ev_comp = [torch.cuda.Event() for _ in range(ROT)]
        ev_out = [torch.cuda.Event() for _ in range(ROT)]

        def e2e_step(i):
            j = i % ROT
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_comp[j])          # the compute that last read xs[j] is done
                xs[j].copy_(hx[i % 2], non_blocking=True)
                ev_in[j].record(s_in)
            s_comp.wait_event(ev_in[j])
            s_comp.wait_event(ev_out[j])             # the copy-out that last read ys[j] is done
            step(i)
            ev_comp[j].record(s_comp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_comp[j])
                hy[i % 2].copy_(ys[j], non_blocking=True)
                ev_out[j].record(s_out)

        def e2e_region(iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record(s_comp)
            s_in.wait_event(a)
            for i in range(iters):
                e2e_step(i)
            s_comp.wait_stream(s_out)
            s_comp.wait_stream(s_in)
            b.record(s_comp)
            b.synchronize()
            return a.elapsed_time(b)

        e2e_region(3)
        barrier()
        e2e_steps = max(3, min(args.steps, 20))
        e2e_ms = e2e_region(e2e_steps)
        barrier()
        # ---- the dominant kernel alone: int8 GEMM on pre-quantized operands
        q = torch.empty((M, K), dtype=torch.int8, device="cuda")
        rs = torch.empty(M, dtype=torch.float32, device="cuda")
        w8 = [torch.empty((N, K), dtype=torch.int8, device="cuda") for _ in range(ROT)]
        qs = [torch.empty_like(q) for _ in range(ROT)]
        for i in range(ROT):
            t = keep[i]
            sfq.check(sfq.lib.sfq_unpack_w4a8_int8(sfq.ptr(t[0]), sfq.ptr(t[1]), sfq.ptr(t[3]), sfq.ptr(w8[i]), N, K, 16,
                                                   sfq.stream_ptr()))
            sfq.check(sfq.lib.sfq_quantize_int8_token(sfq.ptr(xs[i]), None, sfq.ptr(qs[i]), sfq.ptr(rs), None, M, K, 1,
                                                      sfq.stream_ptr()))
        eps = [sfq.Epilogue(sfq.ptr(rs), sfq.ptr(keep[i][2]), 1.0, sfq.ptr(keep[i][4]), sfq.F32, sfq.ACT_NONE)
               for i in range(ROT)]

        def gemm_only(i):
            j = i % ROT
            sfq.check(sfq.lib.sfq_gemm_int8(sfq.ptr(qs[j]), sfq.ptr(w8[j]), C.byref(eps[j]), sfq.ptr(ys[j]), M, N, K,
                                            sfq.stream_ptr()))

        def quant_only(i):
            j = i % ROT
            sfq.check(sfq.lib.sfq_quantize_int8_token(sfq.ptr(xs[j]), None, sfq.ptr(qs[j]), sfq.ptr(rs), None, M, K, 1,
                                                      sfq.stream_ptr()))

        def unpack_only(i):
            j = i % ROT
            t = keep[j]
            sfq.check(sfq.lib.sfq_unpack_w4a8_int8(sfq.ptr(t[0]), sfq.ptr(t[1]), sfq.ptr(t[3]), sfq.ptr(w8[j]), N, K, 16,
                                                   sfq.stream_ptr()))

        kern = {}
        for name, fn in (("gemm_int8", gemm_only), ("quantize_int8_token", quant_only), ("unpack_w4a8", unpack_only)):
            for i in range(3):
                fn(i)
            torch.cuda.synchronize()
            kern[name] = time_region(torch, fn, max(args.steps, 10)) / max(args.steps, 10)
        barrier()
    status = sfq.device_status()

    times = torch.tensor([ms, e2e_ms / e2e_steps], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_max, e2e_ms_step = times[0].item(), times[1].item()
    flops_step = 2.0 * M * N * K
    value = world * flops_step * args.steps / (ms_max * 1e-3) / 1e12
    e2e_value = world * flops_step / (e2e_ms_step * 1e-3) / 1e12

    if rank == 0:
        int8_peak = 2.0 * peaks["bf16_tflops"]
        gemm_tflops = flops_step / (kern["gemm_int8"] * 1e-3) / 1e12
        quant_bytes = 2.0 * M * K + M * K + 4.0 * M
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_max / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": WORKLOAD, "seed": SEED, "rows_per_gpu": M,
                       "l2": f"inputs rotate over {ROT} distinct buffer sets (~{ROT * 97} MB) larger than the 126 MB L2",
                       "parallelism": f"token-sharded x{world}, weights replicated, no collective"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 2 * M * K, "d2h_bytes_per_step": 2 * M * N,
                    "ms_per_step": e2e_ms_step},
            "gpu_launches": 3 * args.steps,
            "clocks": clocks.summary(),
            "roofline": {"bound": "tensor", "kernel": "gemm_pair_kernel<int8> (CTA pair, 256x256 tile)", "achieved": gemm_tflops,
                         "peak": int8_peak, "unit": "TFLOP/s", "frac": gemm_tflops / int8_peak, "traffic": profile_value("bench_config2_w4a8_launch_list.md", "dram_bytes_per_launch"),
                         "traffic_note": "dram__bytes_read.sum + dram__bytes_write.sum of one launch of this GEMM on cold "
                                         "operands (ncu, profiles/bench_config2_w4a8_launch_list.md); algorithmic bytes "
                                         f"{M * K + N * K + 2 * M * N}; part of the 42 MB output is still in L2 when the kernel ends",
                         "peak_note": f"2 x {peaks['source']} dense bf16 burst ({peaks['bf16_tflops']} TFLOP/s); "
                                      "nominal dense int8 is 4500",
                         "ms_per_launch": kern["gemm_int8"]},
            "kernels_ms": kern,
            "streaming": {"quantize_int8_token_GBps": quant_bytes / (kern["quantize_int8_token"] * 1e-3) / 1e9,
                          "unpack_w4a8_GBps": (N * K / 2 + N * K / 16 + N * K) / (kern["unpack_w4a8"] * 1e-3) / 1e9,
                          "hbm_peak_GBps": peaks["hbm_gbs"], "peak_source": peaks["source"]},
            "device_status": status,
        }
        if world == 1:
            line["cpu_baseline"] = cpu_baseline(np, data, steps=2, warmup=1)
        if args.extra and world == 1:
            del xs, ys, w8, qs
            torch.cuda.empty_cache()
            line["extra"] = extra_measurements(torch, np, sfq, peaks)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def extra_measurements(torch, np, sfq, peaks):
    """GEMM-only throughput at the other DiT shapes (random operands, GEMM timed alone)."""
    import ctypes as C

    out = {}
    shapes = [("attn_proj_M4096", 4096, 5120, 5120), ("ffn_up_M32760", 32760, 13824, 5120),
              ("ffn_down_M32760", 32760, 5120, 13824), ("attn_proj_M32760", 32760, 5120, 5120)]
    for name, m, n, k in shapes:
        a8 = torch.randint(-128, 128, (m, k), dtype=torch.int8, device="cuda")
        w8 = torch.randint(-127, 128, (n, k), dtype=torch.int8, device="cuda")
        rs = torch.rand(m, device="cuda") * 0.01
        cs = torch.rand(n, device="cuda") * 0.01
        y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        ep = sfq.Epilogue(sfq.ptr(rs), sfq.ptr(cs), 1.0, None, sfq.F32, sfq.ACT_NONE)
        fn = lambda i: sfq.check(sfq.lib.sfq_gemm_int8(sfq.ptr(a8), sfq.ptr(w8), C.byref(ep), sfq.ptr(y), m, n, k,  # noqa: E731
                                                       sfq.stream_ptr()))
        # nvfp4 at the same shape: random nibbles, scales near 1
        aq = torch.randint(0, 256, (m, k // 2), dtype=torch.uint8, device="cuda")
        wq = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda")
        asf = torch.randint(0x30, 0x40, (sfq.lib.sfq_nvfp4_act_scale_bytes(m, k),), dtype=torch.uint8, device="cuda")
        wsf = torch.randint(0x30, 0x40, (n * k // 16,), dtype=torch.uint8, device="cuda")
        ep4 = sfq.Epilogue(None, None, 1e-3, None, sfq.F32, sfq.ACT_NONE)
        fn4 = lambda i: sfq.check(sfq.lib.sfq_gemm_nvfp4(sfq.ptr(aq), sfq.ptr(asf), sfq.ptr(wq), sfq.ptr(wsf),  # noqa: E731
                                                         C.byref(ep4), sfq.ptr(y), m, n, k, sfq.stream_ptr()))
        reps = 20 if m <= 4096 else 5
        for tile_n in (0, 256):  # 0 = default (CTA pairs on 256x256 tiles), 256 = one CTA per 128x256 tile
            sfq.lib.sfq_test_gemm_variant(tile_n, 0, 0)
            for kind, f, mult in (("int8", fn, 2), ("nvfp4", fn4, 4)):
                for i in range(2):
                    f(i)
                torch.cuda.synchronize()
                ms = time_region(torch, f, reps) / reps
                tf = 2.0 * m * n * k / ms / 1e9
                out[f"{kind}_{name}_{'pair' if tile_n == 0 else 'bn%d' % tile_n}"] = {"ms": round(ms, 4), "tflops": round(tf, 1),
                                                    f"frac_of_{mult}x_bf16": round(tf / (mult * peaks["bf16_tflops"]), 3)}
        sfq.lib.sfq_test_gemm_variant(0, 0, 0)
        del a8, w8, aq, wq, asf, wsf, y
        torch.cuda.empty_cache()
    out["device_status"] = sfq.device_status()
    return out


def run_case(name, band=0):
    """One kernel, three launches, on operands larger than L2: the target of an ncu capture. `band` (GEMM cases): row
    tiles of 128 per raster band, through the stand-alone GEMMs' test hook (0 = the kernels' default)."""
    import ctypes as C

    import torch

    import slopfab_b200 as sfq

    torch.cuda.set_device(0)
    sfq.lib.sfq_test_gemm_variant(0, band, 0)
    m, n, k = 16384, 5120, 5120
    reps = 3
    y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    if name == "gemm_int8":
        a8 = torch.randint(-128, 128, (m, k), dtype=torch.int8, device="cuda")
        w8 = torch.randint(-127, 128, (n, k), dtype=torch.int8, device="cuda")
        rs, cs = torch.rand(m, device="cuda") * 0.01, torch.rand(n, device="cuda") * 0.01
        ep = sfq.Epilogue(sfq.ptr(rs), sfq.ptr(cs), 1.0, None, sfq.F32, sfq.ACT_NONE)
        fn = lambda i: sfq.check(sfq.lib.sfq_gemm_int8(sfq.ptr(a8), sfq.ptr(w8), C.byref(ep), sfq.ptr(y), m, n, k,  # noqa: E731
                                                       sfq.stream_ptr()))
        work = 2.0 * m * n * k
    elif name in ("gemm_w4a8_fused", "gemm_w4a8_unpack_then_gemm"):
        # W4A8 Linear at M rows (env SFQ_W4_ROWS, default 16384), weight in storage form: the int8 rows produced inside the GEMM,
        # against the stand-alone expansion into a dense copy followed by the int8 GEMM (what `forward` does without `prepare`)
        m = int(os.environ.get("SFQ_W4_ROWS", "16384"))
        y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        a8 = torch.randint(-128, 128, (m, k), dtype=torch.int8, device="cuda")
        packed = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda")
        gs = torch.randint(0x28, 0x39, (n * k // 16,), dtype=torch.uint8, device="cuda")
        book = (torch.arange(16, dtype=torch.float32, device="cuda") - 8.0)
        w8 = torch.empty((n, k), dtype=torch.int8, device="cuda")
        rs, cs = torch.rand(m, device="cuda") * 0.01, torch.rand(n, device="cuda") * 0.01
        ep = sfq.Epilogue(sfq.ptr(rs), sfq.ptr(cs), 1.0, None, sfq.F32, sfq.ACT_NONE)
        if name == "gemm_w4a8_fused":
            fn = lambda i: sfq.check(sfq.lib.sfq_gemm_w4a8_fused(sfq.ptr(a8), sfq.ptr(packed), sfq.ptr(gs), sfq.ptr(book), C.byref(ep),  # noqa: E731
                                                                 sfq.ptr(y), m, n, k, sfq.stream_ptr()))
        else:
            def fn(i):
                sfq.check(sfq.lib.sfq_unpack_w4a8_int8(sfq.ptr(packed), sfq.ptr(gs), sfq.ptr(book), sfq.ptr(w8), n, k, 16, sfq.stream_ptr()))
                sfq.check(sfq.lib.sfq_gemm_int8(sfq.ptr(a8), sfq.ptr(w8), C.byref(ep), sfq.ptr(y), m, n, k, sfq.stream_ptr()))
        work = 2.0 * m * n * k
        reps = 10
    elif name == "gemm_int8_c2":
        # the benchmark's own GEMM (config 2) on four rotating operand sets, so that a captured launch reads cold data
        m, reps = 4096, 7
        sets = []
        for _ in range(4):
            sets.append((torch.randint(-128, 128, (m, k), dtype=torch.int8, device="cuda"),
                         torch.randint(-127, 128, (n, k), dtype=torch.int8, device="cuda"),
                         torch.empty((m, n), dtype=torch.bfloat16, device="cuda")))
        rs, cs = torch.rand(m, device="cuda") * 0.01, torch.rand(n, device="cuda") * 0.01
        ep = sfq.Epilogue(sfq.ptr(rs), sfq.ptr(cs), 1.0, None, sfq.F32, sfq.ACT_NONE)
        fn = lambda i: sfq.check(sfq.lib.sfq_gemm_int8(sfq.ptr(sets[i % 4][0]), sfq.ptr(sets[i % 4][1]), C.byref(ep),  # noqa: E731
                                                       sfq.ptr(sets[i % 4][2]), m, n, k, sfq.stream_ptr()))
        work = 2.0 * m * n * k
    elif name == "gemm_nvfp4":
        aq = torch.randint(0, 256, (m, k // 2), dtype=torch.uint8, device="cuda")
        wq = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda")
        asf = torch.randint(0x30, 0x40, (sfq.lib.sfq_nvfp4_act_scale_bytes(m, k),), dtype=torch.uint8, device="cuda")
        wsf = torch.randint(0x30, 0x40, (n * k // 16,), dtype=torch.uint8, device="cuda")
        ep = sfq.Epilogue(None, None, 1e-3, None, sfq.F32, sfq.ACT_NONE)
        fn = lambda i: sfq.check(sfq.lib.sfq_gemm_nvfp4(sfq.ptr(aq), sfq.ptr(asf), sfq.ptr(wq), sfq.ptr(wsf),  # noqa: E731
                                                        C.byref(ep), sfq.ptr(y), m, n, k, sfq.stream_ptr()))
        work = 2.0 * m * n * k
    elif name == "gemm_nvfp4_ffn_up":
        # the benchmark's dominant kernel at a quarter of its rows (27900 x 5120 -> 13824): 0.9 GB on the device
        m, n = TOKENS // 4, 13824
        y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        aq = torch.randint(0, 256, (m, k // 2), dtype=torch.uint8, device="cuda")
        wq = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda")
        asf = torch.randint(0x30, 0x40, (sfq.lib.sfq_nvfp4_act_scale_bytes(m, k),), dtype=torch.uint8, device="cuda")
        wsf = torch.randint(0x30, 0x40, (n * k // 16,), dtype=torch.uint8, device="cuda")
        ep = sfq.Epilogue(None, None, 1e-3, None, sfq.F32, sfq.ACT_NONE)
        fn = lambda i: sfq.check(sfq.lib.sfq_gemm_nvfp4(sfq.ptr(aq), sfq.ptr(asf), sfq.ptr(wq), sfq.ptr(wsf),  # noqa: E731
                                                        C.byref(ep), sfq.ptr(y), m, n, k, sfq.stream_ptr()))
        work = 2.0 * m * n * k
    elif name == "unpack_w4a8":
        n = 13824
        packed = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda").view(torch.int8)
        s_rel = torch.randint(0x28, 0x39, (n * k // 16,), dtype=torch.uint8, device="cuda")
        book = torch.arange(16, dtype=torch.float32, device="cuda") - 8.0
        outs = [torch.empty((n, k), dtype=torch.int8, device="cuda") for _ in range(3)]
        fn = lambda i: sfq.check(sfq.lib.sfq_unpack_w4a8_int8(sfq.ptr(packed), sfq.ptr(s_rel), sfq.ptr(book), sfq.ptr(outs[i % 3]), n, k,  # noqa: E731
                                                              16, sfq.stream_ptr()))
        work = n * k / 2 + n * k / 16 + n * k
    elif name in ("quantize_int8", "quantize_nvfp4", "quantize_int8_k13824"):
        m = 32768
        if name == "quantize_int8_k13824":  # the FFN-down input of config 3
            m, k, name = 16384, 13824, "quantize_int8"
        x = torch.randn((m, k), device="cuda").to(torch.bfloat16)
        q = torch.empty((m, k), dtype=torch.int8, device="cuda")
        rs = torch.empty(m, device="cuda")
        sc = torch.empty(sfq.lib.sfq_nvfp4_act_scale_bytes(m, k), dtype=torch.uint8, device="cuda")
        if name == "quantize_int8":
            fn = lambda i: sfq.check(sfq.lib.sfq_quantize_int8_token(sfq.ptr(x), None, sfq.ptr(q), sfq.ptr(rs), None, m, k,  # noqa: E731
                                                                     1, sfq.stream_ptr()))
            work = 3.0 * m * k + 4 * m
        else:
            fn = lambda i: sfq.check(sfq.lib.sfq_quantize_nvfp4_block(sfq.ptr(x), None, sfq.ptr(q), sfq.ptr(sc), None, m,  # noqa: E731
                                                                      k, sfq.NVFP4_ACT_GEMM_FEED, sfq.stream_ptr()))
            work = 2.0 * m * k + m * k / 2 + m * k / 16
    elif name in ("attention", "attention_torch"):
        # a quarter of configuration 4's sequence (75600 / 4 tokens), its 40 heads of 128; Gaussian q, k, v
        seq, heads = int(os.environ.get("SFQ_ATTN_SEQ", "18900")), 40
        g = torch.Generator(device="cuda").manual_seed(7)
        qkv = torch.randn((seq, 3 * heads * 128), device="cuda", generator=g).to(torch.bfloat16)
        w = heads * 128
        q, kk, v = qkv[:, :w], qkv[:, w:2 * w], qkv[:, 2 * w:]
        out = torch.empty((seq, w), dtype=torch.bfloat16, device="cuda")
        work = 4.0 * seq * seq * 128 * heads
        if name == "attention":
            nbytes = C.c_size_t()
            sfq.check(sfq.lib.sfq_attention_workspace_bytes(seq, heads, 128, C.byref(nbytes)))
            ws = torch.empty(nbytes.value, dtype=torch.uint8, device="cuda")
            fn = lambda i: sfq.check(sfq.lib.sfq_attention_forward(q.data_ptr(), 3 * w, kk.data_ptr(), v.data_ptr(), 3 * w, out.data_ptr(), w,  # noqa: E731
                                                                   seq, seq, heads, heads, 128, 0.0, ws.data_ptr(), nbytes.value,
                                                                   sfq.stream_ptr()))
        else:  # the library kernel on the same tensors, for the comparison line only
            sh = lambda t: t.reshape(1, seq, heads, 128).transpose(1, 2)  # noqa: E731  [1, heads, seq, 128] views, no copy
            fn = lambda i: torch.nn.functional.scaled_dot_product_attention(sh(q), sh(kk), sh(v))  # noqa: E731
    else:
        raise SystemExit("unknown case " + name)
    fn(0)
    torch.cuda.synchronize()
    reps = int(os.environ.get("SFQ_CASE_REPS", reps))
    with ClockSampler(0) as clocks:
        ms = time_region(torch, fn, reps) / reps
    print(json.dumps({"case": name, "band": band, "ms_per_launch": ms, "work_per_second": work / (ms * 1e-3), "clocks": clocks.summary(),
                      "device_status": sfq.device_status()}))


def run_block_stack(blocks=40, rows=75600, hidden=5120, heads=40, ffn=13824):
    """benchmark configuration 4: NVFP4 DiT block stack, random init, 21x45x80 = 75600 tokens. Reports the Linear-path
    milliseconds (norm+quant, GEMMs, gated residuals) and the whole-block milliseconds, attention included (this library's
    tcgen05 kernel on the thirds of the fused projection)."""
    import torch

    from slopfab_b200.block import BlockWeights, Nvfp4Block, Nvfp4Linear
    import slopfab_b200 as sfq

    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn((rows, hidden), device="cuda", generator=g).to(torch.bfloat16)
    names = ["scale_msa", "shift_msa", "gate_msa", "scale_mlp", "shift_mlp", "gate_mlp"]
    mod = {n: 0.1 * torch.randn((3, hidden), device="cuda", generator=g) for n in names}
    index = torch.zeros(rows, dtype=torch.int32, device="cuda")  # all video rows: tag 0 of timestep 0
    ones = torch.ones(hidden, dtype=torch.bfloat16, device="cuda")
    ws = [BlockWeights(Nvfp4Linear.random(3 * hidden, hidden, seed=4 * b), Nvfp4Linear.random(hidden, hidden, seed=4 * b + 1),
                       Nvfp4Linear.random(ffn, hidden, seed=4 * b + 2), Nvfp4Linear.random(hidden, ffn, seed=4 * b + 3),
                       ones, ones) for b in range(blocks)]
    blk = Nvfp4Block(rows, hidden, heads, ffn)
    blk.forward(x.clone(), ws[0], mod, index)  # warm-up
    torch.cuda.synchronize()
    blk.linear_ms = 0.0
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for w in ws:
        blk.forward(x, w, mod, index, time_linears=True)
    b.record()
    b.synchronize()
    total = a.elapsed_time(b)
    flops_linear = 2.0 * rows * hidden * (3 * hidden + hidden + 2 * ffn)
    print(json.dumps({"case": "config4_block_stack", "blocks": blocks, "tokens": rows, "block_ms": total / blocks,
                      "linear_path_ms_per_block": blk.linear_ms / blocks,
                      "linear_path_tflops": flops_linear / (blk.linear_ms / blocks * 1e-3) / 1e12,
                      "attention": "attention_kernel of this library (bf16 tcgen05, head_dim 128)",
                      "attention_ms_per_block": (total - blk.linear_ms) / blocks,
                      "attention_tflops": 4.0 * rows * rows * hidden / ((total - blk.linear_ms) / blocks * 1e-3) / 1e12,
                      "finite": bool(torch.isfinite(x.float()).all().item()), "device_status": sfq.device_status()}))


def run_config3(rows=32760, hidden=5120, ffn=13824, group=64, reps=5):
    """benchmark configuration 3: W6A8 FFN pair at 32760 tokens through the runner: prepare() once per layer (the int8
    expansion), then up-projection with GELU-tanh in the epilogue and down-projection, as a DiT chunk loop does."""
    import torch

    import slopfab_b200 as sfq

    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda").manual_seed(2)

    def w6(n, k):
        packed = torch.randint(0, 256, (n, k * 3 // 4), dtype=torch.uint8, device="cuda", generator=g).view(torch.int8)
        s_rel = torch.randint(0x28, 0x39, (n * k // group,), dtype=torch.uint8, device="cuda", generator=g)
        s_ch = (torch.rand(n, device="cuda", generator=g) + 1.0) * 2.0 ** -8
        return (packed, s_rel, s_ch), sfq.new_weight(format=sfq.W6A8, data=sfq.ptr(packed), out_features=n, in_features=k,
                                                     block_scale=sfq.ptr(s_rel), weight_scale=sfq.ptr(s_ch),
                                                     packed_group_size=group, convrot=1, convrot_group=256)

    keep_up, w_up = w6(ffn, hidden)
    keep_dn, w_dn = w6(hidden, ffn)
    x = torch.randn((rows, hidden), device="cuda", generator=g).to(torch.bfloat16)
    h = torch.empty((rows, ffn), dtype=torch.bfloat16, device="cuda")
    y = torch.empty((rows, hidden), dtype=torch.bfloat16, device="cuda")
    up, dn = sfq.LinearRunner(), sfq.LinearRunner()
    up.set_activation(sfq.ACT_GELU_TANH)
    up.reserve(up.workspace_bytes(w_up, rows))
    dn.reserve(dn.workspace_bytes(w_dn, rows))
    p_up, used_up = up.prepare(w_up, rows)
    p_dn, used_dn = dn.prepare(w_dn, rows)

    def pair(i):
        up.forward_prepared(w_up, p_up, used_up, x, h)
        dn.forward_prepared(w_dn, p_dn, used_dn, h, y)

    pair(0)
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    t_up = t_dn = 0.0
    for _ in range(reps):
        ev[0].record()
        up.forward_prepared(w_up, p_up, used_up, x, h)
        ev[1].record()
        dn.forward_prepared(w_dn, p_dn, used_dn, h, y)
        ev[2].record()
        ev[2].synchronize()
        t_up += ev[0].elapsed_time(ev[1]) / reps
        t_dn += ev[1].elapsed_time(ev[2]) / reps
    flops = 2.0 * rows * hidden * ffn
    print(json.dumps({"case": "config3_w6a8_ffn_pair", "tokens": rows, "up_ms": t_up, "down_ms": t_dn,
                      "up_tflops": flops / (t_up * 1e-3) / 1e12, "down_tflops": flops / (t_dn * 1e-3) / 1e12,
                      "pair_tflops": 2 * flops / ((t_up + t_dn) * 1e-3) / 1e12,
                      "note": "each projection = fused ConvRot + int8 quantizer + int8 GEMM with fused epilogue; "
                              "the W6 -> int8 expansion is done once by prepare() and not in these times",
                      "finite": bool(torch.isfinite(y.float()).all().item()), "device_status": sfq.device_status()}))


def profile_value(filename, key):
    """A `key = <integer>` line of a summary under profiles/ (the figures an ncu capture gave), or None."""
    path = os.path.join(ROOT, "profiles", filename)
    if not os.path.exists(path):
        return None
    m = re.search(r"^\s*" + re.escape(key) + r"\s*=\s*(\d+)", open(path).read(), re.M)
    return int(m.group(1)) if m else None


def set_pack_threads(n):
    """The host packers run under OpenMP; a launcher that exports OMP_NUM_THREADS=1 would make them crawl."""
    import ctypes as C

    try:
        C.CDLL("libgomp.so.1").omp_set_num_threads(int(n))
    except OSError:
        pass


def config5_weights_host(torch, np):
    """The three weights ~N(0, 0.02), seed 4, in both storage forms, packed on the host by the library's packers.
    The same bytes serve both arms of the benchmark."""
    from helpers import pack_nvfp4, pack_w4a8

    out = {}
    for i, (name, k, n) in enumerate(SHAPES):
        g = torch.Generator().manual_seed(SEED5 * 100 + i)
        w = (0.02 * torch.randn((n, k), generator=g)).numpy()
        data, scale, gs = pack_nvfp4(w)
        packed, s_rel, s_ch, book = pack_w4a8(w)
        out[name] = {"nvfp4": (data, scale, np.float32(gs)), "w4a8": (packed, s_rel, s_ch, book)}
    return out


def config5_activation(torch, rows, k, seed, device):
    """bf16 ~N(0,1) with 0.1 % of the elements x20 (the distribution of configurations 1-2)."""
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn((rows, k), device=device, generator=g)
    x = torch.where(torch.rand((rows, k), device=device, generator=g) < 1e-3, x * 20.0, x)
    return x.to(torch.bfloat16)


def cpu_baseline5(np, torch, weights, steps=1, warmup=0):
    """Reference host path on a bounded sample of every Linear of the step: decode W to dense fp32 (rotate x for W4A8),
    y = x W^T, all host threads."""
    import ctypes as C

    import oracle

    oracle.lib.orc_set_num_threads(host_threads())
    rows = CPU_SAMPLE_ROWS5
    P = lambda a: a.ctypes.data_as(C.c_void_p)  # noqa: E731
    xs = {}
    for k in (5120, 13824):
        x = config5_activation(torch, rows, k, SEED5 + 7, "cpu")
        xs[k] = np.ascontiguousarray(x.view(torch.int16).numpy().view(np.uint16))
    ys = {n: np.empty((rows, n), np.float32) for n in (5120, 13824)}

    def once():
        for name, k, n in SHAPES:
            data, scale, gs = weights[name]["nvfp4"]
            oracle.lib.orc_host_dequant_matmul(0, P(xs[k]), rows, P(data), P(scale), None, None, float(gs), 16, n, k, P(ys[n]))
            packed, s_rel, s_ch, book = weights[name]["w4a8"]
            oracle.lib.orc_host_dequant_matmul(4, P(xs[k]), rows, P(packed), P(s_rel), P(s_ch), P(book), 1.0, 16, n, k, P(ys[n]))

    for _ in range(warmup):
        once()
    t0 = time.perf_counter()
    for _ in range(steps):
        once()
    dt = (time.perf_counter() - t0) / steps
    flops = sum(2.0 * rows * n * k for _, k, n in SHAPES) * len(KINDS)
    return {"value": flops / dt / 1e12, "unit": UNIT, "cores": oracle.lib.orc_num_threads(), "kind": "port",
            "sample": f"{rows} of {TOKENS} rows of each of the six Linears, weight decode included, per step",
            "ms_per_sample": dt * 1e3}


def gpu_reference5(torch, weights_dev, xs, rows, iters=3):
    """The reference's own LinearRunner (unmodified sources compiled for sm_100a under oracle/_ref: dequantize + cuBLAS
    bf16 for NVFP4, its six-launch integer path + cuBLAS int8 for W4A8) timed on the same Linears and rows on this GPU.
    Reference leg only. Returns {linear: {kind: ms}} or a reason string."""
    import ctypes as C

    import slopfab_b200 as sfq
    from helpers import ref_dev, ref_weight_from

    ref = ref_dev()
    if ref is None:
        return "oracle/_ref was not built (the reference tree was absent at build time)"
    out = {}
    for name, k, n in SHAPES:
        y = torch.empty((rows, n), dtype=torch.bfloat16, device="cuda")
        out[name] = {}
        for kind in KINDS:
            rw = ref_weight_from(weights_dev[name][kind][0])
            ms = C.c_float(0.0)
            rc = ref.ref_dev_linear_forward(C.byref(rw), sfq.ptr(xs[k]), rows, sfq.ptr(y), 0, iters, C.byref(ms))
            if rc != 0:
                return "the reference's LinearRunner failed: " + ref.ref_last_error().decode("utf-8", "replace")
            out[name][kind] = ms.value
        del y
    return out


def run_reference(args):
    """--impl reference: the reference's CPU implementation of the path on this box's host cores, rank 0 only."""
    import numpy as np
    import torch

    if int(os.environ.get("RANK", "0")) != 0:
        return
    set_pack_threads(host_threads())
    weights = config5_weights_host(torch, np)
    base = cpu_baseline5(np, torch, weights, steps=max(1, args.steps), warmup=min(max(args.warmup, 0), 2))
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_sample"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD5, "seed": SEED5}, "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def dit_block_ms(torch, sfq, blocks=2, rows=75600, hidden=5120, heads=40, ffn=13824):
    """Configuration 4 on one GPU: `blocks` NVFP4 DiT blocks at 75600 tokens after one warm-up block."""
    from slopfab_b200.block import BlockWeights, Nvfp4Block, Nvfp4Linear

    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn((rows, hidden), device="cuda", generator=g).to(torch.bfloat16)
    names = ["scale_msa", "shift_msa", "gate_msa", "scale_mlp", "shift_mlp", "gate_mlp"]
    mod = {n: 0.1 * torch.randn((3, hidden), device="cuda", generator=g) for n in names}
    index = torch.zeros(rows, dtype=torch.int32, device="cuda")
    ones = torch.ones(hidden, dtype=torch.bfloat16, device="cuda")
    ws = [BlockWeights(Nvfp4Linear.random(3 * hidden, hidden, seed=4 * b), Nvfp4Linear.random(hidden, hidden, seed=4 * b + 1),
                       Nvfp4Linear.random(ffn, hidden, seed=4 * b + 2), Nvfp4Linear.random(hidden, ffn, seed=4 * b + 3), ones, ones)
          for b in range(blocks)]
    blk = Nvfp4Block(rows, hidden, heads, ffn)
    blk.forward(x.clone(), ws[0], mod, index)
    torch.cuda.synchronize()
    blk.linear_ms = 0.0
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for w in ws:
        blk.forward(x, w, mod, index, time_linears=True)
    b.record()
    b.synchronize()
    total = a.elapsed_time(b)
    flops_linear = 2.0 * rows * hidden * (3 * hidden + hidden + 2 * ffn)
    out = {"workload": "config4: one NVFP4 DiT block, 75600 tokens, hidden 5120, 40 heads x128, FFN 13824 (GELU), adaLN-modulated "
                       "RMSNorm, attention in bf16 (this library's tcgen05 kernel)",
           "blocks_timed": blocks, "block_ms": total / blocks, "linear_path_ms": blk.linear_ms / blocks,
           "linear_path_tflops": flops_linear / (blk.linear_ms / blocks * 1e-3) / 1e12,
           "attention_ms": (total - blk.linear_ms) / blocks,
           "attention_tflops": 4.0 * rows * rows * hidden / ((total - blk.linear_ms) / blocks * 1e-3) / 1e12,
           "finite": bool(torch.isfinite(x.float()).all().item())}
    del blk, ws, x
    torch.cuda.empty_cache()
    return out


def run_ours(args):
    """The headline run: configuration 5 on the ranks of this launch (see the module docstring)."""
    import ctypes as C

    import numpy as np
    import torch
    import torch.distributed as dist

    import slopfab_b200 as sfq
    from helpers import dev
    from slopfab_b200.parallel import ColumnSplitPlan, column_shard, token_shard

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peaks = load_peaks()
    steps, warmup = max(1, args.steps), max(args.warmup, 3)
    _, m = token_shard(TOKENS, world, rank)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(values):
        t = torch.tensor(values, dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    # ---- weights: packed once on rank 0 by the library's packers, then replicated to every GPU
    host = None
    if rank == 0:
        set_pack_threads(min(host_threads(), 32))
        host = config5_weights_host(torch, np)
    wdev = {}
    for name, k, n in SHAPES:
        sizes = {"nvfp4": [(n, k // 2), (n * k // 16,)], "w4a8": [(n, k // 2), (n * k // 16,), (n,), (16,)]}
        dtypes = {"nvfp4": [torch.uint8, torch.uint8], "w4a8": [torch.int8, torch.uint8, torch.float32, torch.float32]}
        wdev[name] = {}
        for kind in KINDS:
            if rank == 0:
                arrays = host[name][kind][:2] if kind == "nvfp4" else host[name][kind]
                tensors = [dev(np.ascontiguousarray(a)) for a in arrays]
            else:
                tensors = [torch.empty(sh, dtype=dt, device="cuda") for sh, dt in zip(sizes[kind], dtypes[kind])]
            gs = torch.tensor([float(host[name]["nvfp4"][2]) if rank == 0 else 0.0], dtype=torch.float32, device="cuda")
            if world > 1:
                for t in tensors:
                    dist.broadcast(t, 0)
                dist.broadcast(gs, 0)
            if kind == "nvfp4":
                w = sfq.new_weight(format=sfq.NVFP4, data=sfq.ptr(tensors[0]), out_features=n, in_features=k,
                                   block_scale=sfq.ptr(tensors[1]), global_scale=gs.item())
            else:
                w = sfq.new_weight(format=sfq.W4A8, data=sfq.ptr(tensors[0]), out_features=n, in_features=k,
                                   block_scale=sfq.ptr(tensors[1]), weight_scale=sfq.ptr(tensors[2]), w4_codebook=sfq.ptr(tensors[3]),
                                   packed_group_size=16, convrot=1, convrot_group=256)
            wdev[name][kind] = (w, tensors)
    # ---- activations and outputs of this rank's token rows, resident in HBM
    xs = {k: config5_activation(torch, m, k, SEED5 + 1000 * rank + k, "cuda") for k in (5120, 13824)}
    ys = {n: torch.empty((m, n), dtype=torch.bfloat16, device="cuda") for n in (5120, 13824)}
    runners = {"nvfp4": sfq.LinearRunner(), "w4a8": sfq.LinearRunner()}
    runners["nvfp4"].set_native(True)
    for kind in KINDS:
        runners[kind].reserve(max(runners[kind].workspace_bytes(wdev[name][kind][0], m) for name, _, _ in SHAPES))
    calls = [(kind, name, k, n) for kind in KINDS for name, k, n in SHAPES]
    launches_per_step = sum(2 if kind == "nvfp4" else 3 for kind, *_ in calls)
    flops_step = sum(2.0 * TOKENS * n * k for _, _, k, n in calls)  # the whole job's, all ranks together

    def step(_i=0):
        for kind, name, k, n in calls:
            runners[kind].forward(wdev[name][kind][0], xs[k], ys[n])

    for i in range(warmup):
        step(i)
    barrier()
    with ClockSampler(local) as clocks:
        barrier()
        ms = time_region(torch, step, steps)
        barrier()
    ms_max = max_over_ranks([ms])[0]
    value = flops_step * steps / (ms_max * 1e-3) / 1e12

    # ---- per Linear: the same call alone
    table = []
    reps = 8 if world == 1 else 16
    for kind, name, k, n in calls:
        fn = lambda _i, kind=kind, name=name, k=k, n=n: runners[kind].forward(wdev[name][kind][0], xs[k], ys[n])  # noqa: E731
        fn(0)
        barrier()
        t = max_over_ranks([time_region(torch, fn, reps) / reps])[0]
        tf = 2.0 * TOKENS * n * k / (t * 1e-3) / 1e12
        table.append({"linear": name, "kind": kind, "K": k, "N": n, "ms": t, "tflops": tf, "tflops_per_gpu": tf / world,
                      "frac_of_derived_sustained_peak": tf / world / (PEAK_MULT[kind] * peaks["bf16_tflops_sustained"]),
                      "frac_of_derived_burst_peak": tf / world / (PEAK_MULT[kind] * peaks["bf16_tflops"]),
                      "frac_of_nominal_peak": tf / world / NOMINAL_TFLOPS[kind]})

    # ---- every kernel of the step alone, by CUDA events (the shares an ncu launch list must agree with), and the dominant
    #      one -- the NVFP4 CTA-pair GEMM at the FFN-up shape on pre-quantized operands -- for the roofline
    k_up, n_up = 5120, 13824
    kern = {}
    for name, k, n in SHAPES:
        x, y = xs[k], ys[n]
        xq = torch.empty((m, k // 2), dtype=torch.uint8, device="cuda")
        xsf = torch.empty(sfq.lib.sfq_nvfp4_act_scale_bytes(m, k), dtype=torch.uint8, device="cuda")
        q8 = torch.empty((m, k), dtype=torch.int8, device="cuda")
        rs = torch.empty(m, dtype=torch.float32, device="cuda")
        w8 = torch.empty((n, k), dtype=torch.int8, device="cuda")
        w4, t4 = wdev[name]["nvfp4"]
        w8d, t8 = wdev[name]["w4a8"]
        ep4 = sfq.Epilogue(None, None, w4.global_scale, None, sfq.F32, sfq.ACT_NONE)
        ep8 = sfq.Epilogue(sfq.ptr(rs), sfq.ptr(t8[2]), 1.0, None, sfq.F32, sfq.ACT_NONE)
        S = sfq.stream_ptr()
        fns = {
            "quantize_nvfp4": lambda _i: sfq.check(sfq.lib.sfq_quantize_nvfp4_block(sfq.ptr(x), None, sfq.ptr(xq), sfq.ptr(xsf), None, m, k,
                                                                                    sfq.NVFP4_ACT_GEMM_FEED, S)),
            "gemm_nvfp4": lambda _i: sfq.check(sfq.lib.sfq_gemm_nvfp4(sfq.ptr(xq), sfq.ptr(xsf), sfq.ptr(t4[0]), sfq.ptr(t4[1]), C.byref(ep4),
                                                                      sfq.ptr(y), m, n, k, S)),
            "unpack_w4a8": lambda _i: sfq.check(sfq.lib.sfq_unpack_w4a8_int8(sfq.ptr(t8[0]), sfq.ptr(t8[1]), sfq.ptr(t8[3]), sfq.ptr(w8), n, k, 16, S)),
            "quantize_int8": lambda _i: sfq.check(sfq.lib.sfq_quantize_int8_token(sfq.ptr(x), None, sfq.ptr(q8), sfq.ptr(rs), None, m, k, 1, S)),
            "gemm_int8": lambda _i: sfq.check(sfq.lib.sfq_gemm_int8(sfq.ptr(q8), sfq.ptr(w8), C.byref(ep8), sfq.ptr(y), m, n, k, S)),
        }
        kern[name] = {}
        for kname, fn in fns.items():  # in an order that fills every operand before it is read
            for i in range(2):
                fn(i)
            torch.cuda.synchronize()
            kern[name][kname] = time_region(torch, fn, 10) / 10
        del xq, xsf, q8, rs, w8
    gemm_ms = kern["ffn_up"]["gemm_nvfp4"]
    quant_ms = kern["ffn_up"]["quantize_nvfp4"]
    kern_total = sum(v for d_ in kern.values() for v in d_.values())
    shares = {kname: sum(kern[name][kname] for name, _, _ in SHAPES) / kern_total for kname in next(iter(kern.values()))}

    # ---- end to end: host buffers, copies inside the timed region
    e2e = None
    if not args.no_e2e:
        wide = 13824
        hx = {k: torch.empty((m, k), dtype=torch.bfloat16, pin_memory=True) for k in (5120, 13824)}
        for k in hx:
            hx[k].copy_(xs[k])
        hy = [torch.empty((m, wide), dtype=torch.bfloat16, pin_memory=True) for _ in range(2)]
        dxb = [torch.empty((m, wide), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        dyb = [torch.empty((m, wide), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        s_in, s_out, s_comp = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
        ev_in, ev_comp, ev_out = ([torch.cuda.Event() for _ in range(2)] for _ in range(3))

        def e2e_step(_i):
            for j, (kind, name, k, n) in enumerate(calls):
                b = j % 2
                dx = dxb[b].view(-1)[: m * k].view(m, k)
                dy = dyb[b].view(-1)[: m * n].view(m, n)
                with torch.cuda.stream(s_in):
                    s_in.wait_event(ev_comp[b])  # the Linear that last read this input buffer is done
                    dx.copy_(hx[k], non_blocking=True)
                    ev_in[b].record(s_in)
                s_comp.wait_event(ev_in[b])
                s_comp.wait_event(ev_out[b])  # the copy-out that last read this output buffer is done
                runners[kind].forward(wdev[name][kind][0], dx, dy)
                ev_comp[b].record(s_comp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_comp[b])
                    hy[b].view(-1)[: m * n].view(m, n).copy_(dy, non_blocking=True)
                    ev_out[b].record(s_out)

        def e2e_region(iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record(s_comp)
            s_in.wait_event(a)
            for i in range(iters):
                e2e_step(i)
            s_comp.wait_stream(s_out)
            s_comp.wait_stream(s_in)
            b.record(s_comp)
            b.synchronize()
            return a.elapsed_time(b)

        e2e_region(1)
        barrier()
        e2e_steps = max(2, min(steps, 4))
        e2e_ms = max_over_ranks([e2e_region(e2e_steps) / e2e_steps])[0]
        barrier()
        h2d = sum(2 * m * k for _, _, k, _ in calls)
        d2h = sum(2 * m * n for _, _, _, n in calls)
        e2e = {"value": flops_step / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": e2e_ms, "steps": e2e_steps,
               "note": "bytes are this rank's; every rank moves its own rows, all ranks through the one host memory system"}
        del hx, hy, dxb, dyb
        torch.cuda.empty_cache()

    # ---- FFN-up column split with its one all-gather (secondary scheme)
    column = {}
    if TOKENS % world == 0 and not args.no_column_split:
        c0, nl = column_shard(n_up, world, rank)
        for kind in KINDS:
            w, t = wdev["ffn_up"][kind]
            if kind == "w4a8":
                w8 = torch.empty((nl, k_up), dtype=torch.int8, device="cuda")
                sfq.check(sfq.lib.sfq_unpack_w4a8_int8(sfq.ptr(t[0][c0:c0 + nl].contiguous()), sfq.ptr(t[1].view(n_up, -1)[c0:c0 + nl].contiguous()),
                                                       sfq.ptr(t[3]), sfq.ptr(w8), nl, k_up, 16, sfq.stream_ptr()))
                weight = (w8, t[2][c0:c0 + nl].contiguous())
            else:
                weight = (t[0][c0:c0 + nl].contiguous(), t[1].view(n_up // 128, -1)[c0 // 128:(c0 + nl) // 128].contiguous().view(-1),
                          w.global_scale)
            entry = {}
            for pipeline in (("overlap", "blocking") if world > 1 else ("blocking",)):
                plan = ColumnSplitPlan(kind, m, k_up, nl, weight, world, pipeline=pipeline, rank=rank)
                fwd = lambda _i, plan=plan: plan.forward(xs[k_up])  # noqa: E731
                gat = lambda _i, plan=plan: plan.gather_only()  # noqa: E731
                for i in range(2):
                    fwd(i)
                barrier()
                t_all = time_region(torch, fwd, 5) / 5
                barrier()
                t_gather = time_region(torch, gat, 5) / 5 if world > 1 else 0.0
                barrier()
                t_all, t_gather = max_over_ranks([t_all, t_gather])
                tf = 2.0 * TOKENS * n_up * k_up / (t_all * 1e-3) / 1e12
                entry[pipeline] = {"ms": t_all, "tflops": tf, "collective_alone_ms": t_gather,
                                   "gathered_bytes_per_gpu": plan.gathered_bytes}
                del plan
                torch.cuda.empty_cache()
            token = next(r for r in table if r["linear"] == "ffn_up" and r["kind"] == kind)
            best = min(entry, key=lambda p: entry[p]["ms"])
            entry["best"] = best
            entry["vs_token_sharding"] = entry[best]["tflops"] / token["tflops"]
            # what the collective adds on top of quantizer + GEMMs (which cost about what token sharding's call costs)
            entry["exposed_collective_ms"] = max(0.0, entry[best]["ms"] - token["ms"])
            column[kind] = entry
            del weight
            torch.cuda.empty_cache()
    status = sfq.device_status()

    # ---- single-GPU extras: the reference's GPU path, configuration 4's block, the CPU baseline
    gpu_ref = block = base = None
    if world == 1 and rank == 0:
        if not args.no_gpu_reference:
            gpu_ref = gpu_reference5(torch, wdev, xs, m)
            if isinstance(gpu_ref, dict):
                for r in table:
                    ref_ms = gpu_ref[r["linear"]][r["kind"]]
                    r["reference_kernels_ms"] = ref_ms
                    r["speedup_over_reference_kernels"] = ref_ms / r["ms"]
        del xs, ys
        torch.cuda.empty_cache()
        if not args.no_block:
            block = dit_block_ms(torch, sfq)
        status = status or sfq.device_status()
        if not args.no_cpu:
            base = cpu_baseline5(np, torch, host, steps=2, warmup=1)

    if rank == 0:
        # The kernel is timed over ten back-to-back launches of several milliseconds each, i.e. under the power cap like the
        # step itself, so the denominator is the SUSTAINED bf16 figure (x4 for fp4); the burst figure is quoted beside it.
        derived4 = PEAK_MULT["nvfp4"] * peaks["bf16_tflops_sustained"]
        derived4_burst = PEAK_MULT["nvfp4"] * peaks["bf16_tflops"]
        gemm_tf = 2.0 * m * n_up * k_up / (gemm_ms * 1e-3) / 1e12
        cap_rows = profile_value("gemm_pair_kernel_nvfp4_ffn_up.md", "rows")
        cap_bytes = profile_value("gemm_pair_kernel_nvfp4_ffn_up.md", "dram_bytes_per_launch")
        traffic = int(cap_bytes * (m / cap_rows)) if cap_rows and cap_bytes else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms_max / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "nvfp4+int8", "data": "synthetic", "config": {"workload": WORKLOAD5, "seed": SEED5},
            "detail": {"tokens": TOKENS, "rows_on_rank0": m, "linears_per_step": len(calls),
                       "l2": "every operand of every Linear is larger than the 126 MB L2 (the smallest, one rank's activation at "
                             "8 GPUs, is 143 MB), and six different Linears run between two uses of the same buffers",
                       "parallelism": f"token-sharded x{world}, weights replicated, no collective on the data path",
                       "timed_region_ms": ms_max},
            "e2e": e2e, "gpu_launches": launches_per_step * steps, "clocks": clocks.summary(),
            "roofline": {"bound": "tensor", "kernel": "gemm_pair_kernel<nvfp4> (CTA pair, 256-wide tiles) at FFN-up, this rank's rows",
                         "achieved": gemm_tf, "peak": derived4, "unit": "TFLOP/s", "frac": gemm_tf / derived4, "traffic": traffic,
                         "ms_per_launch": gemm_ms, "frac_of_nominal_9000": gemm_tf / NOMINAL_TFLOPS["nvfp4"],
                         "frac_of_4x_burst": gemm_tf / derived4_burst,
                         "peak_note": f"4 x {peaks['source']} dense bf16 SUSTAINED ({peaks['bf16_tflops_sustained']} TFLOP/s; burst "
                                      f"{peaks['bf16_tflops']}): MEASURED_PEAKS holds no fp4 figure; ten back-to-back launches",
                         "traffic_note": "dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu capture summarised in "
                                         "profiles/gemm_pair_kernel_nvfp4_ffn_up.md, scaled by rows; algorithmic bytes "
                                         f"{int(m * k_up * 0.5625 + n_up * k_up * 0.5625 + 2.0 * m * n_up)}"},
            "linears": table,
            "kernels_ms": kern, "kernel_time_shares": shares,
            "streaming": {"quantize_nvfp4_ffn_up_GBps": (2.0 * m * k_up + m * k_up / 2 + m * k_up / 16) / (quant_ms * 1e-3) / 1e9,
                          "hbm_peak_GBps": peaks["hbm_gbs"], "peak_source": peaks["source"]},
            "column_split": column or None, "dit_block": block, "gpu_reference": gpu_ref if not isinstance(gpu_ref, dict) else "see linears[*].reference_kernels_ms",
            "device_status": status,
        }
        if base is not None:
            line["cpu_baseline"] = base
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config2", action="store_true", help="run benchmark configuration 2 (W4A8 attention projection, M=4096, weak scaling) and exit")
    ap.add_argument("--config3", action="store_true", help="run benchmark configuration 3 (W6A8 FFN pair, M=32760) and exit")
    ap.add_argument("--block-stack", type=int, default=0, metavar="BLOCKS",
                    help="run benchmark configuration 4 (NVFP4 DiT block stack at 75600 tokens) with this many blocks and exit")
    ap.add_argument("--case", default=None, help="run one kernel on a small case (for ncu) and exit: gemm_int8, gemm_int8_c2, "
                    "gemm_nvfp4, gemm_nvfp4_ffn_up, quantize_int8, quantize_int8_k13824, quantize_nvfp4, unpack_w4a8, attention")
    ap.add_argument("--band", type=int, default=0, help="with --case on a GEMM: row tiles per raster band (0 = default)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--extra", action="store_true", help="with --config2: also time the GEMMs at the other DiT shapes (1 GPU)")
    for flag in ("e2e", "column-split", "gpu-reference", "block", "cpu"):
        ap.add_argument("--no-" + flag, action="store_true", help="leave this part of the default run out")
    args = ap.parse_args()
    if args.config3:
        run_config3()
    elif args.case:
        run_case(args.case, args.band)
    elif args.block_stack:
        run_block_stack(args.block_stack)
    elif args.config2:
        run_reference_config2(args) if args.impl == "reference" else run_config2(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
