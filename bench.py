"""Benchmark of the quantized-Linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--extra]

Workload (config.workload): benchmark configuration 2 -- the W4A8 attention projection, M=4096 tokens,
K=N=5120, weights ~N(0,0.02) packed by the library's W4A8 packer, activations bf16 ~N(0,1) with
0.1 % outliers x20, fp32 bias, seed 1. A step is one LinearRunner.forward: expand the packed weight,
fused ConvRot + per-token int8, tcgen05 int8 GEMM with the scale/bias epilogue (3 launches).

value  whole-job TFLOP/s (2*M*N*K per step per GPU) with inputs resident in HBM, K steps between CUDA
       events, max over ranks. Inputs rotate over several distinct buffers whose total exceeds L2.
e2e    the same metric through the same call with HOST buffers: pinned x -> device, forward, y -> host,
       both copies inside the timed region.
roofline   the dominant kernel (the int8 GEMM) timed alone with CUDA events; tensor-bound.
cpu_baseline / --impl reference   the reference's host path (decode to dense fp32, x * W^T) restated in
       oracle/ and timed on the host cores over a bounded row sample.
Multi-GPU: tokens are sharded, weights replicated, no collective on the data path (weak scaling).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

M, N, K = 4096, 5120, 5120
SEED = 1
WORKLOAD = "config2: W4A8 attention projection M=4096 K=N=5120, bf16 in/out, fp32 bias"
METRIC = "quantized_linear_tflops"
UNIT = "TFLOP/s"
CPU_SAMPLE_ROWS = 256


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


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
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
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
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        mhz, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                mhz.append(float(r[0]))
                mx = max(mx, float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = [m for m in mhz if m >= 0.5 * mx] or mhz
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


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


def run_reference(args):
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


# dram__bytes_read.sum + dram__bytes_write.sum of one config-2 GEMM launch (ncu capture of `--case gemm_int8_c2`).
C2_GEMM_DRAM_BYTES = 52883456 + 14948352


def time_region(torch, fn, iters):
    """CUDA-event time of `iters` calls on the current stream, in milliseconds."""
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(iters):
        fn(i)
    b.record()
    b.synchronize()
    return a.elapsed_time(b)


def run_ours(args):
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
                         "peak": int8_peak, "unit": "TFLOP/s", "frac": gemm_tflops / int8_peak, "traffic": C2_GEMM_DRAM_BYTES,
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
            sfq.lib.sfq_gemm_tuning(tile_n, 0, 0)
            for kind, f, mult in (("int8", fn, 2), ("nvfp4", fn4, 4)):
                for i in range(2):
                    f(i)
                torch.cuda.synchronize()
                ms = time_region(torch, f, reps) / reps
                tf = 2.0 * m * n * k / ms / 1e9
                out[f"{kind}_{name}_{'pair' if tile_n == 0 else 'bn%d' % tile_n}"] = {"ms": round(ms, 4), "tflops": round(tf, 1),
                                                    f"frac_of_{mult}x_bf16": round(tf / (mult * peaks["bf16_tflops"]), 3)}
        sfq.lib.sfq_gemm_tuning(0, 0, 0)
        del a8, w8, aq, wq, asf, wsf, y
        torch.cuda.empty_cache()
    out["device_status"] = sfq.device_status()
    return out


def run_case(name):
    """One kernel, three launches, on operands larger than L2: the target of an ncu capture."""
    import ctypes as C

    import torch

    import slopfab_b200 as sfq

    torch.cuda.set_device(0)
    sfq.lib.sfq_gemm_tuning(int(os.environ.get("SFQ_TILE_N", "0")), 0, 0)  # experiments: 128 or 256
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
    ms = time_region(torch, fn, reps) / reps
    print(json.dumps({"case": name, "ms_per_launch": ms, "work_per_second": work / (ms * 1e-3),
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


def run_config5(steps=5):
    """benchmark configuration 5: NVFP4 and W4A8 DiT Linears at M = 31x45x80 = 111600 tokens, token-sharded over the ranks
    of this launch (weights replicated, no collective), plus the FFN-up column split with one all-gather. Launch
    under torch.distributed.run for more than one GPU. One JSON line per (kind, shape, scheme), aggregate TFLOP/s."""
    import torch
    import torch.distributed as dist

    import slopfab_b200 as sfq
    from slopfab_b200.parallel import ColumnSplitPlan, column_shard, token_shard

    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peaks = load_peaks()
    M = 31 * 45 * 80
    _, m = token_shard(M, world, rank)
    g = torch.Generator(device="cuda").manual_seed(4)
    import ctypes as C

    def timed(fn):
        for i in range(2):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(steps):
            fn()
        b.record()
        b.synchronize()
        t = torch.tensor([a.elapsed_time(b) / steps], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    for kname, k, n in (("attn_proj", 5120, 5120), ("ffn_up", 5120, 13824), ("ffn_down", 13824, 5120)):
        x = torch.randn((m, k), device="cuda", generator=g).to(torch.bfloat16)
        y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        # ---- W4A8: int8 expansion held (what prepare() keeps for a chunk loop), fused quantizer + GEMM per call
        w8 = torch.randint(-127, 128, (n, k), dtype=torch.int8, device="cuda", generator=g)
        cs = torch.rand(n, device="cuda", generator=g) * 0.01
        q = torch.empty((m, k), dtype=torch.int8, device="cuda")
        rs = torch.empty(m, device="cuda")
        ep8 = sfq.Epilogue(sfq.ptr(rs), sfq.ptr(cs), 1.0, None, sfq.F32, sfq.ACT_NONE)

        def w4a8():
            sfq.check(sfq.lib.sfq_quantize_int8_token(sfq.ptr(x), None, sfq.ptr(q), sfq.ptr(rs), None, m, k, 1, sfq.stream_ptr()))
            sfq.check(sfq.lib.sfq_gemm_int8(sfq.ptr(q), sfq.ptr(w8), C.byref(ep8), sfq.ptr(y), m, n, k, sfq.stream_ptr()))

        # ---- NVFP4 native
        wq = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda", generator=g)
        wsf = torch.randint(0x30, 0x40, (n * k // 16,), dtype=torch.uint8, device="cuda", generator=g)
        xq = torch.empty((m, k // 2), dtype=torch.uint8, device="cuda")
        xsf = torch.empty(sfq.lib.sfq_nvfp4_act_scale_bytes(m, k), dtype=torch.uint8, device="cuda")
        ep4 = sfq.Epilogue(None, None, 1e-3, None, sfq.F32, sfq.ACT_NONE)

        def nvfp4():
            sfq.check(sfq.lib.sfq_quantize_nvfp4_block(sfq.ptr(x), None, sfq.ptr(xq), sfq.ptr(xsf), None, m, k,
                                                       sfq.NVFP4_ACT_GEMM_FEED, sfq.stream_ptr()))
            sfq.check(sfq.lib.sfq_gemm_nvfp4(sfq.ptr(xq), sfq.ptr(xsf), sfq.ptr(wq), sfq.ptr(wsf), C.byref(ep4), sfq.ptr(y), m, n, k,
                                             sfq.stream_ptr()))

        flops = 2.0 * M * n * k
        for kind, fn, mult in (("w4a8", w4a8, 2), ("nvfp4", nvfp4, 4)):
            ms = timed(fn)
            if rank == 0:
                tf = flops / (ms * 1e-3) / 1e12
                print(json.dumps({"case": "config5", "kind": kind, "linear": kname, "scheme": "token-sharded", "n_gpus": world,
                                  "tokens": M, "ms": ms, "tflops": tf,
                                  "frac_of_peak": tf / (world * mult * peaks["bf16_tflops"]),
                                  "peak_note": f"{mult} x measured dense bf16 burst per GPU"}), flush=True)
        if kname == "ffn_up" and M % world == 0:
            c0, nl = column_shard(n, world, rank)
            plans = {"w4a8": ColumnSplitPlan("w4a8", m, k, nl, (w8[c0:c0 + nl].contiguous(), cs[c0:c0 + nl].contiguous()), world),
                     "nvfp4": ColumnSplitPlan("nvfp4", m, k, nl, (wq[c0:c0 + nl].contiguous(),
                                                                  wsf.view(n // 128, -1)[c0 // 128:(c0 + nl) // 128].contiguous().view(-1), 1e-3), world)}
            for kind, mult in (("w4a8", 2), ("nvfp4", 4)):
                ms = timed(lambda: plans[kind].forward(x))
                if rank == 0:
                    tf = flops / (ms * 1e-3) / 1e12
                    print(json.dumps({"case": "config5", "kind": kind, "linear": kname, "scheme": "column-split, one all-gather",
                                      "n_gpus": world, "tokens": M, "ms": ms, "tflops": tf,
                                      "frac_of_peak": tf / (world * mult * peaks["bf16_tflops"]),
                                      "gathered_bytes_per_gpu": plans[kind].block * (world - 1)}), flush=True)
            del plans
        del x, y, w8, q, wq, wsf, xq, xsf
        torch.cuda.empty_cache()
    st = sfq.device_status()
    if rank == 0:
        print(json.dumps({"case": "config5", "device_status": st}))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config5", action="store_true",
                    help="run benchmark configuration 5 (M=111600 scaling sweep) on the ranks of this launch and exit")
    ap.add_argument("--config3", action="store_true", help="run benchmark configuration 3 (W6A8 FFN pair, M=32760) and exit")
    ap.add_argument("--block-stack", type=int, default=0, metavar="BLOCKS",
                    help="run benchmark configuration 4 (NVFP4 DiT block stack at 75600 tokens) with this many blocks and exit")
    ap.add_argument("--case", default=None, help="run one kernel on a small case (for ncu) and exit: gemm_int8, "
                    "gemm_nvfp4, quantize_int8, quantize_nvfp4")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--extra", action="store_true", help="also time the GEMMs at the other DiT shapes (1 GPU)")
    args = ap.parse_args()
    if args.config3:
        run_config3()
        return
    if args.config5:
        run_config5()
        return
    if args.case:
        run_case(args.case)
        return
    if args.block_stack:
        run_block_stack(args.block_stack)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
