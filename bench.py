#!/usr/bin/env python
"""Benchmark of the quantized block-sparse SpMM path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One JSON line on stdout (rank 0).  A "step" is one pass of the hot path - one SpMM launch over one
batch of synthetic input.  Workloads:

  headline (default)  4096 x 4096, 32x32 tiles, uniform random block mask at 90 % block sparsity,
                      A INT8 per block, B 4096 x 512 INT8 per column, int32 accumulate, fp16 out.
                      With N GPUs the global A is (4096*N) x 4096 sharded ROW_WISE - 4096 rows per
                      rank, B replicated by one NCCL broadcast at set-up, no collective in the step
                      (weak scaling: work per GPU is fixed).
  fp8                 same shape, A and B in FP8 E4M3 (per-block / per-column scales), fp32 accumulate.
  fp32 / fp16         same shape, floating-point void_spmm (fp32 operands multiplied as TF32, or fp16
                      operands; fp32 accumulate; result in the operands' type).  fp32 is the
                      configuration of the reference's published SpMM timings (vs_baseline).
  powerlaw            16384 x 16384, Zipf(1.5) tile-row lengths, N = 256, INT8, Stream-K + GELU, bf16 out.
  sharded             65536 x 65536 at 95 %, N = 1024, INT8, ROW_WISE shards over the ranks (strong
                      scaling: the total work is fixed).
  mid                 16384 x 16384 at 90 %, N = 1024, INT8: a tensor-bound case small enough to profile.

value  = whole-job TOPS over the nonzero tiles (2*nnz*32*32*N per step) with inputs resident in HBM.
e2e    = the same metric through the public operator with HOST buffers: every step copies that step's
         B (and its column scales) from pinned host memory to the device, runs the operator and
         copies C back.  A, the sparse operand, is resident like a weight.
L2     = the step rotates over enough distinct copies of (A, B, C) to exceed the 126 MB L2, so the
         kernel reads its inputs from HBM ("l2": "rotating_inputs" in config).
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "block_sparse_spmm_tops_nonzero_tiles"
# ncu summary of the dominant kernel per workload: roofline.traffic is read from it (dram__bytes_read.sum +
# dram__bytes_write.sum of one launch), it is not measured by this run
PROFILE_OF = {"headline": "spmm_rowacc_int8_headline.md", "fp8": "spmm_rowacc_fp8_headline.md",
              "powerlaw": "spmm_rowacc_int8_powerlaw_streamk.md", "fp32": "spmm_rowacc_tf32_headline.md",
              "sharded": "spmm_rowacc_int8_sharded65536.md", "mid": "spmm_rowacc_int8_mid16384.md"}
L2_BYTES = 126 * 1024 * 1024
STRONG_WORKLOAD = "uniform65536_bs95_n1024"


def profiled_traffic(workload):
    """(bytes per launch, source) from the committed ncu summary of the workload's kernel, or (None, None)."""
    import re
    name = PROFILE_OF.get(workload)
    path = os.path.join(ROOT, "profiles", name) if name else None
    if not path or not os.path.exists(path):
        return None, None
    text = open(path).read()
    unit = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}
    total, seen = 0.0, set()
    for key in ("dram__bytes_read.sum", "dram__bytes_write.sum"):
        m = re.search(r"^\s*" + re.escape(key) + r"\s+([0-9.]+)\s+(byte|Kbyte|Mbyte|Gbyte)\b", text, re.M)
        if m:
            total += float(m.group(1)) * unit[m.group(2)]
            seen.add(key)
    if len(seen) < 2:
        return None, None
    return total, "profiles/%s (ncu capture of one launch, static)" % name


def workload_config(args, world):
    """What both arms print as ``config``: a description of the workload that does not depend on what ran it.
    nnz_tiles is the realised tile count of the first input copy of one GPU (seed 0)."""
    import numpy as np
    from void_b200 import workloads
    if args.workload == "powerlaw":
        nnz = int(workloads.zipf_mask(512, 512, 1.5, 512, 15.36, 0).sum())
        cfg = {"workload": "zipf16384_n256_streamk_gelu", "M_per_gpu": 16384, "K": 16384, "N": 256, "out_dtype": "bfloat16"}
    elif args.workload == "mid":
        nnz = int(workloads.uniform_mask(512, 512, args.sparsity, 0).sum())
        cfg = {"workload": "uniform16384_bs%02d_n1024" % round(args.sparsity * 100), "M_per_gpu": 16384, "K": 16384,
               "N": 1024, "out_dtype": "float16"}
    elif args.workload == "sharded":
        nnz = int(round(2048 * 2048 * 0.05))
        cfg = {"workload": STRONG_WORKLOAD + "_rowshards", "M_per_gpu": 65536 // world, "K": 65536, "N": 1024,
               "out_dtype": "float16"}
    else:
        nnz = int(workloads.uniform_mask(128, 128, args.sparsity, 0).sum())
        out = {"fp32": "float32"}.get(args.workload, "float16")
        cfg = {"workload": "uniform4096_bs%02d_n512%s" % (round(args.sparsity * 100), "" if world == 1 else "_x%d_rowshards" % world),
               "M_per_gpu": 4096, "K": 4096, "N": 512, "out_dtype": out}
    cfg.update({"tile": 32, "nnz_tiles": nnz, "l2": "rotating_inputs", "parallelism": "row_shards_x%d" % world,
                "strong_scaling_workload": STRONG_WORKLOAD if world > 1 else None})
    return cfg


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="headline", choices=["headline", "fp8", "powerlaw", "sharded", "fp32", "fp16", "mid", "floor", "prep"])
    ap.add_argument("--min-timed-ms", type=float, default=50.0, help="repeat the K steps until the timed region lasts this long")
    ap.add_argument("--sparsity", type=float, default=0.9)
    ap.add_argument("--no-graph", action="store_true", help="launch every step from Python instead of a CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-depth", type=int, default=4, help="steps in flight in the end-to-end leg")
    ap.add_argument("--no-strong", action="store_true", help="skip the strong-scaling record of a multi-GPU run")
    ap.add_argument("--copies", type=int, default=0, help="distinct input copies to rotate over (0 = enough for L2)")
    return ap.parse_args()


# The reference's only published timings on this path's shape: fp32 void_spmm, 4096 x 4096, N = 512, on an
# unnamed "RTX GPU" (its README.md:150-158), milliseconds by block sparsity.
PUBLISHED_FP32_MS = {0.70: 0.28, 0.80: 0.19, 0.90: 0.12, 0.95: 0.06, 0.98: 0.04}


def vs_published(args, world, ms_per_step):
    """value / published value for the one configuration the reference published (same tiles and
    operation count on both sides, so the ratio of TFLOP/s is the ratio of times); None otherwise."""
    if args.workload != "fp32" or world != 1:
        return None
    ref_ms = PUBLISHED_FP32_MS.get(round(args.sparsity, 2))
    return None if ref_ms is None else ref_ms / ms_per_step


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Polls SM clock and throttle reasons of one GPU through NVML while the benchmark runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.samples, self.stop_flag, self.window = [], False, [None, None]
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.max_mhz = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((time.perf_counter(), mhz, reasons))
            except Exception:
                pass
            time.sleep(0.002)

    def summary(self):
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        t0, t1 = self.window
        inside = [s for s in self.samples if t0 is not None and t0 <= s[0] <= t1]
        use = inside if inside else self.samples
        mhz = sorted(s[1] for s in use)
        bits = 0
        for s in use:
            bits |= s[2]
        names = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
                 0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
                 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}
        reasons = [n for b, n in names.items() if bits & b and n != "gpu_idle"]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(use), "samples_in_timed_region": len(inside)}


# ----------------------------------------------------------------------------------------------
def cpu_reference_arm(args, rank, world):
    """The reference has no compiled CPU kernel; its arithmetic for this path, restated on the CPU
    (oracle/void_oracle.py: int32 tile-row products through float64 BLAS, mean-scale epilogue), is
    timed on the host cores.  Rank 0 only."""
    if rank != 0:
        return
    import numpy as np
    import torch
    from oracle import void_oracle as vo
    cfg, run, cores = cpu_workload(args, np, torch, vo)
    t_w = time.perf_counter()
    for w in range(args.warmup):
        run()
        if time.perf_counter() - t_w > 30.0:      # the requested warm-up, unless the host is far too slow for it
            break
    t0 = time.perf_counter()
    n = 0
    budget = 150.0
    while n < args.steps and (time.perf_counter() - t0) < budget:
        run()
        n += 1
    dt = (time.perf_counter() - t0) / n
    tops = cfg["ops"] / dt / 1e12
    line = {
        "metric": METRIC, "value": tops, "unit": "TOPS", "n_gpus": args.gpus, "steps": n, "warmup": args.warmup,
        "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong" if args.workload == "sharded" else "weak",
        "vs_baseline": None,
        "dtype": cfg["dtype"], "data": "synthetic", "impl": "reference", "config": workload_config(args, world),
        "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": cores, "kind": "port",
                         "sample": "one GPU's share of the workload (%s, %d tiles) per step, %d steps, %s"
                                   % (cfg["config"]["workload"], cfg["config"]["nnz_tiles"], n, cfg["how"])},
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def cpu_workload(args, np, torch, vo):
    """Host copy of the N=1 workload + a closure that runs the oracle on it once."""
    from void_b200 import workloads
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    if args.workload == "powerlaw":
        mask, N, name = workloads.zipf_mask(512, 512, 1.5, 512, 15.36, 0), 256, "zipf16384_n256"
    else:
        mask, N, name = workloads.uniform_mask(128, 128, args.sparsity, 0), 512, "uniform4096_bs%02d_n512" % round(args.sparsity * 100)
    rows, cols = np.nonzero(mask)
    order = np.argsort(vo.morton_encode_batch(rows, cols))
    rows, cols = rows[order].astype(np.int32), cols[order].astype(np.int32)
    g = torch.Generator().manual_seed(0)
    vals = torch.randn(len(rows), 32, 32, generator=g).numpy()
    b = torch.randn(mask.shape[1] * 32, N, generator=g).numpy()
    shape = (mask.shape[0] * 32, mask.shape[1] * 32)
    how = "numpy tile-row products (float64 BLAS for the integer sums)"
    if args.workload in ("fp32", "fp16"):
        np_dt = np.float32 if args.workload == "fp32" else np.float16
        vals_t, b_t = vals.astype(np_dt), b.astype(np_dt)
        run = lambda: vo.spmm_fp(vals_t, rows, cols, shape, b_t).astype(np_dt)
        dtype = "tf32" if args.workload == "fp32" else "f16"
    elif args.workload == "fp8":
        q, s, _, _ = vo.quantize_fp8_tiles(vals)
        bq, bs, _ = vo.quantize_fp8_cols(b)
        b_deq = vo.fp8_bytes_to_float(bq) * bs[None, :]
        run = lambda: vo.spmm_fp8(q, s, rows, cols, shape, b_deq).astype(np.float16)
        dtype = "f8e4m3"
    else:
        q, s = vo.quantize_int8_tiles(vals)
        bq, bs = vo.quantize_int8_cols(b)
        # the C restatement (int8 x int8 -> int32, OpenMP over tile rows) when it could be built, else the numpy one
        spmm = vo.spmm_int8_c if vo.c_library() is not None else vo.spmm_int8
        how = "C / OpenMP int8 tile-row products" if vo.c_library() is not None else how
        if args.workload == "powerlaw":
            run = lambda: vo.gelu_tanh_sigmoid(spmm(q, s, rows, cols, shape, bq, col_scale=bs))
        else:
            run = lambda: spmm(q, s, rows, cols, shape, bq, col_scale=bs).astype(np.float16)
        dtype = "i8"
    cfg = {"ops": workloads.spmm_ops(len(rows), N), "dtype": dtype, "how": how,
           "config": {"workload": name, "M": shape[0], "K": shape[1], "N": N, "tile": 32, "nnz_tiles": int(len(rows)),
                      "block_sparsity": 1.0 - len(rows) / mask.size}}
    return cfg, run, cores


# ----------------------------------------------------------------------------------------------
def launch_floor(args, torch, void, workloads, _lib, _spmm, dev):
    """What a launch of the headline's shape costs before any work, in the harness of the timed steps (CUDA graph
    of 512 launches back to back, rotating input copies): an empty kernel with the same grid, block, shared memory
    and launch attribute; the SpMM over an EMPTY A of the same shape; and the SpMM itself with its switches."""
    import numpy as np
    import scipy.sparse as sp
    lib = _lib.load()
    ns = args.copies if args.copies > 0 else 34
    sets = []
    for i in range(ns):
        w = workloads.headline(args.sparsity, seed=i, device=dev)
        q = void.quantize_void_tensor(w.a)
        bq, bs = void.quantize_cols_int8(w.b)
        sets.append((q.packed(), bq.contiguous(), bs, torch.empty(4096, 512, dtype=torch.float16, device=dev)))
    empty = void.quantize_void_tensor(void.csr_to_void(sp.csr_matrix((4096, 4096), dtype=np.float32), device=dev)).packed()
    torch.cuda.synchronize()

    def timed(fn, steps=512, reps=8):
        for i in range(8):
            fn(i)
        torch.cuda.synchronize()
        st = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(st):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                for i in range(steps):
                    fn(i)
            g.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(st)
            for _ in range(reps):
                g.replay()
            e1.record(st)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (reps * steps) * 1e3

    def spmm(pk, **kw):
        def fn(i):
            _, bq, bs, out = sets[i % ns]
            _spmm.spmm(pk(i), bq, out, scale_mode=_lib.SCALE_ROW_MEAN, col_scale=bs, **kw)
        return fn
    own = lambda i: sets[i % ns][0]
    res = {
        "null_kernel_us": timed(lambda i: lib.void_launch_floor(512, 224, 50176, _lib.stream_ptr(dev))),
        "empty_a_us": timed(spmm(lambda i: empty)),
        "spmm_us": timed(spmm(own)),
        "spmm_one_store_per_tile_us": timed(spmm(own, flags=_spmm.FLAG_STORE_PER_TILE)),
        "spmm_direct_stores_us": timed(spmm(own, flags=_spmm.FLAG_DIRECT_STORES)),
        "spmm_a_not_read_early_us": timed(spmm(own, flags=_spmm.FLAG_NO_EARLY_A)),
    }
    _lib.check_device_status(dev)
    print(json.dumps({"workload": "floor", "shape": "uniform4096_bs%02d_n512" % round(args.sparsity * 100),
                      "input_copies": ns, "launches_per_graph": 512, **{k: round(v, 3) for k, v in res.items()}}))


def prep_kernels(args, torch, void, workloads, _lib, _spmm, dev):
    """The preparation operators of the path (quantisers, tile index + packing, format build), one after the
    other on inputs larger than L2, CUDA events around `reps` back-to-back calls of each.  Every figure is the
    operator's algorithmic bytes (what it must read and write) over its time, against the measured copy peak;
    an operator is one to four kernels, listed in profiles/prep_kernels.md."""
    import numpy as np
    reps = max(1, min(args.steps, 20))
    peak = measured_peaks()["hbm_gbs"]
    nb = 512
    mask = workloads.uniform_mask(nb, nb, 0.85, 0)                  # 39 k tiles: 161 MB of fp32 tile values
    nnz = int(mask.sum())
    g = torch.Generator(device="cpu").manual_seed(0)
    a = workloads.block_sparse(mask, 8, seed=0, device=dev).a
    b = torch.randn(nb * 32, 2048, generator=g).to(dev)             # 134 MB fp32
    dense = torch.randn(8192, 8192, generator=g).to(dev) * (torch.rand(256, 256, generator=g) > 0.5).to(dev).repeat_interleave(32, 0).repeat_interleave(32, 1)
    q = void.quantize_void_tensor(a)
    a8 = void.void_tensor_to_fp8(a)
    K, N = b.shape

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e3

    def pack_i8():
        return _spmm.pack(q.values, q.scales, q.block_rows, q.block_cols, q.shape, _lib.KIND_I8)

    def pack_f8(terms):
        return _spmm.pack_f8_split(a8.values_fp8.view(torch.uint8), a8.scaling_info.scale, a8.block_rows, a8.block_cols, a8.shape, terms)

    idx = nnz * 12 + (nb + 1) * 4
    ops = [
        ("quantize_void_tensor (INT8, per tile)", lambda: void.quantize_void_tensor(a), nnz * (4096 + 1024 + 4)),
        ("void_tensor_to_fp8 (E4M3, per tile)", lambda: void.void_tensor_to_fp8(a), nnz * (4096 + 1024 + 12)),
        ("quantize_cols_int8 (B, per column: absmax pass + quantise pass)", lambda: void.quantize_cols_int8(b), K * N * 9 + N * 4),
        ("quantize_cols_fp8 (B, per column)", lambda: void.quantize_cols_fp8(b), K * N * 9 + N * 8),
        ("tile index + pack, INT8 (bitmap mark / count / scan / rank, gather, row scales)", pack_i8, nnz * 2048 + 2 * idx),
        ("tile index + pack, FP8 tiles as two E4M3 terms", lambda: pack_f8(2), nnz * 3072 + 2 * idx),
        ("dense_to_void 8192^2 fp32, half of the tiles kept (mark, Morton rank, gather)", lambda: void.dense_to_void(dense),
         dense.numel() * 4 * 2 + (dense.numel() // 2) * 4),
        ("compute_stream_k_workload + plan (O(tile rows): latency bound)", lambda: void.compute_stream_k_workload(q), 0),
    ]
    res = []
    for name, fn, nbytes in ops:
        us = timed(fn)
        gbs = nbytes / (us * 1e-6) / 1e9 if nbytes else None
        res.append({"op": name, "us": round(us, 1), "algorithmic_mb": round(nbytes / 1e6, 1),
                    "gbs": None if gbs is None else round(gbs), "frac_of_measured_hbm": None if gbs is None else round(gbs / peak, 3)})
    _lib.check_device_status(dev)
    print(json.dumps({"workload": "prep", "tiles": nnz, "b": [K, N], "reps": reps, "hbm_peak_gbs": peak, "ops": res}))


def strong_scaling_record(torch, dist, void, workloads, _lib, dev, rank, world):
    """The multi-GPU workload, measured in the same run as the weak-scaling line: A 65536 x 65536 at 95 % block
    sparsity, INT8 per block, B 65536 x 1024 INT8 per column, fp16 row shards.  Total work is fixed:
      ms_1gpu        rank 0 alone multiplies all 2048 tile rows (the other ranks idle at a barrier);
      ms_per_step    every rank multiplies its ROW_WISE shard, no collective in the step, max over ranks;
      column_wise_*  the same product from COLUMN_WISE shards, summed over ranks inside the kernel (every rank
                     ends with the finished rows it owns), next to what an NCCL all_reduce of the fp32 [M, N]
                     partial results alone would cost (the reference's way of adding them).
    Every rank generates the same A from one seed and shards it; B is made on rank 0 and broadcast.  Steps rotate
    over two copies of B and C so that a rank's working set (27 MB of A at eight ranks) does not stay in L2."""
    import time as _time
    N, K = 1024, 65536
    full, _, nnz = workloads.sharded_int8(world_size=1, rank=0, device=dev)
    g = torch.Generator(device="cpu").manual_seed(0)
    if rank == 0:
        b = torch.randn(K, N, generator=g).to(dev)
        bq0, bs0 = void.quantize_cols_int8(b)
        bq0 = bq0.contiguous()
        del b
    else:
        bq0 = torch.empty(K, N, dtype=torch.int8, device=dev)
        bs0 = torch.empty(N, dtype=torch.float32, device=dev)
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    void.broadcast_b(bq0, src=0, scales=bs0)              # warm the channels
    e0.record()
    void.broadcast_b(bq0, src=0, scales=bs0)
    e1.record()
    torch.cuda.synchronize()
    bcast = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    dist.all_reduce(bcast, op=dist.ReduceOp.MAX)
    bqs = [bq0, torch.roll(bq0, 1, 0).contiguous()]

    def timed(fn, steps, graph=True):
        for i in range(4):
            fn(i)
        torch.cuda.synchronize()
        st = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(st):
            if graph:
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr, stream=st):
                    for i in range(steps):
                        fn(i)
                run = gr.replay
            else:
                run = lambda: [fn(i) for i in range(steps)]
            run()
            torch.cuda.synchronize()
            dist.barrier()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 4
            t0.record(st)
            for _ in range(reps):
                run()
            t1.record(st)
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / (reps * steps)

    # ---- ROW_WISE shards, every rank at once
    d = void.shard_void_tensor(full, void.ShardingStrategy.ROW_WISE)
    shard = d.local_tensor
    outs = [torch.empty(shard.shape[0], N, dtype=torch.float16, device=dev) for _ in range(2)]
    ms_n = timed(lambda i: void.void_spmm_int8(shard, bqs[i % 2], bs0, outs[i % 2]), 20)
    t = torch.tensor([ms_n], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_n = float(t.item())
    _lib.check_device_status(dev)
    del outs

    # ---- one GPU alone on the whole matrix
    ms_1 = 0.0
    if rank == 0:
        outs1 = [torch.empty(full.shape[0], N, dtype=torch.float16, device=dev) for _ in range(2)]
        for i in range(4):
            void.void_spmm_int8(full, bqs[i % 2], bs0, outs1[i % 2])
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for i in range(40):
            void.void_spmm_int8(full, bqs[i % 2], bs0, outs1[i % 2])
        t1.record()
        torch.cuda.synchronize()
        ms_1 = t0.elapsed_time(t1) / 40
        del outs1
    t = torch.tensor([ms_1], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_1 = float(t.item())

    # ---- COLUMN_WISE shards, summed inside the kernel; and the all_reduce the reference would run instead
    col = {}
    try:
        dc = void.shard_void_tensor(full, void.ShardingStrategy.COLUMN_WISE)
        fn = lambda i: void.distributed_void_spmm(dc, bqs[i % 2], b_scale=bs0, out_dtype=torch.float16, gather_output=False)
        ms_c = timed(fn, 10, graph=False)
        part = torch.zeros(full.shape[0], N, dtype=torch.float32, device=dev)
        ms_ar = timed(lambda i: dist.all_reduce(part), 5, graph=False)
        t = torch.tensor([ms_c, ms_ar], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        scratch = next(iter(dc.__dict__["_reduce_states"].values())).scratch
        col = {"column_wise_fused_ms": float(t[0]), "allreduce_fp32_result_only_ms": float(t[1]),
               "peer_memory": "symmetric memory" if not isinstance(scratch.keep, tuple) else "CUDA IPC"}
        _lib.check_device_status(dev)
    except Exception as ex:                                  # the row-shard numbers stand without it
        col = {"column_wise_error": repr(ex)[:200]}

    rows_local = shard.shape[0] // 32
    np_ = 2
    items = rows_local * (N // 128 // np_)
    ctas = 4 * void._spmm.sm_count(dev)
    a_mb, b_mb, c_mb = shard.n_blocks * 1032 / 1e6, K * N / 1e6, shard.shape[0] * N * 2 / 1e6
    limiter = ("every rank reads all of B: %.0f MB of its %.0f MB per launch; %d work items on %d resident CTAs = %.2f waves"
               % (b_mb, a_mb + b_mb + c_mb, items, ctas, items / ctas))
    return {"workload": STRONG_WORKLOAD, "nnz_tiles": int(nnz), "ms_1gpu": ms_1, "ms_per_step": ms_n,
            "speedup": ms_1 / ms_n if ms_n > 0 else None, "efficiency": ms_1 / ms_n / world if ms_n > 0 else None,
            "tops": workloads.spmm_ops(int(nnz), N) / (ms_n * 1e-3) / 1e12 if ms_n > 0 else None,
            "b_broadcast_ms": float(bcast.item()), "l2": "two copies of B and C in rotation", "limiter": limiter, **col}


def build_rank_inputs(args, rank, world, torch, void, workloads, copies_hint):
    """Per-rank operands: a list of (A quantised, B 8-bit, B scales, out) copies to rotate over."""
    dev = torch.device("cuda", torch.cuda.current_device())
    sets = []
    if args.workload == "sharded":
        shard, (start, end), nnz_global = workloads.sharded_int8(world_size=world, rank=rank, device=dev)
        g = torch.Generator(device="cpu").manual_seed(0)
        N, K = 1024, 65536
        if rank == 0:
            b = torch.randn(K, N, generator=g).to(dev)
            bq, bs = void.quantize_cols_int8(b)
            bq = bq.contiguous()
            del b
        else:
            bq = torch.empty(K, N, dtype=torch.int8, device=dev)
            bs = torch.empty(N, dtype=torch.float32, device=dev)
        out = torch.empty(shard.shape[0], N, dtype=torch.float16, device=dev)
        sets.append([shard, bq, bs, out])
        info = {"name": "uniform65536_bs95_n1024_rowshards", "M": 65536, "K": K, "N": N, "out": torch.float16,
                "kind": "i8", "nnz_local": shard.n_blocks, "rows_local": shard.shape[0], "nbr_local": shard.block_grid[0]}
        return sets, info
    if args.workload == "powerlaw":
        make = lambda seed: workloads.power_law(seed=seed, device=dev)
        N, out_dtype, kind = 256, torch.bfloat16, "i8"
    elif args.workload == "mid":
        make = lambda seed: workloads.block_sparse(workloads.uniform_mask(512, 512, args.sparsity, seed), 1024, seed, dev,
                                                   "uniform16384_bs%02d_n1024" % round(args.sparsity * 100))
        N, out_dtype, kind = 1024, torch.float16, "i8"
    else:
        make = lambda seed: workloads.headline(args.sparsity, seed=seed, device=dev)
        N, out_dtype, kind = 512, torch.float16, ("f8e4m3" if args.workload == "fp8" else "i8")
        if args.workload in ("fp32", "fp16"):
            out_dtype = torch.float32 if args.workload == "fp32" else torch.float16
            kind = "tf32" if args.workload == "fp32" else "f16"
    # every rank owns different tile rows of the global A (its own seeds); with several ranks the B
    # quantised here is overwritten by rank 0's B in the broadcast that follows
    n_copies = None
    i = 0
    while n_copies is None or i < n_copies:
        w = make(seed=1000 * rank + i)
        if kind == "i8":
            a = void.quantize_void_tensor(w.a)
            bq, bs = void.quantize_cols_int8(w.b)
            a.packed()
        elif kind == "f8e4m3":
            a = void.void_tensor_to_fp8(w.a)
            bq, bs, _ = void.quantize_cols_fp8(w.b)
            a.packed()
        else:   # floating-point operands: no scales
            a, bq, bs = w.a.to_dtype(out_dtype), w.b.to(out_dtype), torch.ones(1, device=dev)
        out = torch.empty(w.shape[0], N, dtype=out_dtype, device=dev)
        sets.append([a, bq.contiguous(), bs, out])
        if n_copies is None:
            per_copy = workloads.algorithmic_bytes(w.nnz, w.shape[0] // 32, w.shape[1], N, w.shape[0], out.element_size(),
                                                   bq.element_size())
            n_copies = copies_hint if copies_hint > 0 else max(2, -(-2 * L2_BYTES // per_copy))
            if world > 1:
                # every rank must hold the same number of copies (one broadcast of B per copy follows);
                # the realised tile count, and with it the bytes per copy, differs a little from rank to rank
                import torch.distributed as dist
                agreed = torch.tensor([n_copies], dtype=torch.int64, device=dev)
                dist.all_reduce(agreed, op=dist.ReduceOp.MAX)
                n_copies = int(agreed.item())
        del w
        i += 1
    info = {"name": None, "N": N, "out": out_dtype, "kind": kind}
    return sets, info


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        cpu_reference_arm(args, rank, world)
        return
    # stdout carries the one JSON line: NCCL writes its version banner and warnings to stdout unless told otherwise
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")

    import numpy as np
    import torch
    import torch.distributed as dist
    import void_b200 as void
    from void_b200 import _lib, _spmm, workloads, stream_k

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (this path has no CPU implementation; see --impl reference)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # a short collective timeout: a rank that falls out of step ends the run in minutes, not in ten
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    if args.gpus != world and rank == 0:
        print("bench.py: --gpus %d but WORLD_SIZE=%d; using WORLD_SIZE" % (args.gpus, world), file=sys.stderr)

    if args.workload in ("floor", "prep"):
        if rank == 0:
            (launch_floor if args.workload == "floor" else prep_kernels)(args, torch, void, workloads, _lib, _spmm, dev)
        return
    sampler = ClockSampler(local_rank)
    sampler.start()

    sets, info = build_rank_inputs(args, rank, world, torch, void, workloads, args.copies)
    # replicate B: one broadcast per copy from rank 0 over NCCL (set-up, timed separately)
    bcast_ms = None
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in sets:
            void.broadcast_b(s[1], src=0, scales=s[2])
        e1.record()
        torch.cuda.synchronize()
        bcast_ms = e0.elapsed_time(e1) / len(sets)

    kind = info["kind"]
    is_powerlaw = args.workload == "powerlaw"

    def step(i):
        a, bq, bs, out = sets[i % len(sets)]
        if is_powerlaw:
            void.void_spmm_stream_k(a, bq, b_scale=bs, out=out, activation=_lib.ACT_GELU)
        elif kind == "i8":
            void.void_spmm_int8(a, bq, bs, out)
        elif kind == "f8e4m3":
            void.void_spmm_fp8(a, bq, out.dtype, b_scale=bs, out=out)
        else:
            void.void_spmm(a, bq, out)

    # per-step work of this rank
    nnz_local = [s[0].n_blocks for s in sets]
    N = info["N"]
    ops_per_step_local = float(np.mean([workloads.spmm_ops(n, N) for n in nnz_local]))
    a0 = sets[0][0]
    M_local, K = a0.shape
    bytes_per_step = float(np.mean([workloads.algorithmic_bytes(n, a0.block_grid[0], K, N, M_local,
                                                                sets[0][3].element_size(), sets[0][1].element_size())
                                   for n in nnz_local]))

    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize()
    _lib.check_device_status(dev)

    # The timed steps are replayed CUDA graphs, so that the GPU is not waiting for the Python launch path between
    # kernels.  One pass = exactly K steps.  A replay costs a few microseconds by itself, as much as one step
    # here, so a small K is captured several passes to a graph (a "block" of ppg passes, about a thousand
    # launches); a large K is cut into graphs of at most 256 steps.
    K_steps = args.steps
    stream = torch.cuda.Stream(device=dev)
    graphs = []
    ppg = 1                                   # passes per block
    if not args.no_graph:
        if K_steps <= 256:
            ppg = max(1, 1024 // K_steps)
            glen = K_steps * ppg
        else:
            glen = 256
            while glen > 1 and glen % len(sets) != 0 and glen > len(sets):
                glen -= 1
        with torch.cuda.stream(stream):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for i in range(glen):
                    step(i)
            rem = 0 if ppg > 1 or K_steps <= 256 else K_steps % glen
            g_rem = None
            if rem:
                g_rem = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g_rem, stream=stream):
                    for i in range(rem):
                        step(i)
        graphs = [(g, 1 if K_steps <= 256 else K_steps // glen), (g_rem, 1 if rem else 0)]
        with torch.cuda.stream(stream):
            g.replay()
        torch.cuda.synchronize()

    def run_timed():                          # one block: ppg passes of K steps
        with torch.cuda.stream(stream):
            if graphs:
                for gr, reps in graphs:
                    for _ in range(reps):
                        gr.replay()
            else:
                for i in range(K_steps):
                    step(i)

    # A block lasts a few milliseconds at most, too short for the clock sampler and for a stable mean, so blocks
    # are repeated back to back until the timed region covers at least MIN_TIMED_MS; every block is bracketed
    # by its own pair of events on the launching stream.
    MIN_TIMED_MS = args.min_timed_ms
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        p0.record(stream)
    run_timed()
    with torch.cuda.stream(stream):
        p1.record(stream)
    torch.cuda.synchronize()
    probe_ms = max(p0.elapsed_time(p1), 1e-3)
    passes = int(min(max(1, -(-MIN_TIMED_MS // probe_ms)), 4000))
    if world > 1:
        agreed = torch.tensor([passes], dtype=torch.int64, device=dev)
        dist.all_reduce(agreed, op=dist.ReduceOp.MAX)
        passes = int(agreed.item())
        dist.barrier()
    torch.cuda.synchronize()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(passes + 1)]
    sampler.window[0] = time.perf_counter()
    with torch.cuda.stream(stream):
        marks[0].record(stream)
    for r in range(passes):
        run_timed()
        with torch.cuda.stream(stream):
            marks[r + 1].record(stream)
    torch.cuda.synchronize()
    sampler.window[1] = time.perf_counter()
    if world > 1:
        dist.barrier()
    block_ms = [marks[r].elapsed_time(marks[r + 1]) for r in range(passes)]
    ms_total = marks[0].elapsed_time(marks[passes]) / (passes * ppg)      # mean time of one pass of K steps
    ms_min = min(block_ms) / ppg
    passes *= ppg
    _lib.check_device_status(dev)

    # ---- end to end through the public operator with host buffers: every step copies its B (and
    # scales) from pinned host memory, runs the operator and copies C back to pinned host memory.
    # Measured twice: one step at a time (the caller waits for each result: latency), and as a
    # pipeline of three steps in flight on three streams (copy-in, operator, copy-out; a serving
    # loop: throughput).  Each step of the pipeline still moves its own inputs and result.
    a_e, bq_e, bs_e, out_e = sets[0]
    DEPTH = max(1, args.e2e_depth)
    slots = []
    for _ in range(DEPTH):
        h_b = torch.empty(bq_e.view(torch.uint8).shape, dtype=torch.uint8).pin_memory()
        h_b.copy_(bq_e.view(torch.uint8).cpu())
        slots.append({"h_b": h_b, "h_s": bs_e.cpu().pin_memory(),
                      "h_c": torch.empty(out_e.shape, dtype=out_e.dtype).pin_memory(),
                      "d_b": torch.empty_like(bq_e), "d_s": torch.empty_like(bs_e), "out": torch.empty_like(out_e),
                      "ev_in": torch.cuda.Event(), "ev_op": torch.cuda.Event(), "ev_out": torch.cuda.Event()})
    h_b, h_s, h_c = slots[0]["h_b"], slots[0]["h_s"], slots[0]["h_c"]
    s_in, s_op, s_out = (torch.cuda.Stream(device=dev) for _ in range(3))

    def operator(d_b, d_s, out):
        if is_powerlaw:
            void.void_spmm_stream_k(a_e, d_b, b_scale=d_s, out=out, activation=_lib.ACT_GELU)
        elif kind == "i8":
            void.void_spmm_int8(a_e, d_b, d_s, out)
        elif kind == "f8e4m3":
            void.void_spmm_fp8(a_e, d_b, out.dtype, b_scale=d_s, out=out)
        else:
            void.void_spmm(a_e, d_b, out)

    def e2e_step_serial():
        sl = slots[0]
        sl["d_b"].view(torch.uint8).copy_(sl["h_b"], non_blocking=True)
        sl["d_s"].copy_(sl["h_s"], non_blocking=True)
        operator(sl["d_b"], sl["d_s"], sl["out"])
        sl["h_c"].copy_(sl["out"], non_blocking=True)
        torch.cuda.current_stream().synchronize()      # the caller owns the result on the host

    def e2e_step_pipelined(i):
        sl = slots[i % DEPTH]
        sl["ev_out"].synchronize()                     # the slot's previous result has reached the host
        with torch.cuda.stream(s_in):
            sl["d_b"].view(torch.uint8).copy_(sl["h_b"], non_blocking=True)
            sl["d_s"].copy_(sl["h_s"], non_blocking=True)
            sl["ev_in"].record(s_in)
        with torch.cuda.stream(s_op):
            s_op.wait_event(sl["ev_in"])
            operator(sl["d_b"], sl["d_s"], sl["out"])
            sl["ev_op"].record(s_op)
        with torch.cuda.stream(s_out):
            s_out.wait_event(sl["ev_op"])
            sl["h_c"].copy_(sl["out"], non_blocking=True)
            sl["ev_out"].record(s_out)

    def time_e2e(fn, n):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for i in range(n):
            fn(i)
        torch.cuda.synchronize()                       # every result is on the host
        return (time.perf_counter() - t0) * 1e3 / n

    # The same three steps in flight with each slot's step (copy-in, operator, copy-out) captured once as
    # a CUDA graph and replayed on the slot's own stream: the work per step is unchanged, the Python
    # launch path (about ten API calls per step) leaves the timed loop.
    E2E_WHAT = "; B arrives already quantised (8-bit B and its column scales are the step's input), A is resident"
    e2e_mode = "host wall clock, %d steps in flight (copy-in / operator / copy-out streams)" % DEPTH
    slot_graphs = None
    # (not for the planned launch: its split-row scratch belongs to one launch at a time, and the
    # slots' graphs run on streams of their own)
    if not args.no_graph and not is_powerlaw:
        try:
            slot_graphs = []
            for sl in slots:
                st_k = torch.cuda.Stream(device=dev)
                with torch.cuda.stream(st_k):
                    gk = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gk, stream=st_k):
                        sl["d_b"].view(torch.uint8).copy_(sl["h_b"], non_blocking=True)
                        sl["d_s"].copy_(sl["h_s"], non_blocking=True)
                        operator(sl["d_b"], sl["d_s"], sl["out"])
                        sl["h_c"].copy_(sl["out"], non_blocking=True)
                slot_graphs.append((gk, st_k))
            torch.cuda.synchronize()
            e2e_mode = "host wall clock, %d steps in flight, each step (copy-in, operator, copy-out) one CUDA graph" % DEPTH
        except Exception as ex:                            # capture not possible: keep the three-stream loop
            print("bench.py: e2e graph capture failed (%r), using the stream pipeline" % (ex,), file=sys.stderr)
            slot_graphs = None

    if world > 1:
        # the timed loops below hold a barrier each: every rank must take the same ones
        okf = torch.tensor([1 if slot_graphs is not None else 0], dtype=torch.int64, device=dev)
        dist.all_reduce(okf, op=dist.ReduceOp.MIN)
        if int(okf.item()) == 0:
            slot_graphs = None

    def e2e_step_graph(i):
        sl = slots[i % DEPTH]
        gk, st_k = slot_graphs[i % DEPTH]
        sl["ev_out"].synchronize()
        with torch.cuda.stream(st_k):
            gk.replay()
            sl["ev_out"].record(st_k)

    e2e_steps = max(3, min(K_steps, 200))
    # the pipelined legs run long enough for the filling of the pipeline (DEPTH steps, a few hundred microseconds) to
    # be a small share of the timed region whatever K is: at least 400 steps
    e2e_pipe_steps = max(2 * e2e_steps, 400)
    e2e_serial_ms = time_e2e(lambda i: e2e_step_serial(), e2e_steps)
    e2e_streams_ms = time_e2e(e2e_step_pipelined, e2e_pipe_steps)
    e2e_ms = e2e_streams_ms
    if slot_graphs is not None:
        for sl in slots:
            sl["h_c"].zero_()                              # the check below must see what the graphs wrote
        e2e_ms = time_e2e(e2e_step_graph, e2e_pipe_steps)
        if e2e_ms > e2e_streams_ms:
            e2e_ms, e2e_mode = e2e_streams_ms, "host wall clock, %d steps in flight (copy-in / operator / copy-out streams)" % DEPTH
    e2e_check = bool(torch.equal(slots[1]["h_c"], slots[0]["h_c"]) and
                     torch.equal(slots[0]["h_c"], slots[0]["out"].cpu()))

    sampler.stop_flag = True
    sampler.join(timeout=1.0)

    # ---- first step after B appears on rank 0 (sharded workload, several ranks): broadcast of all of B and then
    # the product, against B travelling in 256-column panels with every panel multiplied as it arrives
    first_step = None
    if world > 1 and args.workload == "sharded":
        a_s, bq_s, bs_s, out_s = sets[0]
        nbc = a_s.shape[1] // 32
        dt_s = void.DistributedVOIDTensor(a_s, void.ShardingStrategy.ROW_WISE, world, rank, (info["M"], info["K"]),
                                          (0, 0), (0, nbc))

        def timed_once(fn):
            torch.cuda.synchronize()
            dist.barrier()
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record()
            fn()
            f1.record()
            torch.cuda.synchronize()
            return f0.elapsed_time(f1)

        def serial():
            void.broadcast_b(bq_s, src=0, scales=bs_s)
            void.void_spmm_int8(a_s, bq_s, bs_s, out_s)

        def overlapped():
            void.broadcast_spmm_overlapped(dt_s, bq_s, bs_s, src=0, panel_cols=256, out=out_s)

        for fn in (serial, overlapped):                 # warm both paths (allocations, NCCL channels)
            timed_once(fn)
        ts = torch.tensor([min(timed_once(serial) for _ in range(3)), min(timed_once(overlapped) for _ in range(3))],
                          dtype=torch.float64, device=dev)
        dist.all_reduce(ts, op=dist.ReduceOp.MAX)
        first_step = {"broadcast_then_spmm_ms": float(ts[0]), "overlapped_panels_ms": float(ts[1]), "panel_cols": 256}

    strong = None
    if world > 1 and args.workload == "headline" and not args.no_strong:
        strong = strong_scaling_record(torch, dist, void, workloads, _lib, dev, rank, world)
    # ---- aggregate over ranks: max time, summed work
    t = torch.tensor([ms_total, e2e_ms, e2e_serial_ms, ms_min], dtype=torch.float64, device=dev)
    work = torch.tensor([ops_per_step_local, float(np.mean(nnz_local))], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(work, op=dist.ReduceOp.SUM)
    ms_total, e2e_ms, e2e_serial_ms, ms_min = (float(x) for x in t.tolist())
    ops_per_step, nnz_total = (float(x) for x in work.tolist())

    if rank == 0:
        ms_per_step = ms_total / K_steps
        value = ops_per_step / (ms_per_step * 1e-3) / 1e12
        peaks = measured_peaks()
        achieved = bytes_per_step / (ms_per_step * 1e-3) / 1e9
        ops_per_byte = ops_per_step_local / bytes_per_step
        clocks = sampler.summary()
        # ops/byte above (dense 8-bit peak / HBM peak) makes the tensor cores the bound; the 8-bit peak is
        # taken as twice the measured bf16 GEMM rate (the ratio of the nominal dense figures)
        # (fp16: the bf16 rate itself; fp32 operands as TF32: half of it)
        traffic, traffic_source = profiled_traffic(args.workload) if world == 1 else (None, None)
        peak_tops = {"tf32": 0.5, "f16": 1.0}.get(kind, 2.0) * peaks["bf16_tflops"]
        tensor_bound = ops_per_byte > peak_tops * 1e12 / (peaks["hbm_gbs"] * 1e9)
        local_tops = ops_per_step_local / (ms_per_step * 1e-3) / 1e12
        roofline = {"bound": "tensor" if tensor_bound else "hbm",
                    "achieved": local_tops if tensor_bound else achieved,
                    "peak": peak_tops if tensor_bound else peaks["hbm_gbs"],
                    "unit": "TOPS" if tensor_bound else "GB/s",
                    "frac": (local_tops / peak_tops) if tensor_bound else achieved / peaks["hbm_gbs"],
                    "traffic": traffic, "traffic_source": traffic_source,
                    "peak_source": peaks["source"] + (" (2 x bf16 GEMM)" if tensor_bound else " (copy)"),
                    "algorithmic_bytes_per_launch": bytes_per_step, "algorithmic_ops_per_launch": ops_per_step_local,
                    "ops_per_byte": ops_per_byte, "hbm_gbs_achieved": achieved, "kernel_us": ms_per_step * 1e3}
        line = {
            "metric": METRIC, "value": value, "unit": "TOPS", "n_gpus": world, "steps": K_steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if args.workload == "sharded" else "weak",
            "vs_baseline": vs_published(args, world, ms_per_step),
            "dtype": kind, "data": "synthetic",
            "config": workload_config(args, world),
            "run": {"nnz_tiles_mean_all_gpus": nnz_total, "input_copies": len(sets), "cuda_graph": not args.no_graph,
                    "timed_launches": passes * K_steps, "passes_of_k_steps": passes, "timed_ms": ms_total * passes,
                    "ms_per_step_min_pass": ms_min / K_steps, "b_broadcast_ms": bcast_ms, "first_step": first_step},
            "strong_scaling": strong,
            "roofline": roofline,
            "e2e": {"value": ops_per_step / (e2e_ms * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(h_b.numel() + h_s.numel() * 4),
                    "d2h_bytes_per_step": int(h_c.numel() * h_c.element_size()),
                    "mode": e2e_mode + E2E_WHAT,
                    "timed_steps": e2e_pipe_steps,
                    "one_step_at_a_time_ms": e2e_serial_ms,
                    "one_step_at_a_time_value": ops_per_step / (e2e_serial_ms * 1e-3) / 1e12,
                    "results_identical_across_slots": e2e_check},
            "gpu_launches": passes * K_steps,
            "clocks": clocks,
        }
        if not args.no_cpu_baseline and world == 1 and args.workload not in ("sharded", "mid"):
            from oracle import void_oracle as vo
            cfg, run, cores = cpu_workload(args, np, torch, vo)
            run()
            t0 = time.perf_counter()
            n = 0
            while n < 5000 and time.perf_counter() - t0 < 10.0:     # about 10 s of CPU work
                run()
                n += 1
            dt = (time.perf_counter() - t0) / n
            line["cpu_baseline"] = {"value": cfg["ops"] / dt / 1e12, "unit": "TOPS", "cores": cores, "kind": "port",
                                    "sample": "whole workload x %d runs (%.1f s), %s" % (n, dt * n, cfg["how"])}
            if args.workload != "powerlaw":
              try:
                # the reference's only non-Triton compute path, its dispatch fallback torch.mm(a.to_dense(), B) in
                # fp32 (void/dispatch.py:261-267), on the same host cores; to_dense is outside the timed region
                dense = sets[0][0].to_dense().float().cpu() if hasattr(sets[0][0], "to_dense") else None
                if dense is None:
                    src = sets[0][0]
                    vals = src.values.float() if hasattr(src, "values") else src.values_fp8.float()
                    dense = void.VOIDTensor(vals, src.block_rows, src.block_cols, torch.zeros(0), src.shape, (32, 32),
                                            0, src.n_blocks, 0.0).to_dense().cpu()
                b_host = torch.randn(dense.shape[1], N)
                torch.mm(dense, b_host)
                t0 = time.perf_counter()
                n = 0
                while n < 50 and time.perf_counter() - t0 < 5.0:
                    torch.mm(dense, b_host)
                    n += 1
                dtd = (time.perf_counter() - t0) / n
                line["cpu_baseline"]["dense_fallback"] = {
                    "ms": dtd * 1e3, "value": cfg["ops"] / dtd / 1e12, "unit": "TOPS over the nonzero tiles",
                    "what": "torch.mm(a.to_dense(), B) fp32 on %d threads: the reference's dispatch fallback" % torch.get_num_threads()}
              except Exception as ex:       # an extra datum: never let it take the bench line down
                print("bench.py: dense fallback timing skipped (%r)" % (ex,), file=sys.stderr)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
