"""Benchmark of the block-sparse attention forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (`config.workload`): the forward of B=1, H=1, N=17536, D=64, fp16, 64x64 block mask with
Bernoulli(0.1) blocks plus the diagonal, q,k,v ~ N(0,1), sm_scale = 1/8 — synthetic, seeded,
standing in for the reference's kernel-test.py inputs.  At N GPUs every rank runs its own head of
that shape (weak scaling, no collective on the data path).

One step = the whole forward path on resident inputs: one launch of the forward kernel, which
lists the kept key blocks of each mask row itself (no separate list kernel).  `value` is
active-tile TFLOP/s = listed tiles * 4*64*64*64 FLOP / step time; L2 is flushed (untimed) between
steps because the inputs are smaller than L2.  `roofline` times the forward kernel alone with its
own CUDA events inside the same steps.  `e2e` runs the public op flash_attention_custom_mask from
pinned host buffers (H2D of q,k,v,mask and D2H of O inside the timed region).  `cpu_baseline` /
`--impl reference` time the reference's naive matmul + masked softmax arithmetic
(kernel-test.py:37-40) on the host cores.  `extra` holds the other BASELINE.json configurations
(sharded over the ranks with fa2_custom_mask.sharding when N > 1), the HBM-bound kernels, and the
reference's own Triton kernel timed on the same GPU from an unmodified copy, if one is present.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "customize-block-sparse-attention-with-triton_b200")
for _p in (PKG, ROOT):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

N_CTX, HEAD_DIM, DENSITY, SM_SCALE = 17536, 64, 0.1, 0.125
FLOP_PER_TILE = 4 * 64 * 64 * HEAD_DIM
WORKLOAD = "fwd fp16 B=1,H=1,N=17536,D=64, 64x64 block mask Bernoulli(0.1)+diagonal (per GPU)"
METRIC = "fwd_active_tile_tflops_N17536_d64_p0.1"
# DRAM bytes (read + write) of one forward-kernel launch on this workload as an ncu capture of it
# counted them (dram__bytes_read.sum + dram__bytes_write.sum); not measured by this script.
FWD_KERNEL_DRAM_BYTES = 6_878_464
CONFIG = {"workload": WORKLOAD, "data": "seeded synthetic q,k,v ~ N(0,1) and block mask"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured"
    return 1590.0, 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU while the timed region runs: NVML from a
    thread every two milliseconds (read-only queries), or nvidia-smi at its finest interval if the
    NVML module is missing."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    REASON_BITS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
                   0x4: "sw_power_cap"}

    def __init__(self, index):
        self.proc = None
        self.thread = None
        self.samples = []
        try:
            import threading
            import pynvml
            pynvml.nvmlInit()
            handle = None
            try:
                uuid = str(torch.cuda.get_device_properties(index).uuid)
                handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            reasons_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            self.stop_flag = threading.Event()

            def loop():
                while not self.stop_flag.is_set():
                    try:
                        self.samples.append((float(pynvml.nvmlDeviceGetClockInfo(
                            handle, pynvml.NVML_CLOCK_SM)), int(reasons_fn(handle))))
                    except Exception:
                        pass
                    time.sleep(0.002)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.thread is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            sm = [s[0] for s in self.samples]
            reasons = set()
            for _, bits in self.samples:
                for bit, name in self.REASON_BITS.items():
                    if bits & bit:
                        reasons.add(name)
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_mhz,
                    "reasons": sorted(reasons), "samples": len(sm), "source": "nvml"}
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
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm), "source": "nvidia-smi"}


def synth_qkv(B, H, N, seed, dtype, n=3):
    """n seeded tensors ~ N(0,1) of shape [B,H,N,64], generated on the host in fp32 then cast."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    return [torch.randn(B, H, N, HEAD_DIM, generator=g).to(dtype) for _ in range(n)]


def synth_block_mask(B, H, nb, density, seed, causal=False):
    """Seeded Bernoulli(density) block mask with the diagonal forced on; `causal` samples only the
    blocks below the diagonal."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    m = torch.rand(B, H, nb, nb, generator=g) < density
    if causal:
        m = torch.tril(m, diagonal=-1)
    return m | torch.eye(nb, dtype=torch.bool)


def make_inputs(seed, device=None, pinned=False):
    q, k, v = synth_qkv(1, 1, N_CTX, seed, torch.float16)
    mask = synth_block_mask(1, 1, N_CTX // 64, DENSITY, seed)
    tiles = int(mask.sum())
    if pinned:
        return [t.pin_memory() for t in (q, k, v, mask)], tiles
    if device is not None:
        return [t.to(device) for t in (q, k, v, mask)], tiles
    return [q, k, v, mask], tiles


CPU_SAMPLE_ROWS = 4096  # query rows of the workload that one CPU step computes (all keys)
CPU_SAMPLE = ("first 4096 of the 17536 query rows against all keys, fp32 naive matmul + "
              "masked softmax (kernel-test.py:37-40)")


def cpu_sample(q, k, v, mask):
    """fp32 host tensors of the bounded CPU sample and the number of listed tiles it covers."""
    rows = CPU_SAMPLE_ROWS
    sub = mask[:, :, : rows // 64].cpu()
    dense = sub.repeat_interleave(64, dim=-2).repeat_interleave(64, dim=-1)
    return (q[:, :, :rows].float().cpu(), k.float().cpu(), v.float().cpu(), dense), int(sub.sum())


def cpu_reference_step(q, k, v, dense, threads):
    """One pass of the reference's naive path on the host cores over the sample."""
    from oracle import oracle
    torch.set_num_threads(threads)
    t0 = time.perf_counter()
    out = oracle.naive_cpu_forward(q, k, v, dense, SM_SCALE)
    dt = time.perf_counter() - t0
    return dt, out


def run_reference(args, rank, world):
    """--impl reference: the naive matmul + masked softmax on the host cores, rank 0 only."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    (q, k, v, mask), _ = make_inputs(seed=2)
    (q, k, v, dense), tiles = cpu_sample(q, k, v, mask)
    for _ in range(args.warmup):
        cpu_reference_step(q, k, v, dense, threads)
    times = [cpu_reference_step(q, k, v, dense, threads)[0] for _ in range(args.steps)]
    total = sum(times)
    value = tiles * FLOP_PER_TILE * args.steps / total / 1e12
    sample = CPU_SAMPLE + ", one sample per step"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": CONFIG,
        "path": "naive matmul + masked softmax on host cores",
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }))


class Timer:
    """CUDA-event timing of one call at a time on the current stream, L2 flushed (untimed) before
    every timed call."""

    def __init__(self, dev, flush):
        self.dev, self.flush = dev, flush

    def times(self, fn, iters, warm=3):
        for _ in range(warm):
            fn()
        out = []
        for _ in range(iters):
            self.flush.zero_()
            a = torch.cuda.Event(enable_timing=True)
            b = torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize(self.dev)
            out.append(a.elapsed_time(b))
        return out

    def median(self, fn, iters, warm=3):
        return statistics.median(self.times(fn, iters, warm))


def device_problem(dev, B, H, N, p, dtype, seed, causal=False, n=3):
    g = torch.Generator(device=dev).manual_seed(seed)
    t = [torch.randn(B, H, N, HEAD_DIM, generator=g, device=dev).to(dtype) for _ in range(n)]
    nb = N // 64
    m = torch.rand(B, H, nb, nb, generator=g, device=dev) < p
    if causal:
        m = torch.tril(m, -1)
    m |= torch.eye(nb, dtype=torch.bool, device=dev)
    return t, m


def sharded_measurements(dev, timer, rank, world, peak_tf):
    """BASELINE.json configurations 3 (row split of the one head), 4 and 5 ((batch, head) split),
    partitioned over the ranks by fa2_custom_mask.sharding.plan: strong scaling, no collective on
    the data path.  Every rank times its own share; the job's time is the slowest rank's."""
    import torch.distributed as dist
    from fa2_custom_mask import (attention_backward, attention_forward, attention_forward_masked,
                                 build_tile_lists, sharding)

    def job(ms, tiles):
        t = torch.tensor([ms, float(tiles)], dtype=torch.float64, device=dev)
        if world > 1:
            both = [torch.zeros_like(t) for _ in range(world)]
            dist.all_gather(both, t)
            ms = max(float(x[0]) for x in both)
            tiles = sum(float(x[1]) for x in both)
        return ms, tiles

    out = {}
    # config 3, one head: fewer (b, h) units than ranks -> query-block rows, balanced by tiles
    (q, k, v, mask), _ = make_inputs(seed=2, device=dev)
    row_tiles = mask[0, 0].sum(-1).tolist()
    kind, (r0, r1) = sharding.plan(1, 1, world, rank, row_tiles) if world > 1 else ("rows", (0, len(row_tiles)))
    o = torch.empty_like(q)
    lse2 = torch.empty(1, 1, N_CTX, dtype=torch.float32, device=dev)
    ms = timer.median(lambda: attention_forward_masked(q, k, v, mask, SM_SCALE, rows=(r0, r1),
                                                       out=(o, lse2)), 20) if r1 > r0 else 0.0
    ms, tiles = job(ms, sum(row_tiles[r0:r1]))
    tf = tiles * FLOP_PER_TILE / (ms * 1e-3) / 1e12
    out["cfg3_H1_N17536_p0.1_f16_row_split"] = {
        "split": "query-block rows by listed tiles", "ranks": world, "tiles": tiles, "fwd_ms": ms,
        "fwd_tflops": tf, "fwd_frac_of_measured_peak_per_gpu": tf / world / peak_tf}
    del q, k, v, mask, o, lse2

    specs = [("cfg4_H32_N32000_p0.1_bf16", 1, 32, 32000, 0.1, False, False),
             ("cfg5_B2_H16_N16384_causal_p0.25_bf16", 2, 16, 16384, 0.25, True, True)]
    for name, B, H, N, p, causal, with_bwd in specs:
        a, b = sharding.shard_heads(B * H, world, rank)
        units = b - a
        rec = {"split": "(batch, head)", "ranks": world}
        if units > 0:
            # this rank's (b, h) units as a batch of single heads, seeded by the unit index range
            (q, k, v, do), m = device_problem(dev, units, 1, N, p, torch.bfloat16, seed=1000 * len(name) + a,
                                              causal=causal, n=4)
            lists = build_tile_lists(m, want_csc=with_bwd)
            tiles = int(m.sum())
            o = torch.empty_like(q)
            lse2 = torch.empty(units, 1, N, dtype=torch.float32, device=dev)
            fms = timer.median(lambda: attention_forward(q, k, v, lists, SM_SCALE, out=(o, lse2)), 5)
            bms = timer.median(lambda: attention_backward(q, k, v, o, lse2, do, lists, SM_SCALE), 5) \
                if with_bwd else 0.0
            del q, k, v, do, m, lists, o, lse2
        else:
            tiles, fms, bms = 0, 0.0, 0.0
        fms, total = job(fms, tiles)
        ftf = total * FLOP_PER_TILE / (fms * 1e-3) / 1e12
        rec.update({"tiles": total, "fwd_ms": fms, "fwd_tflops": ftf,
                    "fwd_frac_of_measured_peak_per_gpu": ftf / world / peak_tf})
        if with_bwd:
            bms, _ = job(bms, tiles)
            btf = total * 10 * 64 * 64 * HEAD_DIM / (bms * 1e-3) / 1e12
            rec.update({"bwd_ms": bms, "bwd_tflops": btf,
                        "bwd_frac_of_measured_peak_per_gpu": btf / world / peak_tf})
        out[name] = rec
    return out


REF_CHILD = r"""
import json, sys, time, torch
sys.path.insert(0, sys.argv[1])
from fa2_custom_mask.fa2_custom_mask import build_groups_from_block_mask, flash_attention_custom_mask
from fa2_custom_mask.fa2_fwd import _attn_fwd
dev = "cuda"
flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
out = {}
for name, B, H, N, p, dt in json.loads(sys.argv[2]):
    dtype = torch.float16 if dt == "f16" else torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(len(name))
    q, k, v = (torch.randn(B, H, N, 64, generator=g, device=dev).to(dtype) for _ in range(3))
    nb = N // 64
    m = (torch.rand(B, H, nb, nb, generator=g, device=dev) < p) | torch.eye(nb, dtype=torch.bool, device=dev)
    flash_attention_custom_mask(q, k, v, m, 0.125); torch.cuda.synchronize()   # autotune
    t0 = time.perf_counter(); flash_attention_custom_mask(q, k, v, m, 0.125); torch.cuda.synchronize()
    whole_ms = 1e3 * (time.perf_counter() - t0)
    groups, nlist = build_groups_from_block_mask(m)
    M = torch.empty(B, H, N, device=dev, dtype=torch.float32); o = torch.empty_like(q)
    def kern():
        _attn_fwd[(groups.shape[0],)](q, k, v, groups, nlist, 0.125, M, o, *q.stride(), *k.stride(),
                                       *v.stride(), *o.stride(), B, H, N, HEAD_DIM=64)
    for _ in range(3): kern()
    ts = []
    for _ in range(10):
        flush.zero_()
        a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
        a.record(); kern(); b.record(); torch.cuda.synchronize(); ts.append(a.elapsed_time(b))
    ts.sort()
    tiles = int(m.sum())
    out[name] = {"tiles": tiles, "kernel_ms": ts[len(ts) // 2], "whole_call_ms": whole_ms,
                 "kernel_tflops": tiles * 1048576 / (ts[len(ts) // 2] * 1e-3) / 1e12}
    del q, k, v, m, groups, nlist, M, o
print("REFJSON " + json.dumps(out))
"""


def reference_triton_on_box():
    """The reference's own forward (`_attn_fwd`, autotuned, from an unmodified copy of the
    reference under baseline/_ref if one travelled with the tree) on this GPU: kernel alone
    (pre-built groups, L2 flushed, CUDA events, median of 10) and its whole public call, which also
    runs the reference's Python list loop.  A comparison record only."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.exists(os.path.join(ref_dir, "fa2_custom_mask", "fa2_fwd.py")):
        return {"unavailable": "no copy of the reference under baseline/_ref"}
    cases = [["headline_H1_N17536_p0.1_f16", 1, 1, 17536, 0.1, "f16"],
             ["H8_N17536_p0.1_f16", 1, 8, 17536, 0.1, "f16"],
             ["dense_H1_N17536_f16", 1, 1, 17536, 1.0, "f16"],
             ["cfg4_H32_N32000_p0.1_bf16", 1, 32, 32000, 0.1, "bf16"]]
    try:
        proc = subprocess.run([sys.executable, "-c", REF_CHILD, ref_dir, json.dumps(cases)],
                              capture_output=True, text=True, timeout=900)
    except subprocess.TimeoutExpired:
        return {"unavailable": "the reference's child process ran past 900 s"}
    for line in proc.stdout.splitlines():
        if line.startswith("REFJSON "):
            return json.loads(line[8:])
    return {"unavailable": "the reference did not run here: " + proc.stderr.strip()[-300:]}


def single_gpu_measurements(dev, timer, peak_tf, peak_gbs):
    """Kernels timed alone on one GPU, L2 flushed before every timed call.  Reported next to the
    headline, never as `value`."""
    from fa2_custom_mask import (_lib, attention_forward, build_tile_lists,
                                 flash_attention_custom_mask, reduce_dense_mask)
    lib = _lib.load()
    out = {}
    for name, B, H, N, p in (("fwd_kernel_test_shape_H8_N17536_p0.1_f16", 1, 8, 17536, 0.1),
                             ("fwd_N17536_dense_f16", 1, 1, 17536, 1.0)):
        (q, k, v), m = device_problem(dev, B, H, N, p, torch.float16, seed=len(name))
        lists = build_tile_lists(m, want_csc=False)
        tiles = int(m.sum())
        o = torch.empty_like(q)
        lse2 = torch.empty(B, H, N, dtype=torch.float32, device=dev)
        ms = timer.median(lambda: attention_forward(q, k, v, lists, SM_SCALE, out=(o, lse2)), 10)
        tf = tiles * FLOP_PER_TILE / (ms * 1e-3) / 1e12
        out[name] = {"tiles": tiles, "fwd_ms": ms, "fwd_tflops": tf, "fwd_frac_of_measured_peak": tf / peak_tf}
        del q, k, v, m, lists, o, lse2
    # the forward from a DENSE boolean mask: mask reduction + forward in one public call
    # (BASELINE.json configs 2 and 3 "including dense-mask -> block preprocessing")
    for N in (6400, 17536):
        (q, k, v), m = device_problem(dev, 1, 1, N, DENSITY, torch.float16, seed=N)
        dense = m.repeat_interleave(64, dim=-2).repeat_interleave(64, dim=-1)
        tiles = int(m.sum())
        with torch.no_grad():
            ms_dense = timer.median(lambda: flash_attention_custom_mask(q, k, v, dense, SM_SCALE), 20)
            ms_block = timer.median(lambda: flash_attention_custom_mask(q, k, v, m, SM_SCALE), 20)
            ms_reduce = timer.median(lambda: reduce_dense_mask(dense), 20)
        out[f"fwd_from_dense_mask_N{N}_p0.1_f16"] = {
            "tiles": tiles, "ms_with_mask_preprocessing": ms_dense, "ms_from_block_mask": ms_block,
            "mask_reduce_ms": ms_reduce, "mask_reduce_GBps": N * N / (ms_reduce * 1e-3) / 1e9,
            "mask_reduce_frac_of_measured_hbm": N * N / (ms_reduce * 1e-3) / 1e9 / peak_gbs}
        del q, k, v, m, dense
    dense = synth_block_mask(1, 1, 500, DENSITY, seed=32000).to(dev)
    dense = dense.repeat_interleave(64, dim=-2).repeat_interleave(64, dim=-1)
    ms = timer.median(lambda: reduce_dense_mask(dense), 20)
    gbs = 32000 * 32000 / (ms * 1e-3) / 1e9
    out["mask_reduce_N32000"] = {"ms": ms, "GBps": gbs, "frac_of_measured_hbm": gbs / peak_gbs}
    del dense
    # tile lists (row and column lists) from the block mask: bytes = the mask read once, the four
    # list arrays written once
    for name, B, H, N, p, causal in (("cfg3_H1_N17536", 1, 1, 17536, 0.1, False),
                                     ("cfg4_H32_N32000", 1, 32, 32000, 0.1, False),
                                     ("cfg5_B2_H16_N16384_causal", 2, 16, 16384, 0.25, True)):
        g = torch.Generator(device=dev).manual_seed(N)
        nb = N // 64
        m = torch.rand(B, H, nb, nb, generator=g, device=dev) < p
        if causal:
            m = torch.tril(m, -1)
        m |= torch.eye(nb, dtype=torch.bool, device=dev)
        nnz, rows = int(m.sum()), B * H * nb
        ms = timer.median(lambda: build_tile_lists(m, want_csr=True, want_csc=True), 20)
        nbytes = B * H * nb * nb + 4 * (2 * nnz + 2 * (rows + 1))
        out[f"tile_lists_{name}"] = {"ms": ms, "bytes": nbytes, "GBps": nbytes / (ms * 1e-3) / 1e9,
                                     "frac_of_measured_hbm": nbytes / (ms * 1e-3) / 1e9 / peak_gbs,
                                     "note": "three launches over a few MB: launch-latency bound"}
        del m
    # delta (HBM-bound: O and dO read once, one float per row written), config 5 shape
    B, H, N = 2, 16, 16384
    o, do = (torch.randn(B, H, N, HEAD_DIM, device=dev).to(torch.bfloat16) for _ in range(2))
    delta = torch.empty((B, H, N), dtype=torch.float32, device=dev)
    ms = timer.median(lambda: lib.bsa_attn_bwd_delta(
        _lib.ptr(o), _lib.ptr(do), _lib.strides4(o), _lib.ptr(delta), _lib.dtype_code(o.dtype),
        B, H, N, HEAD_DIM, _lib.stream_ptr(dev)), 10)
    gbs = (2 * o.numel() * o.element_size() + delta.numel() * 4) / (ms * 1e-3) / 1e9
    out["bwd_delta_cfg5"] = {"ms": ms, "GBps": gbs, "frac_of_measured_hbm": gbs / peak_gbs}
    del o, do, delta
    # head-wise token reorder on the reference's own grid (13 x 30 x 45 image tokens), sized past L2
    from fa2_custom_mask import apply_head_wise_reorder, permute_qkv_triton
    Bv, Hv, Fv, Yv, Xv = 2, 48, 13, 30, 45
    x = torch.randn(Bv, Hv, Fv * Yv * Xv, HEAD_DIM, device=dev, dtype=torch.float16)
    orders = torch.tensor([[0, 1, 2], [0, 2, 1], [1, 0, 2], [1, 2, 0], [2, 0, 1], [2, 1, 0]],
                          device=dev, dtype=torch.int32)[torch.arange(Hv, device=dev) % 6]
    ms = timer.median(lambda: apply_head_wise_reorder(x, orders, Fv, Yv, Xv), 10)
    gbs = 2 * x.numel() * x.element_size() / (ms * 1e-3) / 1e9
    out["reorder_B2_H48_T17550_f16"] = {"ms": ms, "GBps": gbs, "frac_of_measured_hbm": gbs / peak_gbs}
    del x
    # the whole wrapper as a model calls it: q, k, v with 226 text tokens in front, image tokens
    # gathered out of the slice and copied back in place (two passes per tensor; bytes counted are
    # those of one pass, so 0.5 of the copy bandwidth is the ceiling)
    qkv = [torch.randn(Bv, Hv, 226 + Fv * Yv * Xv, HEAD_DIM, device=dev, dtype=torch.float16)
           for _ in range(3)]
    plan = {"permute": (torch.arange(Hv, device=dev) % 6)[None]}
    ms = timer.median(lambda: permute_qkv_triton(*qkv, plan, 0, Fv, Yv, Xv, 226), 10)
    gbs = 3 * 2 * Bv * Hv * Fv * Yv * Xv * HEAD_DIM * 2 / (ms * 1e-3) / 1e9
    out["permute_qkv_B2_H48_T226+17550_f16"] = {"ms": ms, "GBps_one_pass": gbs,
                                                "frac_of_measured_hbm": gbs / peak_gbs}
    del qkv
    return out


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    from fa2_custom_mask import (attention_forward_masked, check_status,
                                 flash_attention_custom_mask, new_status_word)
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    (q, k, v, mask), tiles = make_inputs(seed=2 + rank, device=dev)
    # 1 GiB: the untimed flush also keeps the GPU busy for a few hundred microseconds, so that the
    # host has enqueued the timed call before the device gets to it (no host gap inside the events)
    flush = torch.empty(1024 * 1024 * 1024, dtype=torch.uint8, device=dev)
    status = new_status_word(dev)
    out_buf = (torch.empty_like(q), torch.empty(1, 1, N_CTX, dtype=torch.float32, device=dev))

    def step():
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record()
        attention_forward_masked(q, k, v, mask, SM_SCALE, status=status, out=out_buf)
        b.record()
        return a, b

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(args.warmup):
        flush.zero_()
        step()
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    # A step is one launch of the forward kernel, so one pair of events per step gives both the
    # step time and the kernel's launch duration (a second pair around the first only added the
    # cost of two more event records to the step).
    step_ev = []
    for _ in range(args.steps):
        flush.zero_()
        step_ev.append(step())
    barrier()
    check_status(status)
    step_ms = sum(a.elapsed_time(b) for a, b in step_ev)
    kern_ms = step_ms

    # ---- end to end: public op, pinned host inputs, D2H of the output ----
    # q, k, v and the mask of a step lie in ONE pinned staging buffer and cross PCIe in one copy;
    # the op is called on views of its device copy
    (hq, hk, hv, hmask), _ = make_inputs(seed=2 + rank)
    parts = [hq.view(torch.uint8).reshape(-1), hk.view(torch.uint8).reshape(-1),
             hv.view(torch.uint8).reshape(-1), hmask.view(torch.uint8).reshape(-1)]
    offs = [0]
    for t in parts:
        offs.append((offs[-1] + t.numel() + 255) // 256 * 256)
    staging = torch.empty(offs[-1], dtype=torch.uint8).pin_memory()
    for t, o0 in zip(parts, offs):
        staging[o0:o0 + t.numel()].copy_(t)
    d_staging = torch.empty_like(staging, device=dev)
    shp = hq.shape

    def dview(i, dtype, shape):
        n = parts[i].numel()
        return d_staging[offs[i]:offs[i] + n].view(dtype).reshape(shape)

    dq, dk, dv = (dview(i, torch.float16, shp) for i in range(3))
    dm = dview(3, torch.bool, hmask.shape)
    h_out = torch.empty_like(hq).pin_memory()

    def e2e_step():
        d_staging.copy_(staging, non_blocking=True)
        with torch.no_grad():
            o = flash_attention_custom_mask(dq, dk, dv, dm, SM_SCALE)
        h_out.copy_(o, non_blocking=True)

    for _ in range(args.warmup):
        e2e_step()
    barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler else None

    red = torch.tensor([step_ms, kern_ms, e2e_ms], dtype=torch.float64, device=dev)
    tl = torch.tensor([float(tiles)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(red, op=dist.ReduceOp.MAX)
        dist.all_reduce(tl, op=dist.ReduceOp.SUM)
    step_ms, kern_ms, e2e_ms = red.tolist()
    total_tiles = tl.item()

    peak_tf, peak_gbs, peak_kind = measured_peaks()
    timer = Timer(dev, flush)
    extra = sharded_measurements(dev, timer, rank, world, peak_tf)
    if rank != 0:
        return

    value = total_tiles * FLOP_PER_TILE * args.steps / (step_ms * 1e-3) / 1e12
    # per-GPU kernel figure: this rank's tiles over its own mean kernel time (max over ranks)
    achieved = (total_tiles / world) * FLOP_PER_TILE * args.steps / (kern_ms * 1e-3) / 1e12
    h2d = staging.numel()
    d2h = h_out.numel() * h_out.element_size()
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "config": CONFIG,
        "path": {"step": "forward kernel with in-kernel tile listing from the block mask",
                 "tiles_per_gpu": total_tiles / world, "sharding": "one head per GPU",
                 "l2": "flushed between steps (1 GiB write, untimed)"},
        "fwd_kernel_ms": kern_ms / args.steps,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                     "frac": achieved / peak_tf, "traffic": FWD_KERNEL_DRAM_BYTES,
                     "traffic_source": "ncu capture of this workload (profiles/), not measured in this run",
                     "kernel": "attn_fwd_kernel", "peak_kind": peak_kind + " (burst bf16 GEMM)"},
        "e2e": {"value": total_tiles * FLOP_PER_TILE * args.steps / (e2e_ms * 1e-3) / 1e12,
                "unit": "TFLOP/s", "ms_per_step": e2e_ms / args.steps,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": args.steps,
        "clocks": clocks,
        "extra": extra,
    }
    if world == 1:
        # the headline step over many more launches than the driver's --steps: run-to-run noise
        ts = sorted(timer.times(lambda: attention_forward_masked(q, k, v, mask, SM_SCALE, out=out_buf), 200))
        extra["headline_200_launches"] = {
            "median_ms": ts[100], "min_ms": ts[0], "p90_ms": ts[180],
            "median_tflops": tiles * FLOP_PER_TILE / (ts[100] * 1e-3) / 1e12,
            "median_frac_of_measured_peak": tiles * FLOP_PER_TILE / (ts[100] * 1e-3) / 1e12 / peak_tf}
        extra.update(single_gpu_measurements(dev, timer, peak_tf, peak_gbs))
        threads = os.cpu_count() or 1
        (cq, ck, cv, dense), sample_tiles = cpu_sample(q, k, v, mask)
        cpu_reference_step(cq, ck, cv, dense, threads)
        times = [cpu_reference_step(cq, ck, cv, dense, threads)[0] for _ in range(7)]
        line["cpu_baseline"] = {
            "value": sample_tiles * FLOP_PER_TILE / statistics.median(times) / 1e12,
            "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": CPU_SAMPLE + ", 1 warm-up + median of 7"}
        del q, k, v, mask, flush
        torch.cuda.empty_cache()
        extra["reference_triton_on_box"] = reference_triton_on_box()
    print(json.dumps(line))


PROFILE_CASES = ("fwd_headline", "fwd_dense", "fwd_bwd_causal", "mask_reduce", "tile_lists", "delta",
                 "reorder")


def run_profile_case(name, iters):
    """One small case of one kernel family, launched `iters` times and nothing else: the command a
    profiler capture is pointed at (a few hundred MB on the device at most, a handful of
    launches).  Prints nothing that is a benchmark value."""
    from fa2_custom_mask import (_lib, apply_head_wise_reorder, attention_backward,
                                 attention_forward, attention_forward_masked, build_tile_lists,
                                 reduce_dense_mask)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if name in ("fwd_headline", "fwd_dense"):
        (q, k, v), m = device_problem(dev, 1, 1, N_CTX, DENSITY if name == "fwd_headline" else 1.0,
                                      torch.float16, seed=3)
        fn = lambda: attention_forward_masked(q, k, v, m, SM_SCALE)
    elif name == "fwd_bwd_causal":
        # BASELINE.json config 5 with 2 x 4 of its 2 x 16 heads
        (q, k, v, do), m = device_problem(dev, 2, 4, 16384, 0.25, torch.bfloat16, seed=5, causal=True, n=4)
        lists = build_tile_lists(m)
        o, lse2, _ = attention_forward(q, k, v, lists, SM_SCALE)
        fn = lambda: (attention_forward(q, k, v, lists, SM_SCALE),
                      attention_backward(q, k, v, o, lse2, do, lists, SM_SCALE))
    elif name == "mask_reduce":
        dense = synth_block_mask(1, 1, N_CTX // 64, DENSITY, seed=1).to(dev)
        dense = dense.repeat_interleave(64, dim=-2).repeat_interleave(64, dim=-1)   # 307 MB > L2
        fn = lambda: reduce_dense_mask(dense)
    elif name == "tile_lists":
        m = synth_block_mask(1, 32, 500, DENSITY, seed=1).to(dev)                   # config 4 mask
        fn = lambda: build_tile_lists(m, want_csr=True, want_csc=True)
    elif name == "delta":
        o, do = (torch.randn(2, 16, 16384, HEAD_DIM, device=dev).to(torch.bfloat16) for _ in range(2))
        delta = torch.empty((2, 16, 16384), dtype=torch.float32, device=dev)
        lib = _lib.load()
        fn = lambda: lib.bsa_attn_bwd_delta(_lib.ptr(o), _lib.ptr(do), _lib.strides4(o), _lib.ptr(delta),
                                            _lib.dtype_code(o.dtype), 2, 16, 16384, HEAD_DIM,
                                            _lib.stream_ptr(dev))
    else:
        x = torch.randn(2, 48, 13 * 30 * 45, HEAD_DIM, device=dev, dtype=torch.float16)  # 216 MB > L2
        orders = torch.tensor([[0, 1, 2], [0, 2, 1], [1, 0, 2], [1, 2, 0], [2, 0, 1], [2, 1, 0]],
                              device=dev, dtype=torch.int32)[torch.arange(48, device=dev) % 6]
        fn = lambda: apply_head_wise_reorder(x, orders, 13, 30, 45)
    for _ in range(iters):
        fn()
    torch.cuda.synchronize(dev)
    print(f"profile case {name}: {iters} iterations done")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--profile-case", default=None, choices=PROFILE_CASES,
                    help="launch one small case --steps times and exit (for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    import __graft_entry__
    if rank == 0:
        __graft_entry__.build()
    if args.profile_case:
        run_profile_case(args.profile_case, args.steps)
        return
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist.barrier()
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
