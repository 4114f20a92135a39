"""Benchmark of the block-sparse attention forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (`config.workload`): the forward of B=1, H=1, N=17536, D=64, fp16, 64x64 block mask with
Bernoulli(0.1) blocks plus the diagonal, q,k,v ~ N(0,1), sm_scale = 1/8 — synthetic, seeded,
standing in for the reference's kernel-test.py inputs.  At N GPUs every rank runs its own head of
that shape (weak scaling, no collective on the data path).

One step = the whole forward path on resident inputs: one launch of the forward kernel, which
lists the kept key blocks of each mask row itself (no separate list kernel).  `value` is active-tile TFLOP/s = listed tiles * 4*64*64*64 FLOP / step time; L2 is flushed
(untimed) between steps because the inputs are smaller than L2.  `roofline` times the forward
kernel alone with its own CUDA events inside the same steps.  `e2e` runs the public op
flash_attention_custom_mask from pinned host buffers (H2D of q,k,v,mask and D2H of O inside the
timed region).  `cpu_baseline` / `--impl reference` time the reference's naive
matmul + masked softmax arithmetic (kernel-test.py:37-40) on the host cores.
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
# DRAM bytes (read + write) of one forward-kernel launch on this workload from the ncu capture
# summarised in profiles/attn_fwd_kernel_N17536_p0.1.md.
FWD_KERNEL_DRAM_BYTES = 6_878_464


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


def make_inputs(seed, device=None, pinned=False):
    from oracle import oracle
    q, k, v = oracle.make_qkv(1, 1, N_CTX, HEAD_DIM, seed=seed, dtype=torch.float16)
    mask = oracle.make_block_mask(1, 1, N_CTX // 64, DENSITY, seed=seed)
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
    from oracle import oracle
    rows = CPU_SAMPLE_ROWS
    sub = mask[:, :, : rows // 64].cpu()
    dense = oracle.expand_block_mask(sub)
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
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "path": "naive matmul + masked softmax on host cores"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }))


def extra_measurements(dev, peak_tf, peak_gbs):
    """Other BASELINE.json configurations, kernels timed alone (CUDA events over back-to-back
    launches, inputs resident, no L2 flush).  Reported next to the headline, never as `value`."""
    from fa2_custom_mask import (attention_backward, attention_forward, build_tile_lists,
                                 reduce_dense_mask)

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(dev)
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize(dev)
        return a.elapsed_time(b) / iters

    def problem(B, H, N, p, dtype, seed, causal=False):
        g = torch.Generator(device=dev).manual_seed(seed)
        t = [torch.randn(B, H, N, HEAD_DIM, generator=g, device=dev).to(dtype) for _ in range(4)]
        nb = N // 64
        m = torch.rand(B, H, nb, nb, generator=g, device=dev) < p
        if causal:
            m = torch.tril(m, -1)
        m |= torch.eye(nb, dtype=torch.bool, device=dev)
        return t, m

    out = {}
    specs = [("fwd_kernel_test_shape_H8_N17536_p0.1_f16", 1, 8, 17536, 0.1, torch.float16, False, False),
             ("fwd_N17536_dense_f16", 1, 1, 17536, 1.0, torch.float16, False, False),
             ("fwd_cfg4_H32_N32000_p0.1_bf16", 1, 32, 32000, 0.1, torch.bfloat16, False, False),
             ("fwd_bwd_cfg5_B2_H16_N16384_causal_p0.25_bf16", 2, 16, 16384, 0.25, torch.bfloat16, True, True)]
    for name, B, H, N, p, dtype, causal, with_bwd in specs:
        (q, k, v, do), m = problem(B, H, N, p, dtype, seed=len(name), causal=causal)
        lists = build_tile_lists(m, want_csc=with_bwd)
        tiles = int(m.sum())
        iters = 20 if tiles < 100000 else 5
        ms = timed(lambda: attention_forward(q, k, v, lists, SM_SCALE), iters)
        tf = tiles * FLOP_PER_TILE / (ms * 1e-3) / 1e12
        rec = {"tiles": tiles, "fwd_ms": ms, "fwd_tflops": tf, "fwd_frac_of_measured_peak": tf / peak_tf}
        if with_bwd:
            o, lse2, _ = attention_forward(q, k, v, lists, SM_SCALE)
            bms = timed(lambda: attention_backward(q, k, v, o, lse2, do, lists, SM_SCALE), iters)
            btf = tiles * 10 * 64 * 64 * HEAD_DIM / (bms * 1e-3) / 1e12
            rec.update({"bwd_ms": bms, "bwd_tflops": btf, "bwd_frac_of_measured_peak": btf / peak_tf})
            # the delta kernel alone (HBM-bound: O and dO read once, one float per row written)
            from fa2_custom_mask import _lib
            lib = _lib.load()
            delta = torch.empty((B, H, N), dtype=torch.float32, device=dev)
            dms = timed(lambda: lib.bsa_attn_bwd_delta(
                _lib.ptr(o), _lib.ptr(do), _lib.strides4(o), _lib.ptr(delta),
                _lib.dtype_code(o.dtype), B, H, N, HEAD_DIM, _lib.stream_ptr(dev)), iters)
            dgb = (2 * o.numel() * o.element_size() + delta.numel() * 4) / (dms * 1e-3) / 1e9
            rec.update({"delta_ms": dms, "delta_GBps": dgb, "delta_frac_of_measured_hbm": dgb / peak_gbs})
        out[name] = rec
        del q, k, v, do, m, lists
    for N in (17536, 32000):
        from oracle import oracle
        dense = oracle.expand_block_mask(oracle.make_block_mask(1, 1, N // 64, DENSITY, seed=N).to(dev))
        ms = timed(lambda: reduce_dense_mask(dense), 20)
        gbs = N * N / (ms * 1e-3) / 1e9
        out[f"mask_reduce_N{N}"] = {"ms": ms, "GBps": gbs, "frac_of_measured_hbm": gbs / peak_gbs}
        del dense
    # head-wise token reorder on the reference's own grid (13 x 30 x 45 image tokens), sized past L2
    from fa2_custom_mask import apply_head_wise_reorder
    Bv, Hv, Fv, Yv, Xv = 2, 48, 13, 30, 45
    x = torch.randn(Bv, Hv, Fv * Yv * Xv, HEAD_DIM, device=dev, dtype=torch.float16)
    orders = torch.tensor([[0, 1, 2], [0, 2, 1], [1, 0, 2], [1, 2, 0], [2, 0, 1], [2, 1, 0]],
                          device=dev, dtype=torch.int32)[torch.arange(Hv, device=dev) % 6]
    ms = timed(lambda: apply_head_wise_reorder(x, orders, Fv, Yv, Xv), 10)
    gbs = 2 * x.numel() * x.element_size() / (ms * 1e-3) / 1e9
    out["reorder_B2_H48_T17550_f16"] = {"ms": ms, "GBps": gbs, "frac_of_measured_hbm": gbs / peak_gbs}
    del x
    # the whole wrapper as a model calls it: q, k, v with 226 text tokens in front, image tokens
    # gathered out of the slice and copied back in place (two passes per tensor; bytes counted are
    # those of one pass, so 0.5 of the copy bandwidth is the ceiling)
    from fa2_custom_mask import permute_qkv_triton
    qkv = [torch.randn(Bv, Hv, 226 + Fv * Yv * Xv, HEAD_DIM, device=dev, dtype=torch.float16)
           for _ in range(3)]
    plan = {"permute": (torch.arange(Hv, device=dev) % 6)[None]}
    ms = timed(lambda: permute_qkv_triton(*qkv, plan, 0, Fv, Yv, Xv, 226), 10)
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
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    status = new_status_word(dev)

    def step():
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record()
        out = attention_forward_masked(q, k, v, mask, SM_SCALE, status=status)
        b.record()
        return out, a, b

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
        _, a, b = step()
        step_ev.append((a, b))
    barrier()
    check_status(status)
    step_ms = sum(a.elapsed_time(b) for a, b in step_ev)
    kern_ms = step_ms

    # ---- end to end: public op, pinned host inputs, D2H of the output ----
    (hq, hk, hv, hmask), _ = make_inputs(seed=2 + rank, pinned=True)
    h_out = torch.empty_like(hq).pin_memory()

    def e2e_step():
        dq, dk, dv, dm = (t.to(dev, non_blocking=True) for t in (hq, hk, hv, hmask))
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
    if rank != 0:
        return

    peak_tf, peak_gbs, peak_kind = measured_peaks()
    value = total_tiles * FLOP_PER_TILE * args.steps / (step_ms * 1e-3) / 1e12
    # per-GPU kernel figure: this rank's tiles over its own mean kernel time (max over ranks)
    achieved = (total_tiles / world) * FLOP_PER_TILE * args.steps / (kern_ms * 1e-3) / 1e12
    h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv, hmask))
    d2h = h_out.numel() * h_out.element_size()
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "step": "forward kernel with in-kernel tile listing from the block mask",
                   "tiles_per_gpu": total_tiles / world, "sharding": "one head per GPU",
                   "l2": "flushed between steps (256 MiB write, untimed)"},
        "fwd_kernel_ms": kern_ms / args.steps,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                     "frac": achieved / peak_tf, "traffic": FWD_KERNEL_DRAM_BYTES,
                     "kernel": "attn_fwd_kernel", "peak_kind": peak_kind + " (burst bf16 GEMM)"},
        "e2e": {"value": total_tiles * FLOP_PER_TILE * args.steps / (e2e_ms * 1e-3) / 1e12,
                "unit": "TFLOP/s", "ms_per_step": e2e_ms / args.steps,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": args.steps,
        "clocks": clocks,
    }
    if world == 1:
        threads = os.cpu_count() or 1
        (cq, ck, cv, dense), sample_tiles = cpu_sample(q, k, v, mask)
        cpu_reference_step(cq, ck, cv, dense, threads)
        times = [cpu_reference_step(cq, ck, cv, dense, threads)[0] for _ in range(7)]
        line["extra"] = extra_measurements(dev, peak_tf, peak_gbs)
        line["cpu_baseline"] = {
            "value": sample_tiles * FLOP_PER_TILE / statistics.median(times) / 1e12,
            "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": CPU_SAMPLE + ", 1 warm-up + median of 7"}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
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
