"""Benchmark of the dilution-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Headline (the JSON line's metric/value): forward + backward of the training-shape
operator, B=4 H=16 T=16384 d=64, bf16 inputs (q,k = 0.5*N(0,1), v = N(0,1),
dout = 1e-2*N(0,1)), fp32 accumulation, as TFLOP/s by the 7-matmul causal count
7 * N * T*(T+1) * D.  One step = one forward + one backward of that batch.
With N GPUs every rank runs its own batch*head slab (weak scaling, no collective).

Also on the line:
  roofline      the dominant kernel (backward main pass) against the measured
                dense-bf16 peak; per-kernel CUDA-event times in `kernels_ms`;
  e2e           the same step through the public op with pinned HOST buffers:
                H2D of q,k,v,dout and D2H of out,dq,dk,dv inside the timed region;
  decode        cached decode tok/s at a 128K KV cache (batch 64 x 16 heads),
                against the measured HBM copy bandwidth;
  cpu_baseline  the CPU oracle timed on this box's host cores on a bounded sample.

--impl reference times the reference's CPU implementation (restated in oracle/)
on the host cores for the same metric.
"""

from __future__ import annotations

import argparse
import importlib
import json
import math
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

TRAIN = dict(B=4, H=16, T=16384, D=64)
DECODE = dict(batch=64, H=16, D=64, L=131072, steps=64)
METRIC = "fwd+bwd TFLOP/s @T=16K,d=64"


def causal_flops(n_rows, t, d, matmuls):
    return matmuls * n_rows * t * (t + 1) * d


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            m = json.load(f)
        return dict(hbm=m["hbm_gbs"], tensor=m["bf16_tflops_sustained"], burst=m["bf16_tflops"],
                    source="measured")
    return dict(hbm=6650.0, tensor=1400.0, burst=1590.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while a region runs."""

    def __init__(self, index):
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                    nv.nvmlDeviceGetCurrentClocksThrottleReasons
                bits = get(self.h)
                for bit, name in names.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def cpu_sample(t, reps):
    """The CPU oracle, forward + autograd backward, one (b,h) row at length t."""
    from oracle import dilution_oracle as O
    g = torch.Generator().manual_seed(1339)
    q, k = (torch.randn(1, 1, t, 64, generator=g) * 0.5 for _ in range(2))
    v = torch.randn(1, 1, t, 64, generator=g)
    dout = torch.randn(1, 1, t, 64, generator=g) * 1e-2
    O.dilution_backward(q[:, :, :256], k[:, :, :256], v[:, :, :256], dout[:, :, :256])   # warm
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        O.dilution_backward(q, k, v, dout)
        times.append(time.perf_counter() - t0)
    return statistics.median(times)


def cpu_baseline_block(t=8192, reps=5):
    sec = cpu_sample(t, reps)
    return {"value": causal_flops(1, t, 64, 7) / sec / 1e12, "unit": "TFLOP/s",
            "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"1 (batch,head) row at T={t}, d=64, fp32 forward + autograd backward, "
                      f"median of {reps}; {os.cpu_count()} logical CPUs"}


def run_reference(args, rank):
    """The reference's CPU path (oracle port of kernels.py:40-68) on the host cores."""
    if rank != 0:
        return
    # torchrun exports OMP_NUM_THREADS=1 to every rank; the other ranks exit without work, so
    # rank 0 takes all the host's cores, as it does when launched without torchrun
    torch.set_num_threads(os.cpu_count() or 1)
    t = 8192
    for _ in range(args.warmup):
        cpu_sample(t, 1)
    times = [cpu_sample(t, 1) for _ in range(args.steps)]
    sec = sum(times) / len(times)
    value = causal_flops(1, t, 64, 7) / sec / 1e12
    sample = (f"each step = 1 (batch,head) row at T={t} of the B4 H16 T16384 workload, fp32 forward + "
              f"autograd backward on {torch.get_num_threads()} host threads")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": {"workload": "train_fwd_bwd_B4_H16_T16384_d64", "sample": sample},
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                             "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def make_train_inputs(dev, rank):
    """Seeded synthetic inputs of the training shape; pinned host copies kept for e2e."""
    B, H, T, D = (TRAIN[x] for x in "BHTD")
    g = torch.Generator().manual_seed(1339 + rank)
    host = {}
    for name, scale, dt in (("q", 0.5, torch.bfloat16), ("k", 0.5, torch.bfloat16),
                            ("v", 1.0, torch.bfloat16), ("dout", 1e-2, torch.float32)):
        x = torch.empty(B, H, T, D, dtype=torch.float32).normal_(generator=g).mul_(scale).to(dt)
        host[name] = x.pin_memory()
    return host, {k: v.to(dev, non_blocking=True) for k, v in host.items()}


def train_step(K, q, k, v, dout):
    q.grad = k.grad = v.grad = None
    out = K.dilution_attention(q, k, v, dot_precision="bf16")
    out.backward(dout)
    return out


def run_ours(args, rank, world):
    pkg = importlib.import_module("dilution-attention_b200")
    K, L = pkg.kernels, pkg._lib
    L.load()
    local = int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    distributed = world > 1
    if distributed:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    peaks = measured_peaks()
    if args.no_train:
        def sync_only():
            if distributed:
                dist.barrier()
            torch.cuda.synchronize()
        decode = run_decode(K, L, dev, rank, world, peaks, sync_only, distributed)
        if rank == 0:
            print(json.dumps({"decode": decode}), flush=True)
        if distributed:
            dist.destroy_process_group()
        return
    B, H, T, D = (TRAIN[x] for x in "BHTD")
    n_rows = B * H

    host, devt = make_train_inputs(dev, rank)
    q, k, v = (devt[x].requires_grad_(True) for x in "qkv")
    dout = devt["dout"]
    torch.cuda.synchronize()

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        train_step(K, q, k, v, dout)
    barrier()

    # --- timed region: K steps, device-resident inputs, CUDA events, per-kernel events on
    launches0 = L.launch_count()
    L.profile(True)
    L.profile_collect()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        barrier()
        start.record()
        for _ in range(args.steps):
            train_step(K, q, k, v, dout)
        stop.record()
        barrier()
    ms = start.elapsed_time(stop)
    prof = L.profile_collect()
    L.profile(False)
    launches = L.launch_count() - launches0
    if distributed:
        tms = torch.tensor([ms], device=dev)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms = tms.item()
    ms_per_step = ms / args.steps
    total_flops = causal_flops(n_rows, T, D, 7) * world
    value = total_flops / (ms_per_step * 1e-3) / 1e12

    # dominant kernel and its roofline (5 of the 7 matmuls live in the backward main pass)
    kernels_ms = {name: tot / cnt for name, (cnt, tot) in prof.items()}
    # algorithmic matmuls per kernel: the backward main pass carries all five backward products,
    # the forward main pass QK^T and share@V; the other passes are recomputation overhead
    share = {"backward_main": 5, "forward_main": 2}
    dom = max(kernels_ms, key=kernels_ms.get) if kernels_ms else None
    roofline = None
    if dom is not None:
        mm = next((m for key, m in share.items() if key in dom), 0)
        achieved = causal_flops(n_rows, T, D, mm) / (kernels_ms[dom] * 1e-3) / 1e12
        # DRAM bytes per launch: ncu dram__bytes_read.sum + dram__bytes_write.sum of this kernel at
        # T=4096 (64 rows, 528 causal 128x128 tiles per row: 1354.26 MB), scaled by the number of
        # causal tiles this launch processes -- the dQ tile reductions dominate it and grow with
        # the tile count.  Only the backward main pass has a captured figure.
        tiles = n_rows * (T // 128) * (T // 128 + 1) // 2
        traffic = 1354.26e6 / (64 * 528) * tiles if "backward_main" in dom else None
        roofline = {"bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peaks["tensor"],
                    "unit": "TFLOP/s", "frac": achieved / peaks["tensor"], "traffic": traffic,
                    "traffic_source": "ncu capture at T=4096 (profiles/train_kernels_T4096_ncu_full.md), "
                                      "scaled by causal 128x128 tiles per launch; bytes",
                    "peak_source": f"{peaks['source']} sustained bf16", "matmuls_in_kernel": mm,
                    "step_frac_of_peak": value / world / peaks["tensor"],
                    # matmul-equivalents the tensor cores actually run per step: QK^T in the row,
                    # column-sum, main, reverse and correction passes (5), share@V, dO V^T, dV, dQ,
                    # dK (5), and the two correction products W Q and W^T K (2); the ones columns
                    # that give row sums and ghat (N = 80 instead of 64) are not counted
                    "executed": {"matmuls_per_step": 12,
                                 "value": value / world * 12 / 7, "unit": "TFLOP/s",
                                 "frac": value / world * 12 / 7 / peaks["tensor"]}}

    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(args, K, host, devt, dev, barrier, distributed, total_flops)
    del devt, q, k, v, dout
    torch.cuda.empty_cache()

    # --- cached decode at a 128K cache (heads sharded across ranks)
    decode = None
    if not args.no_decode:
        decode = run_decode(K, L, dev, rank, world, peaks, barrier, distributed)

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"train_fwd_bwd_B{B}_H{H}_T{T}_d{D}", "rows_per_gpu": n_rows,
                           "global_rows": n_rows * world, "seq_len": T, "head_dim": D,
                           "parallelism": f"batch*head slab per GPU x{world}, no collective",
                           "l2": "inputs exceed L2 (q,k,v 134 MB each, dout/out 268 MB at T=16384)",
                           "flop_count": "7*N*T*(T+1)*D"},
                "roofline": roofline, "kernels_ms": kernels_ms, "e2e": e2e, "gpu_launches": launches,
                "clocks": clocks.summary(), "decode": decode}
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline_block()
        print(json.dumps(line), flush=True)
    if distributed:
        dist.destroy_process_group()


def run_e2e(args, K, host, devt, dev, barrier, distributed, total_flops):
    """The step through the public host-buffer entry point (`dilution_attention_host`): pinned
    HOST q, k, v, dout in; pinned HOST out, dq, dk, dv back.  All copies are inside the timed
    region; the call pipelines row slabs over three streams."""
    import torch.distributed as dist
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    out = torch.empty_like(host["dout"]).pin_memory()
    grads = tuple(torch.empty_like(host[n]).pin_memory() for n in "qkv")

    def e2e_step():
        K.dilution_attention_host(host["q"], host["k"], host["v"], host["dout"], dot_precision="bf16",
                                  device=dev, slabs=8, out=out, grads=grads)

    e2e_step()
    barrier()
    e2e_steps = max(1, min(args.steps, 3))
    start.record()
    for _ in range(e2e_steps):
        e2e_step()
    stop.record()
    barrier()
    e2e_ms = start.elapsed_time(stop) / e2e_steps
    if distributed:
        tms = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        e2e_ms = tms.item()
    h2d = sum(host[n].numel() * host[n].element_size() for n in ("q", "k", "v", "dout"))
    d2h = out.numel() * out.element_size() + sum(x.numel() * x.element_size() for x in grads)
    return {"value": total_flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "path": "dilution_attention_host: 8 row slabs pipelined over copy-in / compute / copy-out streams"}


def run_decode(K, L, dev, rank, world, peaks, barrier, distributed):
    import torch.distributed as dist
    cfg = DECODE
    rows = cfg["rows"] // world                       # heads sharded across ranks
    d, L0, steps = cfg["D"], cfg["L"], cfg["steps"]
    warm = 3
    cap = L0 + steps + warm
    gen = torch.Generator(device=dev).manual_seed(4 + rank)
    kc = torch.empty(rows, cap, d, device=dev, dtype=torch.bfloat16).normal_(generator=gen)
    vc = torch.empty(rows, cap, d, device=dev, dtype=torch.bfloat16).normal_(generator=gen)
    committed = torch.zeros(rows, cap, device=dev)
    # demand after a 128K prefix: running a T=128K prefill for 1024 rows is minutes of work, so
    # the accumulator is filled with the mean-field value of column sums, sum_{i>=j} 1/i ~ ln(L0/j)
    j = torch.arange(1, L0 + 1, device=dev, dtype=torch.float32)
    committed[:, :L0] = (math.log(L0) - torch.log(j) + 1.0 / j)[None, :]
    scratch = K.decode_scratch(rows, cap, d, dev)
    newq = torch.empty(steps + warm, rows, 1, d, device=dev, dtype=torch.bfloat16).normal_(generator=gen)
    kc4, vc4, c3 = kc.view(1, rows, cap, d), vc.view(1, rows, cap, d), committed.view(1, rows, cap)

    def step(i, length):
        return K.dilution_decode_step(newq[i].view(1, rows, 1, d), kc4, vc4, c3, length, scratch=scratch)

    for i in range(warm):
        step(i, L0 + i + 1)
    barrier()
    L.profile(True)
    L.profile_collect()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        step(warm + i, L0 + warm + i + 1)
    stop.record()
    barrier()
    ms = start.elapsed_time(stop) / steps
    prof = L.profile_collect()
    L.profile(False)
    if distributed:
        tms = torch.tensor([ms], device=dev)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms = tms.item()
    mean_len = L0 + warm + (steps + 1) / 2
    algo_bytes = rows * mean_len * (2 * d * 2 + 4 + 4)
    kernel_ms = sum(tot / cnt for cnt, tot in prof.values())
    achieved = algo_bytes / (kernel_ms * 1e-3) / 1e9
    del kc, vc, committed, scratch
    torch.cuda.empty_cache()
    return {"metric": "decode tok/s @128K KV", "value": cfg["rows"] / cfg["H"] / (ms * 1e-3), "unit": "tok/s",
            "ms_per_step": ms, "rows_per_gpu": rows, "cache_len": L0, "steps": steps,
            "config": "batch 64 x 16 heads, d=64, bf16 KV, fp32 demand; heads sharded across GPUs; "
                      "demand initialised analytically (ln(L/j)), KV N(0,1) generated on device",
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm"],
                         # ncu capture at 64 rows x 128K keys: scores + sweep kernels read and wrote
                         # 2.2319 GB of DRAM for 64 * 131074 keys = 266 B per key; bytes per step
                         "traffic": 266.0 * rows * mean_len,
                         "traffic_source": "ncu capture at 64 rows (profiles/decode_rows64_len131072_ncu_full.md), "
                                           "scaled by keys per step; bytes",
                         "algorithmic_bytes_per_key": 2 * d * 2 + 8,
                         "peak_source": f"{peaks['source']} copy bandwidth"},
            "kernels_ms": {n: tot / cnt for n, (cnt, tot) in prof.items()}}


PREFILL = dict(H=16, T=131072, D=64)


def run_prefill(args, rank, world):
    """Long-context prefill (forward + demand vector), B=1 H=16 T=131072 d=64 bf16, sequence-parallel:
    rank r owns a contiguous, equal-causal-area query chunk, all-gathers K/V, exchanges per-key
    demand once.  Strong scaling: the problem is fixed, value = 2*H*T*(T+1)*D / time."""
    import torch.distributed as dist
    pkg = importlib.import_module("dilution-attention_b200")
    P = pkg.partition
    pkg._lib.load()
    local = int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    H, T, D = (PREFILL[x] for x in "HTD")
    T = args.seq if args.seq != TRAIN["T"] else T
    bounds = P.equal_area_bounds(T, world)
    a, b = bounds[rank], bounds[rank + 1]
    gen = torch.Generator(device=dev).manual_seed(1340 + rank)
    ql, kl, vl = (torch.empty(H, b - a, D, device=dev, dtype=torch.bfloat16).normal_(generator=gen)
                  for _ in range(3))

    def step():
        return P.sequence_parallel_prefill(ql, kl, vl, T, bounds, dot_precision="bf16")

    for _ in range(args.warmup):
        step()
    dist.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        start.record()
        for _ in range(args.steps):
            out, demand = step()
        stop.record()
        dist.barrier()
        torch.cuda.synchronize()
    tms = torch.tensor([start.elapsed_time(stop) / args.steps], device=dev)
    dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    ms = tms.item()
    status = pkg._lib.load().dilution_device_status()
    if rank == 0:
        flops = causal_flops(H, T, D, 2)
        print(json.dumps({"metric": "prefill TFLOP/s @T=128K (B1 H16 d64, forward + demand)",
                          "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
                          "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
                          "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
                          "data": "synthetic", "device_status": status,
                          "config": {"workload": f"prefill_B1_H{H}_T{T}_d{D}", "query_chunk_bounds": bounds,
                                     "parallelism": f"sequence-parallel x{world}: K/V all-gather + "
                                                    "all-gather/masked-sum exscan of per-key demand",
                                     "flop_count": "2*H*T*(T+1)*D"},
                          "clocks": clocks.summary()}), flush=True)
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="train", choices=["train", "prefill"],
                    help="train: the headline fwd+bwd step (default); prefill: 128K sequence-parallel forward")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--no-train", action="store_true", help="skip the training-shape step (decode only)")
    ap.add_argument("--decode-rows", type=int, default=DECODE["batch"] * DECODE["H"],
                    help="(batch*head) rows of the decode workload (profiling captures use fewer)")
    ap.add_argument("--decode-steps", type=int, default=DECODE["steps"])
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--seq", type=int, default=TRAIN["T"],
                    help="sequence length of the training-shape operator (profiling captures use a smaller one)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    TRAIN["T"] = args.seq
    DECODE["rows"] = args.decode_rows
    DECODE["steps"] = args.decode_steps
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    if args.workload == "prefill":
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29541")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
        run_prefill(args, rank, world)
        return
    run_ours(args, rank, world)


if __name__ == "__main__":
    main()
