"""Benchmark of the dilution-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference|triton]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Headline (the JSON line's metric/value): forward + backward of the training-shape
operator, B=4 H=16 T=16384 d=64, bf16 inputs (q,k = 0.5*N(0,1), v = N(0,1),
dout = 1e-2*N(0,1)), fp32 accumulation, as TFLOP/s by the 7-matmul causal count
7 * N * T*(T+1) * D.  One step = one forward + one backward of that batch.
With N GPUs every rank runs its own batch*head slab (weak scaling, no collective).

Also on the line:
  roofline       the dominant kernel against the measured dense-bf16 peak; per-kernel
                 CUDA-event times in `kernels_ms`;
  e2e            the same step through the public op with pinned HOST buffers: H2D of
                 q,k,v,dout and D2H of out,dq,dk,dv inside the timed region, with the
                 achieved host<->device rate beside a plain pinned-copy ceiling taken in
                 the same run;
  train_sharded  the same 64 (batch, head) rows split 64/N per rank (strong scaling);
  prefill        B=1 H=16 T=131072 forward + demand, sequence-parallel over the N ranks
                 (strong scaling), with per-phase CUDA-event times;
  decode         cached decode tok/s at 131072 and 16384 cached keys (batch 64 x 16
                 heads, 256 steps, heads sharded over ranks) against the measured HBM
                 copy bandwidth;
  other_shapes   (1 GPU) forward + backward at the smaller shapes the reference publishes, and at
                 an fp32 ("tf32") and a head_dim-128 shape, which run on the fp32 tile kernels with tf32
                 tensor-core products;
  config1_fp32   (1 GPU) BASELINE config 1 on the tile kernels with fp32 FMA products, with the reference's
                 CPU operator at the same shape;
  lm             (1 GPU, when a copy of the reference package is installed under
                 baseline/_ref) the reference's unmodified DilutionLM on these kernels:
                 train-step tokens/s at B=4 T=16384 and prefill 32K + 512 greedy
                 tokens at batch 16;
  cpu_baseline   the reference's CPU path timed on this box's host cores on a bounded
                 sample.

--impl reference times the reference's CPU implementation on the host cores for the
same metric (and, beside it, its Triton kernels on this GPU when they run).
--impl triton times the reference's own Triton kernels alone.
"""

from __future__ import annotations

import argparse
import importlib
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
REF_DIR = os.path.join(ROOT, "baseline", "_ref")

TRAIN = dict(B=4, H=16, T=16384, D=64)
DECODE = dict(batch=64, H=16, D=64, lengths=(131072, 16384), steps=256)
PREFILL = dict(H=16, T=131072, D=64)
LM = dict(layers=12, d_model=1024, heads=16, ffn=4096, vocab=50304, train_B=4, train_T=16384,
          gen_batch=16, gen_prompt=32768, gen_new=512)
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


def reference_package():
    """The unmodified reference package, if a copy is installed under baseline/_ref."""
    if not os.path.isdir(os.path.join(REF_DIR, "dilution")):
        return None
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    return importlib.import_module("dilution")


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


# ------------------------------------------------------------------------------ CPU arm
def cpu_sample(t, reps):
    """The reference's CPU path, forward + autograd backward, one (b,h) row at length t:
    the unmodified `dilution_attention_reference` when the reference package is installed
    here, else its restatement in oracle/.  Returns (median seconds, kind)."""
    ref = reference_package()
    if ref is not None:
        from dilution.kernels import dilution_attention_reference as op
        kind = "reference"
    else:
        from oracle.dilution_oracle import dilution_dense as op
        kind = "port"
    g = torch.Generator().manual_seed(1339)
    q, k = (torch.randn(1, 1, t, 64, generator=g) * 0.5 for _ in range(2))
    v = torch.randn(1, 1, t, 64, generator=g)
    dout = torch.randn(1, 1, t, 64, generator=g) * 1e-2

    def fwd_bwd(n):
        qs, ks, vs = (x[:, :, :n].clone().requires_grad_(True) for x in (q, k, v))
        op(qs, ks, vs).backward(dout[:, :, :n])

    fwd_bwd(256)   # warm
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        fwd_bwd(t)
        times.append(time.perf_counter() - t0)
    return statistics.median(times), kind


def cpu_baseline_block(t=8192, reps=5):
    sec, kind = cpu_sample(t, reps)
    return {"value": causal_flops(1, t, 64, 7) / sec / 1e12, "unit": "TFLOP/s",
            "cores": torch.get_num_threads(), "kind": kind,
            "sample": f"1 (batch,head) row at T={t}, d=64, fp32 forward + autograd backward, "
                      f"median of {reps}; {os.cpu_count()} logical CPUs"}


def run_reference(args, rank):
    """The reference's CPU path (kernels.py:40-68) on the host cores; beside it, the
    reference's Triton kernels on this GPU, run in a child process so that a failure to
    compile or run them cannot take this line down."""
    if rank != 0:
        return
    # torchrun exports OMP_NUM_THREADS=1 to every rank; the other ranks exit without work, so
    # rank 0 takes all the host's cores, as it does when launched without torchrun
    torch.set_num_threads(os.cpu_count() or 1)
    t = 8192
    kind = "port"
    for _ in range(args.warmup):
        _, kind = cpu_sample(t, 1)
    times = []
    for _ in range(args.steps):
        sec, kind = cpu_sample(t, 1)
        times.append(sec)
    sec = sum(times) / len(times)
    value = causal_flops(1, t, 64, 7) / sec / 1e12
    sample = (f"each step = 1 (batch,head) row at T={t} of the B4 H16 T16384 workload, fp32 forward + "
              f"autograd backward on {torch.get_num_threads()} host threads")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": {"workload": "train_fwd_bwd_B4_H16_T16384_d64", "sample": sample},
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                             "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    if not args.no_triton:
        line["triton"] = triton_child(args)
    print(json.dumps(line), flush=True)


def triton_child(args):
    """`bench.py --impl triton` in a child process on one GPU; its JSON line, or why not."""
    env = {k: v for k, v in os.environ.items()
           if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT", "OMP_NUM_THREADS",
                        "GROUP_RANK", "LOCAL_WORLD_SIZE", "ROLE_RANK", "ROLE_WORLD_SIZE",
                        "TORCHELASTIC_RUN_ID")}
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "triton", "--steps", str(max(args.steps, 3)),
           "--warmup", str(max(args.warmup, 3))]
    try:
        proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    except subprocess.TimeoutExpired:
        return {"impl": "triton", "unavailable": "child process exceeded 900 s"}
    for text in reversed(proc.stdout.strip().splitlines()):
        if text.startswith("{"):
            try:
                return json.loads(text)
            except json.JSONDecodeError:
                break
    tail = (proc.stderr or proc.stdout).strip().splitlines()[-1:] or ["no output"]
    return {"impl": "triton", "unavailable": f"exit {proc.returncode}: {tail[0][:300]}"}


def run_triton(args):
    """The reference's own Triton kernels (src/dilution/kernels.py, unmodified, imported from
    baseline/_ref) on this GPU at the headline shape, timed the way the reference times them
    (scripts/profile_kernels.py:115-124: warm-up, then the median of per-iteration CUDA-event
    times), and its decode kernel at a 16384-key cache."""
    def unavailable(why):
        print(json.dumps({"impl": "triton", "unavailable": why[:400]}), flush=True)

    if not torch.cuda.is_available():
        return unavailable("no CUDA device")
    if reference_package() is None:
        return unavailable("no installed copy of the reference under baseline/_ref")
    try:
        import dilution.kernels as rk
        if not rk.HAS_TRITON:
            return unavailable("triton is not importable")
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        B, H, T, D = (TRAIN[x] for x in "BHTD")
        _, devt = make_train_inputs(dev, 0)
        q, k, v = (devt[x].requires_grad_(True) for x in "qkv")
        dout = devt["dout"]

        def step():
            q.grad = k.grad = v.grad = None
            rk.dilution_attention(q, k, v, dot_precision="bf16").backward(dout)

        for _ in range(max(args.warmup, 3)):
            step()
        torch.cuda.synchronize()
        times = []
        for _ in range(max(args.steps, 3)):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            step()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        ms = statistics.median(times)
        del devt, q, k, v, dout
        torch.cuda.empty_cache()
        # decode at a 16384-key cache, 1024 rows, as the reference's kernel is called by the model
        rows, L0, steps = 1024, 16384, 64
        gen = torch.Generator(device=dev).manual_seed(4)
        cap = L0 + steps + 4
        kc = torch.empty(1, rows, cap, D, device=dev, dtype=torch.bfloat16).normal_(generator=gen)
        vc = torch.empty(1, rows, cap, D, device=dev, dtype=torch.bfloat16).normal_(generator=gen)
        com = torch.zeros(1, rows, cap, device=dev)
        j = torch.arange(1, L0 + 1, device=dev, dtype=torch.float32)
        com[:, :, :L0] = (math.log(L0) - torch.log(j) + 1.0 / j)[None, None, :]
        qs = torch.empty(steps + 3, 1, rows, 1, D, device=dev, dtype=torch.bfloat16).normal_(generator=gen)
        for i in range(3):
            rk.dilution_decode_step(qs[i], kc, vc, com, L0 + i + 1)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(steps):
            rk.dilution_decode_step(qs[3 + i], kc, vc, com, L0 + 3 + i + 1)
        b.record()
        torch.cuda.synchronize()
        dms = a.elapsed_time(b) / steps
        other = time_other_shapes(rk.dilution_attention, dev)
        try:
            other_ffma = time_shapes(rk.dilution_attention, dev, TILE_SHAPES, iters=5)
        except Exception as e:  # noqa: BLE001
            other_ffma = {"error": f"{type(e).__name__}: {str(e)[:200]}"}
        try:
            import dilution.kernels_bid as rkb
            variants = time_variants(rkb.dilution_attention, dev)
        except Exception as e:  # noqa: BLE001
            variants = {"error": f"{type(e).__name__}: {str(e)[:200]}"}
        import triton
        print(json.dumps({
            "impl": "triton", "other_shapes": other, "fp32_and_d128_shapes": other_ffma, "variants": variants, "metric": METRIC, "value": causal_flops(B * H, T, D, 7) / (ms * 1e-3) / 1e12,
            "unit": "TFLOP/s", "ms_per_step": ms, "steps": len(times), "n_gpus": 1, "dtype": "bf16",
            "config": {"workload": f"train_fwd_bwd_B{B}_H{H}_T{T}_d{D}",
                       "path": "dilution.kernels.dilution_attention of the reference, Triton "
                               f"{triton.__version__}, median of per-iteration CUDA-event times"},
            "decode": {"metric": "decode tok/s @16K KV", "value": 64 / (dms * 1e-3), "unit": "tok/s",
                       "ms_per_step": dms, "rows": rows, "cache_len": L0, "steps": steps,
                       "hbm_gbs": rows * (L0 + 3 + (steps + 1) / 2) * 264 / (dms * 1e-3) / 1e9}}), flush=True)
    except Exception as e:  # noqa: BLE001
        unavailable(f"{type(e).__name__}: {e}")


# Smaller shapes the reference publishes times for (docs/kernels.md:206-209 of the reference,
# measured there on another card), bf16, d=64: (batch, heads, seq).
OTHER_SHAPES = ((32, 12, 1024), (8, 8, 4096), (2, 12, 16384))


# Shapes that run on the fp32 tile kernels here, with tf32 tensor-core products (fp32 tensors under
# "tf32", as the model's non-autocast path passes them, and head_dim 128):
# (batch, heads, seq, head_dim, dtype, precision).
TILE_SHAPES = ((8, 8, 4096, 64, torch.float32, "tf32"), (4, 8, 4096, 128, torch.bfloat16, "bf16"))


def time_shapes(op, dev, shapes, iters=10):
    """Median CUDA-event ms of forward + backward of `op` at the given shapes (warm-up 3)."""
    out = {}
    for b, h, t, d, dtype, prec in shapes:
        g = torch.Generator(device=dev).manual_seed(b * t + d)
        q, k, v = (torch.empty(b, h, t, d, device=dev, dtype=torch.float32).normal_(generator=g)
                   .mul_(0.5 if i < 2 else 1.0).to(dtype).requires_grad_(True) for i in range(3))
        dout = torch.empty(b, h, t, d, device=dev).normal_(generator=g).mul_(1e-2)

        def step():
            q.grad = k.grad = v.grad = None
            op(q, k, v, dot_precision=prec).backward(dout)

        for _ in range(3):
            step()
        torch.cuda.synchronize()
        times = []
        for _ in range(iters):
            a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            step()
            e.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(e))
        ms = statistics.median(times)
        name = f"B{b}_H{h}_T{t}" + ("" if (d, dtype) == (64, torch.bfloat16) else f"_d{d}_{str(dtype)[6:]}_{prec}")
        out[name] = {"ms": ms, "tflops": causal_flops(b * h, t, d, 7) / (ms * 1e-3) / 1e12}
        del q, k, v, dout
    torch.cuda.empty_cache()
    return out


# The bid / share ablations at the shape the reference's ablation configurations train at
# (configs/bid_8192: context 8192, 8 heads of 64, bf16): (bid, share_cumsum).
VARIANTS = (("sigmoid", True), ("softmax", "exclusive"), ("softmax", False), ("sigmoid", False), ("softplus", True))
VARIANT_SHAPE = (4, 8, 8192, 64, torch.bfloat16, "bf16")


def time_variants(op_bid, dev, iters=5):
    """Forward + backward of the kernels_bid entry point `op_bid` under each variant."""
    out = {}
    for bid, share in VARIANTS:
        def op(q, k, v, dot_precision):
            return op_bid(q, k, v, dot_precision=dot_precision, bid=bid, share_cumsum=share)
        r = time_shapes(op, dev, [VARIANT_SHAPE], iters)
        key = f"{bid}_{ {True: 'inclusive', False: 'none'}.get(share, share) }"
        out[key] = next(iter(r.values()))
    b, h, t, d = VARIANT_SHAPE[:4]
    out["shape"] = f"B{b}_H{h}_T{t}_d{d}_bf16"
    return out


def time_other_shapes(op, dev, iters=10):
    return time_shapes(op, dev, [(b, h, t, 64, torch.bfloat16, "bf16") for b, h, t in OTHER_SHAPES], iters)


# ------------------------------------------------------------------------------ our arm
def make_train_inputs(dev, rank, rows=None):
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


class Ctx:
    """What every block needs: package handles, device, ranks, barrier, max-over-ranks."""

    def __init__(self):
        self.pkg = importlib.import_module("dilution-attention_b200")
        self.K, self.L, self.P = self.pkg.kernels, self.pkg._lib, self.pkg.partition
        self.L.load()
        self.rank = int(os.environ.get("RANK", 0))
        self.world = int(os.environ.get("WORLD_SIZE", 1))
        self.local = int(os.environ.get("LOCAL_RANK", 0))
        self.dev = torch.device("cuda", self.local)
        torch.cuda.set_device(self.dev)
        self.distributed = self.world > 1
        if self.distributed:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist
        self.peaks = measured_peaks()

    def barrier(self):
        if self.distributed:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, x):
        if not self.distributed:
            return x
        t = torch.tensor([x], device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.item()

    def min_over_ranks(self, x):
        if not self.distributed:
            return x
        t = torch.tensor([x], device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return t.item()

    def timed(self, fn, steps):
        """ms per step of `steps` calls of fn, CUDA events, barrier + synchronize on both
        sides, max over ranks."""
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        start.record()
        for i in range(steps):
            fn(i)
        stop.record()
        self.barrier()
        return self.max_over_ranks(start.elapsed_time(stop) / steps)

    def close(self):
        if self.distributed:
            self.dist.destroy_process_group()


def train_roofline(kernels_ms, n_rows, T, D, value_per_gpu, peaks):
    """Roofline block of the dominant kernel of the training step."""
    # algorithmic matmuls per kernel: the backward main pass carries all five backward products,
    # the forward main pass QK^T and share@V; the other passes are recomputation overhead
    share = {"backward_main": 5, "forward_main": 2, "forward_fused": 2}      # longest launch of the step
    dom = max(kernels_ms, key=kernels_ms.get) if kernels_ms else None
    if dom is None:
        return None
    mm = next((m for key, m in share.items() if key in dom), 0)
    achieved = causal_flops(n_rows, T, D, mm) / (kernels_ms[dom] * 1e-3) / 1e12
    # DRAM bytes per launch: dram__bytes_read.sum + dram__bytes_write.sum of this kernel in one
    # ncu capture at T=4096 (64 rows, 528 causal 128x128 tiles per row: 1341.02 MB), scaled by the
    # number of causal tiles this launch processes -- the dQ tile reductions dominate it and grow
    # with the tile count.  Only the backward main pass has a captured figure.
    executed = 11 if any("forward_fused" in name for name in kernels_ms) else 12
    tiles = n_rows * (T // 128) * (T // 128 + 1) // 2
    traffic = 1341.92e6 / (64 * 528) * tiles if "backward_main" in dom else None
    return {"bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peaks["tensor"],
            "unit": "TFLOP/s", "frac": achieved / peaks["tensor"], "traffic": traffic,
            "traffic_source": "constant from one ncu capture of this kernel at T=4096, scaled by causal "
                              "128x128 tiles per launch; bytes",
            "peak_source": f"{peaks['source']} sustained bf16", "matmuls_in_kernel": mm,
            "step_frac_of_peak": value_per_gpu / peaks["tensor"],
            # matmul-equivalents the tensor cores actually run per step: QK^T in the row, key-
            # stationary forward, reverse and key-correction passes (4; 5 when the forward runs as
            # column-sum pass + main pass), share@V, dO V^T, dV, dQ, dK (5), the pk product of the
            # row pass and the key-correction product W Q (2); the ones columns that give row sums
            # and ghat (N = 80 instead of 64) are not counted
            "executed": {"matmuls_per_step": executed, "value": value_per_gpu * executed / 7, "unit": "TFLOP/s",
                         "frac": value_per_gpu * executed / 7 / peaks["tensor"]}}


def run_ours(args):
    c = Ctx()
    K, L = c.K, c.L
    if args.only:
        blocks = {"decode": run_decode, "prefill": run_prefill, "lm": run_lm,
                  "tile": lambda c_, a_: time_shapes(c_.K.dilution_attention, c_.dev, TILE_SHAPES, iters=3),
                  "variants": lambda c_, a_: time_variants(c_.pkg.kernels_bid.dilution_attention, c_.dev, iters=3)}
        res = blocks[args.only](c, args)
        if c.rank == 0:
            print(json.dumps({args.only: res}), flush=True)
        c.close()
        return
    B, H, T, D = (TRAIN[x] for x in "BHTD")
    n_rows = B * H
    host, devt = make_train_inputs(c.dev, c.rank)
    q, k, v = (devt[x].requires_grad_(True) for x in "qkv")
    dout = devt["dout"]
    torch.cuda.synchronize()

    for _ in range(args.warmup):
        train_step(K, q, k, v, dout)
    c.barrier()

    # --- timed region: K steps, device-resident inputs, CUDA events, per-kernel events on
    launches0 = L.launch_count()
    L.profile(True)
    L.profile_collect()
    with ClockSampler(c.local) as clocks:
        ms_per_step = c.timed(lambda i: train_step(K, q, k, v, dout), args.steps)
    prof = L.profile_collect()
    L.profile(False)
    launches = L.launch_count() - launches0
    total_flops = causal_flops(n_rows, T, D, 7) * c.world
    value = total_flops / (ms_per_step * 1e-3) / 1e12
    kernels_ms = {name: tot / cnt for name, (cnt, tot) in prof.items()}
    roofline = train_roofline(kernels_ms, n_rows, T, D, value / c.world, c.peaks)

    other = fp32_c1 = None
    if c.world == 1 and not args.no_other:
        other = time_other_shapes(K.dilution_attention, c.dev)
        other["tile_kernels"] = time_shapes(K.dilution_attention, c.dev, TILE_SHAPES, iters=5)
        other["variants"] = time_variants(c.pkg.kernels_bid.dilution_attention, c.dev)
        fp32_c1 = run_config1(c)
    sharded = None if args.no_sharded else run_train_sharded(c, args, devt)
    e2e = None if args.no_e2e else run_e2e(c, args, host, total_flops)
    del devt, q, k, v, dout, host
    torch.cuda.empty_cache()
    prefill = None if args.no_prefill else run_prefill(c, args)
    decode = None if args.no_decode else run_decode(c, args)
    lm = None
    if not args.no_lm:
        lm = run_lm(c, args)

    # 0 unless a kernel of this run gave up one of its bounded waits (rank 0's device)
    device_status = c.L.load().dilution_device_status()
    if c.rank == 0:
        line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": c.world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"train_fwd_bwd_B{B}_H{H}_T{T}_d{D}", "rows_per_gpu": n_rows,
                           "global_rows": n_rows * c.world, "seq_len": T, "head_dim": D,
                           "parallelism": f"batch*head slab per GPU x{c.world}, no collective",
                           "l2": "inputs exceed L2 (q,k,v 134 MB each, dout/out 268 MB at T=16384)",
                           "flop_count": "7*N*T*(T+1)*D"},
                "roofline": roofline, "kernels_ms": kernels_ms, "e2e": e2e, "gpu_launches": launches,
                "device_status": device_status, "clocks": clocks.summary(), "other_shapes": other, "config1_fp32": fp32_c1,
                "train_sharded": sharded, "prefill": prefill,
                "decode": decode, "lm": lm}
        if c.world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline_block()
        print(json.dumps(line), flush=True)
    c.close()


def run_config1(c, iters=10):
    """BASELINE config 1 (B1 H4 T512 d64 fp32, forward + autograd backward of
    dilution_attention_reference): this library's fp32 tile kernels (FMA products) on the GPU, and the reference's
    CPU operator at the same shape on the host cores."""
    g = torch.Generator().manual_seed(1338)
    hq, hk, hv, hd = (torch.randn(1, 4, 512, 64, generator=g) for _ in range(4))
    q, k, v = (x.to(c.dev).requires_grad_(True) for x in (hq, hk, hv))
    dout = hd.to(c.dev)

    def step():
        q.grad = k.grad = v.grad = None
        c.K.dilution_attention_reference(q, k, v).backward(dout)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step()
        e.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(e))
    res = {"workload": "B1_H4_T512_d64 fp32 forward + backward", "gpu_ms": statistics.median(times),
           "gpu_path": "fp32 tile kernels, FMA products (dot_precision ieee)"}
    if reference_package() is not None:
        from dilution.kernels import dilution_attention_reference as ref
        cpu = []
        for _ in range(4):
            qs, ks, vs = (x.clone().requires_grad_(True) for x in (hq, hk, hv))
            t0 = time.perf_counter()
            ref(qs, ks, vs).backward(hd)
            cpu.append((time.perf_counter() - t0) * 1e3)
        res["cpu_reference_ms"] = statistics.median(cpu[1:])
        res["cpu_threads"] = torch.get_num_threads()
    return res


def run_train_sharded(c, args, devt):
    """The headline's 64 (batch, head) rows split 64/N per rank: strong scaling, no collective
    (rows are independent).  value = the whole batch's FLOPs / max-over-ranks time."""
    B, H, T, D = (TRAIN[x] for x in "BHTD")
    n_rows = B * H
    a, b = c.P.row_shard(n_rows, c.rank, c.world)
    if b == a:
        return {"skipped": f"{n_rows} rows cannot be split over {c.world} ranks"}
    flat = {x: devt[x].reshape(1, n_rows, T, D)[:, a:b] for x in ("q", "k", "v", "dout")}
    q, k, v = (flat[x].detach().clone().requires_grad_(True) for x in "qkv")
    dout = flat["dout"].contiguous()
    for _ in range(2):
        train_step(c.K, q, k, v, dout)
    ms = c.timed(lambda i: train_step(c.K, q, k, v, dout), args.steps)
    return {"metric": METRIC, "value": causal_flops(n_rows, T, D, 7) / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "ms_per_step": ms, "scaling": "strong", "rows_total": n_rows, "rows_per_gpu": b - a,
            "steps": args.steps,
            "parallelism": f"{n_rows} batch*head rows sharded over {c.world} rank(s), no collective"}


def copy_ceiling(c, nbytes=1 << 29, reps=4):
    """Plain pinned cudaMemcpyAsync rates of this rank with every rank copying at the same
    time: host->device alone, device->host alone, and both at once on two streams (GB/s)."""
    hbuf = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    hbuf2 = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    dbuf = torch.empty(nbytes, dtype=torch.uint8, device=c.dev)
    dbuf2 = torch.empty(nbytes, dtype=torch.uint8, device=c.dev)
    s1, s2 = torch.cuda.Stream(c.dev), torch.cuda.Stream(c.dev)

    def h2d(i):
        dbuf.copy_(hbuf, non_blocking=True)

    def d2h(i):
        hbuf2.copy_(dbuf2, non_blocking=True)

    def both(i):
        with torch.cuda.stream(s1):
            dbuf.copy_(hbuf, non_blocking=True)
        with torch.cuda.stream(s2):
            hbuf2.copy_(dbuf2, non_blocking=True)
        torch.cuda.current_stream().wait_stream(s1)
        torch.cuda.current_stream().wait_stream(s2)

    out = {}
    for name, fn, factor in (("h2d", h2d, 1), ("d2h", d2h, 1), ("both", both, 2)):
        fn(0)
        ms = c.timed(fn, reps)
        out[name + "_gbs"] = factor * nbytes / (ms * 1e-3) / 1e9
    return out


def run_e2e(c, args, host, total_flops):
    """The step through the public host-buffer entry point (`dilution_attention_host`): pinned
    HOST q, k, v (bf16) and dout in; pinned HOST out (fp32), dq, dk, dv (bf16) back.  All copies
    are inside the timed region; the call pipelines row slabs over three streams.  dout is kept
    in bf16 on the host, as a bf16 model's upstream gradient is, and read by the kernels as it
    is; `fp32_dout` repeats the measurement with an fp32 dout."""
    K = c.K
    out = torch.empty(host["dout"].shape, dtype=torch.float32).pin_memory()
    grads = tuple(torch.empty_like(host[n]).pin_memory() for n in "qkv")
    dout16 = host["dout"].bfloat16().pin_memory()

    def measure(dout):
        def e2e_step(i):
            K.dilution_attention_host(host["q"], host["k"], host["v"], dout, dot_precision="bf16",
                                      device=c.dev, slabs=8, out=out, grads=grads)
        e2e_step(0)
        return c.timed(e2e_step, args.steps)

    ms = measure(dout16)
    ms32 = measure(host["dout"])
    h2d = sum(host[n].numel() * host[n].element_size() for n in "qkv") + dout16.numel() * 2
    d2h = out.numel() * out.element_size() + sum(x.numel() * x.element_size() for x in grads)
    ceiling = copy_ceiling(c)
    return {"value": total_flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms, "steps": args.steps,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "h2d_gbs_per_rank": h2d / (ms * 1e-3) / 1e9, "d2h_gbs_per_rank": d2h / (ms * 1e-3) / 1e9,
            "copy_ceiling_per_rank": ceiling,
            "fp32_dout": {"value": total_flops / (ms32 * 1e-3) / 1e12, "ms_per_step": ms32,
                          "h2d_bytes_per_step": h2d + dout16.numel() * 2},
            "path": "dilution_attention_host: 8 row slabs pipelined over copy-in / compute / copy-out "
                    "streams; bf16 q,k,v,dout in, fp32 out and bf16 dq,dk,dv back"}


def run_decode(c, args):
    """Cached decode, batch 64 x 16 heads, d=64, bf16 KV + fp32 demand, 256 steps of one new
    token per sequence at each cache length; heads sharded over ranks (strong scaling)."""
    res = {}
    for L0 in DECODE["lengths"]:
        res[f"len{L0}"] = decode_at(c, args, L0)
    main = res[f"len{DECODE['lengths'][0]}"]
    out = dict(main)
    out["other_lengths"] = {k: v for k, v in res.items() if v is not main}
    return out


def demand_by_prefill(c, q, kc, L0, slab=128):
    """Per-key demand after a prefix of L0 keys: this repository's own forward on the cached K
    with seeded random Q, in row slabs (the carry scratch is quadratic in L0)."""
    rows, _, d = kc.shape
    total = torch.empty(rows, L0, device=c.dev)
    for a in range(0, rows, slab):
        b = min(a + slab, rows)
        qs = q[a:b].view(1, b - a, L0, d)
        ks = kc[a:b, :L0].reshape(1, b - a, L0, d)
        _, aux = c.K.dilution_attention_forward(qs, ks, ks, dot_precision="bf16", return_aux=True)
        total[a:b] = aux["committed_total"][0]
        del aux
    return total


def decode_at(c, args, L0):
    K, L = c.K, c.L
    rows_total = args.decode_rows
    a, b = c.P.row_shard(rows_total, c.rank, c.world)
    rows = b - a
    d, steps = DECODE["D"], args.decode_steps
    warm = 3
    cap = L0 + steps + warm
    gen = torch.Generator(device=c.dev).manual_seed(4 + c.rank)
    kc = torch.empty(rows, cap, d, device=c.dev, dtype=torch.bfloat16).normal_(generator=gen)
    vc = torch.empty(rows, cap, d, device=c.dev, dtype=torch.bfloat16).normal_(generator=gen)
    committed = torch.zeros(rows, cap, device=c.dev)
    if L0 <= 16384:
        # demand by running the prefill on the same K with seeded N(0,1) Q
        qp = torch.empty(rows, L0, d, device=c.dev, dtype=torch.bfloat16).normal_(generator=gen)
        committed[:, :L0] = demand_by_prefill(c, qp, kc, L0)
        del qp
        how = "demand initialised by this repository's prefill on the same K with seeded N(0,1) Q"
    else:
        # a 131072-key prefill of 1024 rows is ~20 s of GPU work; the step's time does not depend on
        # the demand's values (see `demand_init_check`), so the mean-field column sums
        # sum_{i>=j} 1/i ~ ln(L0/j) stand in
        j = torch.arange(1, L0 + 1, device=c.dev, dtype=torch.float32)
        committed[:, :L0] = (math.log(L0) - torch.log(j) + 1.0 / j)[None, :]
        how = "demand initialised analytically (ln(L/j))"
    torch.cuda.empty_cache()
    scratch = K.decode_scratch(rows, cap, d, c.dev)
    newq, newk, newv = (torch.empty(steps + warm, 1, rows, 1, d, device=c.dev, dtype=torch.bfloat16)
                        .normal_(generator=gen) for _ in range(3))
    out = torch.empty(rows, d, device=c.dev, dtype=torch.bfloat16)
    cache = {"k": kc.view(1, rows, cap, d), "v": vc.view(1, rows, cap, d), "len": L0,
             "committed": committed.view(1, rows, cap)}

    def step(i):
        # one new q, k, v token per sequence: appended and attended to in the same three launches
        return K.dilution_decode_append_step(newq[i], newk[i], newv[i], cache, scratch=scratch, out=out)

    for i in range(warm):
        step(i)
    L.profile(True)
    L.profile_collect()
    ms = c.timed(lambda i: step(warm + i), steps)
    prof = L.profile_collect()
    L.profile(False)
    mean_len = L0 + warm + (steps + 1) / 2
    algo_bytes = rows * mean_len * (2 * d * 2 + 4 + 4)
    kernel_ms = sum(tot / cnt for cnt, tot in prof.values())
    achieved = algo_bytes / (kernel_ms * 1e-3) / 1e9
    check = None
    if L0 <= 16384 and c.rank == 0:
        # the same steps with the analytic demand instead: time is value-independent
        j = torch.arange(1, L0 + 1, device=c.dev, dtype=torch.float32)
        committed.zero_()
        committed[:, :L0] = (math.log(L0) - torch.log(j) + 1.0 / j)[None, :]
        cache["len"] = L0
        for i in range(warm):
            step(i)
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a0.record()
        for i in range(steps):
            step(warm + i)
        a1.record()
        torch.cuda.synchronize()
        check = {"ms_per_step_prefill_demand": ms, "ms_per_step_analytic_demand": a0.elapsed_time(a1) / steps}
    del kc, vc, committed, scratch, cache
    torch.cuda.empty_cache()
    return {"metric": f"decode tok/s @{L0 // 1024}K KV", "value": rows_total / DECODE["H"] / (ms * 1e-3),
            "unit": "tok/s", "ms_per_step": ms, "rows_per_gpu": rows, "cache_len": L0, "steps": steps,
            "scaling": "strong",
            "config": f"batch {rows_total // DECODE['H']} x 16 heads, d=64, bf16 KV, fp32 demand; heads sharded "
                      f"across GPUs; each step appends one N(0,1) q,k,v token per sequence; {how}; KV N(0,1) "
                      "generated on device",
            "demand_init_check": check,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": c.peaks["hbm"], "unit": "GB/s",
                         "frac": achieved / c.peaks["hbm"],
                         # one ncu capture at 64 rows x 128K keys: scores + sweep kernels read and wrote
                         # 2.2319 GB of DRAM for 64 * 131074 keys = 266 B per key; bytes per step
                         "traffic": 266.0 * rows * mean_len,
                         "traffic_source": "constant from one ncu capture at 64 rows x 131072 keys (266 B per "
                                           "key), scaled by keys per step; bytes",
                         "algorithmic_bytes_per_key": 2 * d * 2 + 8,
                         "peak_source": f"{c.peaks['source']} copy bandwidth"},
            "kernels_ms": {n: tot / cnt for n, (cnt, tot) in prof.items()}}


def run_prefill(c, args):
    """Long-context prefill (forward + demand vector), B=1 H=16 T=131072 d=64 bf16, sequence-parallel:
    rank r owns a contiguous, equal-causal-area query chunk, receives the K/V of the earlier ranks
    and exchanges per-key demand once.  Strong scaling: value = 2*H*T*(T+1)*D / max-over-ranks time.
    `phases_ms` are CUDA-event times of this call's phases, max over ranks."""
    H, T, D = (PREFILL[x] for x in "HTD")
    T = args.prefill_seq or T
    bounds = c.P.equal_area_bounds(T, c.world)
    a, b = bounds[c.rank], bounds[c.rank + 1]
    gen = torch.Generator(device=c.dev).manual_seed(1340 + c.rank)
    ql, kl, vl = (torch.empty(H, b - a, D, device=c.dev, dtype=torch.bfloat16).normal_(generator=gen)
                  for _ in range(3))
    if c.distributed:
        def step(mark=None):
            return c.P.sequence_parallel_prefill(ql, kl, vl, T, bounds, dot_precision="bf16", mark=mark)
    else:
        def step(mark=None):
            if mark:
                mark("gather_keys")
            out, total = c.P.prefill_chunk(ql, kl, vl, 0, dot_precision="bf16", mark=mark)
            return out, total

    steps = max(1, min(args.steps, 5))
    for _ in range(2):
        step()
    with ClockSampler(c.local) as clocks:
        ms = c.timed(lambda i: step(), steps)
    # one more call with an event after every phase
    names = ["gather_keys", "passes_1_2", "exchange", "pass_3"]
    events = {"start": torch.cuda.Event(enable_timing=True)}
    c.barrier()
    events["start"].record()

    def mark(name):
        events[name] = torch.cuda.Event(enable_timing=True)
        events[name].record()

    c.L.profile(True)
    c.L.profile_collect()
    out, demand = step(mark)
    c.barrier()
    kernels_ms = {name: tot / cnt for name, (cnt, tot) in c.L.profile_collect().items()}
    c.L.profile(False)
    phases, prev = {}, "start"
    for name in names:
        phases[name] = c.max_over_ranks(events[prev].elapsed_time(events[name]))
        prev = name
    demand_sum = float(demand.double().sum().item()) / H if demand.shape[-1] == T else None
    status = c.L.load().dilution_device_status()
    flops = causal_flops(H, T, D, 2)
    return {"metric": "prefill TFLOP/s @T=128K (B1 H16 d64, forward + demand)",
            "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms, "steps": steps,
            "scaling": "strong", "device_status": status, "phases_ms": phases, "kernels_ms": kernels_ms,
            "demand_sum_over_T": None if demand_sum is None else demand_sum / T,
            "config": {"workload": f"prefill_B1_H{H}_T{T}_d{D}", "query_chunk_bounds": bounds,
                       "parallelism": f"sequence-parallel x{c.world}: triangular point-to-point K/V exchange + "
                                      "all-gather/masked-sum exscan of per-key demand (NCCL)",
                       "flop_count": "2*H*T*(T+1)*D"},
            "clocks": clocks.summary()}


def run_lm(c, args):
    """The reference's unmodified DilutionLM (model.py:342-512) on these kernels: 12 layers,
    d_model 1024, 16 heads of 64, SwiGLU at 4x width, vocabulary 50304, tied embeddings, layers
    alternating softmax attention with RoPE and dilution attention without position encoding
    (layer_attention = [softmax, dilution] * 6 with positional = rope_alt, which rotates layers
    0, 2, 4, ...), weight-only LayerNorm (the reference has no RMSNorm), random initial weights,
    uniform random token ids, bf16 autocast.  The headline figures run with everything this
    library offers installed (dilution kernels, fused decode append, fused head split + RoPE,
    softmax layers' inference on the row pass and the streaming decode kernels);
    `dilution_kernels_only` repeats them with only `dilution.kernels` replaced, i.e. with the
    softmax layers and the head split as the reference's model runs them (SDPA, torch RoPE)."""
    try:
        if reference_package() is None:
            return {"unavailable": "no installed copy of the reference package under baseline/_ref"}
        from dilution.config import ModelConfig
        from dilution.model import DilutionLM
        dev = c.dev
        launches0 = c.L.launch_count()

        def config(ctx):
            return ModelConfig(vocab_size=LM["vocab"], n_layers=LM["layers"], d_model=LM["d_model"],
                               n_heads=LM["heads"], context_length=ctx, layer_attention=["softmax", "dilution"] * 6,
                               positional="rope_alt", mlp="swiglu", ffn_hidden=LM["ffn"])

        res = {"config": {"model": "DilutionLM 12L d1024 16H ffn4096 vocab50304, softmax+RoPE / dilution "
                                   "alternating, weight-only LayerNorm, tied embeddings, random init",
                          "dtype": "bf16 autocast, fp32 master weights"}}
        B, T = LM["train_B"], args.lm_seq or LM["train_T"]
        nb, prompt, new = LM["gen_batch"], args.lm_prompt or LM["gen_prompt"], LM["gen_new"]
        g = torch.Generator().manual_seed(1344)
        idx_h = torch.randint(0, LM["vocab"], (B, T + 1), generator=g).pin_memory()
        idx_gen_full = torch.randint(0, LM["vocab"], (nb, prompt), generator=g).to(dev)

        def shard(model):
            """more than one rank: every rank builds the same weights (same seed), keeps 16 / N heads
            and 1 / N of each MLP, and feeds the same tokens (partition.shard_lm_heads)"""
            return c.pkg.partition.shard_lm_heads(model) if c.world > 1 else model

        def train(steps):
            """forward, loss, backward, gradient clipping, fused AdamW; token ids come from the host
            and the loss is read back every step"""
            torch.manual_seed(1344)
            model = shard(DilutionLM(config(T)).to(dev)).train()
            model.enable_dilution_kernel()
            opt = torch.optim.AdamW(model.parameters(), lr=3e-4, fused=True)

            def step(i):
                tok = idx_h.to(dev, non_blocking=True)
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    _, loss = model(tok[:, :-1], tok[:, 1:])
                loss.backward()
                if c.world > 1:
                    c.pkg.partition.clip_grad_norm_(model, 1.0)
                else:
                    torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
                opt.step()
                opt.zero_grad(set_to_none=True)
                return loss.item()

            for i in range(2):
                step(i)
            torch.cuda.reset_peak_memory_stats(dev)
            ms = c.timed(step, steps)
            out = {"tokens_per_s": B * T / (ms * 1e-3), "ms_per_step": ms, "steps": steps, "batch": B,
                   "seq_len": T, "params": sum(p.numel() for p in model.parameters()),
                   "peak_mem_gb": torch.cuda.max_memory_allocated(dev) / 1e9}
            del model, opt
            torch.cuda.empty_cache()
            return out

        def generate(new_tokens, graphed=False, prompt=prompt):
            """DilutionLM.prefill + greedy decode_step loop (model.py:451-470, 498-509)"""
            idx_gen = idx_gen_full[:, :prompt]
            torch.manual_seed(1345)
            model = shard(DilutionLM(config(prompt + new)).to(dev)).eval()
            model.enable_dilution_kernel()
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
                logits, caches = model.prefill(idx_gen[:, :256], capacity=300)      # warm-up of both paths
                model.decode_step(logits[:, -1].argmax(-1, keepdim=True), 256, caches)
                del caches
                torch.cuda.synchronize()
                ev[0].record()
                logits, caches = model.prefill(idx_gen, capacity=prompt + new)
                ev[1].record()
                tok = logits[:, -1, :].float().argmax(dim=-1, keepdim=True)
                for s in range(new_tokens - 1):
                    logits = model.decode_step(tok, prompt + s, caches)
                    tok = logits[:, -1, :].float().argmax(dim=-1, keepdim=True)
                ev[2].record()
                torch.cuda.synchronize()
            pre_ms, dec_ms = ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2])
            out = {"decode_tok_s": nb * (new_tokens - 1) / (dec_ms * 1e-3),
                   "decode_ms_per_token": dec_ms / (new_tokens - 1), "prefill_ms": pre_ms,
                   "prefill_tok_s": nb * prompt / (pre_ms * 1e-3), "batch": nb, "prompt": prompt,
                   "new_tokens": new_tokens}
            if graphed:
                # the same greedy loop with the per-token layer loop replayed from one CUDA graph
                # (layers.GraphedDecode): first step eager, second recorded, the rest timed
                del caches
                with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
                    logits, caches = model.prefill(idx_gen, capacity=prompt + new)
                dec = c.pkg.GraphedDecode(model, caches)
                tok = logits[:, -1, :].float().argmax(dim=-1, keepdim=True)
                for s in range(2):
                    tok = dec.step(tok)[:, -1, :].float().argmax(dim=-1, keepdim=True)
                torch.cuda.synchronize()
                ev[0].record()
                for s in range(new_tokens - 3):
                    tok = dec.step(tok)[:, -1, :].float().argmax(dim=-1, keepdim=True)
                ev[1].record()
                torch.cuda.synchronize()
                g_ms = ev[0].elapsed_time(ev[1])
                out["graphed"] = {"decode_tok_s": nb * (new_tokens - 3) / (g_ms * 1e-3),
                                  "decode_ms_per_token": g_ms / (new_tokens - 3), "timed_tokens": new_tokens - 3,
                                  "path": "layers.GraphedDecode: DilutionLM.decode_step recorded once, replayed per token"}
                dec.close()
            del model, caches
            torch.cuda.empty_cache()
            return out

        steps = max(1, min(args.steps, 3))
        c.pkg.install(fused_decode=True)
        c.pkg.install_layers()
        if c.world > 1:
            # the same global batch with the model's heads over the ranks: strong scaling; two
            # all-reduces per block and direction (after c_proj and after the MLP) are the only
            # exchanges (in the graphed decode loop they are recorded with the rest of the step)
            res["parallelism"] = (f"heads sharded over {c.world} ranks (partition.shard_lm_heads): "
                                  f"{LM['heads'] // c.world} heads and 1/{c.world} of each MLP per rank, NCCL "
                                  "all-reduce after c_proj and after the MLP; embedding, LayerNorms, lm_head replicated")
            res["scaling"] = "strong"
            res["train"] = train(steps)
            res["generate"] = generate(new, graphed=True)
            res["gpu_launches"] = c.L.launch_count() - launches0
            return res
        res["train"] = train(steps)
        res["generate"] = generate(new, graphed=True)
        # a short context, where a token's ~200 launches cost more than the bytes they move
        res["generate_short_context"] = generate(min(new, 256), graphed=True, prompt=min(prompt, 1024))
        c.pkg.uninstall_layers()
        c.pkg.uninstall()
        c.pkg.install()
        res["dilution_kernels_only"] = {"train": train(steps), "generate": generate(min(new, 33))}
        res["gpu_launches"] = c.L.launch_count() - launches0
        return res
    except Exception as e:  # noqa: BLE001
        torch.cuda.empty_cache()
        return {"error": f"{type(e).__name__}: {str(e)[:300]}"}
    finally:
        try:
            c.pkg.uninstall_layers()
            c.pkg.uninstall()
        except Exception:  # noqa: BLE001
            pass


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "triton"])
    ap.add_argument("--only", default=None, choices=["decode", "prefill", "lm", "tile", "variants"],
                    help="run one block alone and print it")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-sharded", action="store_true")
    ap.add_argument("--no-lm", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-other", action="store_true", help="skip the smaller shapes and config 1")
    ap.add_argument("--no-triton", action="store_true", help="--impl reference: skip the Triton child run")
    ap.add_argument("--decode-rows", type=int, default=DECODE["batch"] * DECODE["H"],
                    help="(batch*head) rows of the decode workload (profiling captures use fewer)")
    ap.add_argument("--decode-steps", type=int, default=DECODE["steps"])
    ap.add_argument("--decode-lengths", type=str, default=None, help="comma-separated cache lengths")
    ap.add_argument("--seq", type=int, default=TRAIN["T"],
                    help="sequence length of the training-shape operator (profiling captures use a smaller one)")
    ap.add_argument("--prefill-seq", type=int, default=None)
    ap.add_argument("--lm-seq", type=int, default=None)
    ap.add_argument("--lm-prompt", type=int, default=None)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    TRAIN["T"] = args.seq
    if args.decode_lengths:
        DECODE["lengths"] = tuple(int(x) for x in args.decode_lengths.split(","))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.impl == "triton":
        if rank == 0:
            run_triton(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    run_ours(args)


if __name__ == "__main__":
    main()
