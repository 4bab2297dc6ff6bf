"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (N=1): dense training-shaped forward+backward, B=16 H=16 S=4096 D=128 fp16,
causal, softmax_scale 1/sqrt(128), synthetic N(0,1) inputs.  One step = one forward plus one
backward over that batch.  FLOPs are the algorithmic ones: forward 2*B*H*D*S*(S+1), backward
2.5x forward (five GEMMs; the recompute of the split dQ / dK,dV design is not counted).

Printed keys (one JSON line on rank 0):
  value      fwd+bwd TFLOP/s, inputs resident in HBM, CUDA-event timed, max over ranks
  e2e        the same through the public Python API with pinned HOST inputs copied to the
             device inside the timed region and the loss/gradient checksums read back
  roofline   the kernel with the largest share of the step: algorithmic TFLOP/s of that
             kernel (timed on its own with CUDA events) against the measured cuBLAS bf16 peak
  cpu_baseline  the CPU oracle (fp32 torch restatement of the reference) on this box's
             host cores on a bounded slice of the same workload
  kernels    per-kernel ms and TFLOP/s;  decode  paged-KV decode GB/s (batch 64, Hq32/Hkv8,
             D128, page 256, lengths U[1024,32768]) against the measured HBM copy bandwidth

With N > 1 (torchrun) every rank runs the same per-GPU workload on its own shard of
(batch x head) units -- the units are independent, there is no data-path collective -- so
this is weak scaling: value = N * per-rank FLOPs / max-over-ranks time.

--impl reference times the reference's CPU path (its algorithm restated in oracle/, since the
reference is Triton-on-GPU only and its interpreter cannot travel) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

B, H, S, D = 16, 16, 4096, 128
FWD_FLOPS = 2.0 * B * H * D * S * (S + 1)
BWD_FLOPS = 2.5 * FWD_FLOPS
METRIC = "fwd+bwd TFLOP/s (hd128 causal fp16) & paged-decode HBM GB/s vs B200 peak"
WORKLOAD = "dense fwd+bwd B16 H16 S4096 D128 fp16 causal (BASELINE configs[1])"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(bf16=p["bf16_tflops"], bf16_sustained=p.get("bf16_tflops_sustained"),
                    hbm=p["hbm_gbs"], source="measured")
    return dict(bf16=1590.0, bf16_sustained=1400.0, hbm=6650.0, source="fallback")


class NvmlSampler:
    """SM clock and throttle reasons read through NVML every few ms while the timed region
    runs (read-only queries)."""

    def __init__(self, gpu_index):
        import pynvml
        self.nv = pynvml
        pynvml.nvmlInit()
        self.h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        self.sm, self.reasons, self.stop_flag = [], 0, False

    def start(self):
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _run(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                self.sm.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                self.reasons |= nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
            except Exception:
                break
            time.sleep(0.005)

    def stop(self):
        nv = self.nv
        self.stop_flag = True
        self.thread.join(timeout=1)
        names = []
        for bit, name in ((getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8), "hw_slowdown"),
                          (getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40), "hw_thermal_slowdown"),
                          (getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20), "sw_thermal_slowdown"),
                          (getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4), "sw_power_cap")):
            if self.reasons & bit:
                names.append(name)
        sm = sorted(self.sm)
        try:
            mx = nv.nvmlDeviceGetMaxClockInfo(self.h, nv.NVML_CLOCK_SM)
        except Exception:
            mx = None
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": names,
                "samples": len(sm), "source": "nvml"}


def make_sampler(gpu_index):
    try:
        return NvmlSampler(gpu_index)
    except Exception:
        return ClockSampler(gpu_index)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx = float(r[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                               r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def event_time(fn, iters):
    """Average ms of fn() over `iters` calls, CUDA events on the current stream."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


# ----------------------------------------------------------------------------------------
# CPU arm: the oracle restatement of the reference on the host cores
# ----------------------------------------------------------------------------------------
def cpu_sample(seconds_budget=20.0):
    """fwd+bwd of (batch, head) slices of the headline workload through the fp32 oracle until
    the budget is used.  Returns (TFLOP/s, threads, description)."""
    from oracle import attention_oracle as orc
    torch.set_num_threads(max(torch.get_num_threads(), os.cpu_count() or 1))  # torchrun pins OMP to 1
    g = torch.Generator().manual_seed(0)
    bh = 1
    q = torch.randn(1, S, bh, D, generator=g).half()
    k = torch.randn(1, S, bh, D, generator=g).half()
    v = torch.randn(1, S, bh, D, generator=g).half()
    do = torch.randn(1, S, bh, D, generator=g).half()
    t0 = time.perf_counter()
    n = 0
    while True:
        orc.attention_grads_ref(q, k, v, do, causal=True)
        n += 1
        if time.perf_counter() - t0 > seconds_budget or n >= 64:
            break
    dt = time.perf_counter() - t0
    flops = n * bh * 3.5 * 2.0 * D * S * (S + 1)
    return flops / dt / 1e12, torch.get_num_threads(), (
        f"{n} of {B * H} (batch,head) slices of the workload (S={S}, D={D}, causal), fwd+bwd "
        f"through the fp32 oracle, {dt:.1f} s")


def run_reference(args, rank, world):
    if rank != 0:
        return
    steps = max(args.steps, 1)
    per_step = max(2.0, min(20.0, 60.0 / (steps + args.warmup)))
    vals = []
    for i in range(args.warmup + steps):
        v, cores, sample = cpu_sample(per_step)
        if i >= args.warmup:
            vals.append(v)
    value = sum(vals) / len(vals)
    ms = (FWD_FLOPS + BWD_FLOPS) / (value * 1e12) * 1e3
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "note": "CPU arm: one step = a bounded slice of the workload, "
                       "ms_per_step extrapolated to the full batch"},
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------
def decode_bench(dev, peaks, iters=20):
    """Paged-KV decode, BASELINE configs[3]; returns dict with GB/s."""
    import numpy as np

    import flash_attn_triton_b200 as fa
    Bd, Hq, Hkv, Dd, page, pool, maxp = 64, 32, 8, 128, 256, 4096, 129
    for seed in range(100):
        rng = np.random.default_rng(seed)
        lens = rng.integers(1024, 32769, size=Bd)
        if int(np.sum((lens + 1 + page - 1) // page)) <= pool:
            break
    g = torch.Generator(device=dev).manual_seed(seed)
    kc = torch.randn(pool, page, Hkv, Dd, device=dev, dtype=torch.float16, generator=g)
    vc = torch.randn(pool, page, Hkv, Dd, device=dev, dtype=torch.float16, generator=g)
    q = torch.randn(Bd, 1, Hq, Dd, device=dev, dtype=torch.float16, generator=g)
    kn = torch.randn(Bd, 1, Hkv, Dd, device=dev, dtype=torch.float16, generator=g)
    vn = torch.randn(Bd, 1, Hkv, Dd, device=dev, dtype=torch.float16, generator=g)
    perm = rng.permutation(pool)
    bt = np.zeros((Bd, maxp), dtype=np.int32)
    at = 0
    for b, L in enumerate(lens):
        need = (L + 1 + page - 1) // page
        bt[b, :need] = perm[at:at + need]
        bt[b, need:] = perm[at]
        at += need
    bt = torch.from_numpy(bt).to(dev)
    cl = torch.tensor(lens, dtype=torch.int32, device=dev)
    inv = 1.0 / (10000.0 ** (torch.arange(0, Dd, 2, dtype=torch.float32) / Dd))
    ang = torch.arange(32769 + 8, dtype=torch.float32)[:, None] * inv[None, :]
    cos, sin = torch.cos(ang).half().to(dev), torch.sin(ang).half().to(dev)
    fa.set_validation(False)  # the value checks need a device->host sync per call

    def step():
        fa.flash_attn_with_kvcache(q, kc, vc, kn, vn, cos, sin, cache_seqlens=cl, block_table=bt,
                                   rotary_interleaved=False)
    for _ in range(3):
        step()
    ms = event_time(step, iters)
    fa.set_validation(True)
    bytes_step = float(np.sum(lens + 1)) * Hkv * Dd * 2 * 2
    gbs = bytes_step / ms / 1e6
    return {"metric": "paged-decode HBM GB/s", "value": gbs, "unit": "GB/s", "ms_per_step": ms,
            "bytes_per_step": bytes_step, "seed": seed, "frac_of_measured_hbm": gbs / peaks["hbm"],
            "frac_of_8TBs": gbs / 8000.0,
            "config": "batch 64, Hq32/Hkv8, D128, page 256, pool 4096, lens U[1024,32768], append+rotary"}


def profile_case(args):
    """Forward + backward on B=2 H=16 S=4096 D=128 causal (inputs 128 MiB > L2), W+K steps."""
    from flash_attn_triton_b200 import _native as N
    from flash_attn_triton_b200 import _ops
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    q, k, v, do = (torch.randn(2, S, H, D, device=dev, dtype=torch.float16, generator=g) for _ in range(4))
    scale = 1.0 / math.sqrt(D)
    for _ in range(args.warmup + args.steps):
        o, lse, _ = _ops.dense_forward(q, k, v, scale, True, -1, -1, 0.0, None, 0, N.IMPL_AUTO, "bshd", True)
        _ops.dense_backward(q, k, v, o, lse, do, scale, True, -1, -1, 0.0, None, 0, N.IMPL_AUTO, "bshd")
    torch.cuda.synchronize()
    print(json.dumps({"profile_case": "B2 H16 S4096 D128 causal fwd+bwd", "steps": args.warmup + args.steps,
                      "device_wait_status": N.lib().fa_device_wait_status(0)}))


def extras_bench(dev, peaks):
    """The other BASELINE configs, one number each (rank 0, after the headline measurement)."""
    import numpy as np

    import flash_attn_triton_b200 as fa
    from flash_attn_triton_b200 import _ops
    out = {}
    # config 5: INT8 forward B8 H32 S8192 D128, 1 % of K entries x8
    Bq, Hq, Sq, Dq = 8, 32, 8192, 128
    g = torch.Generator(device=dev).manual_seed(5)
    q = torch.randn(Bq, Hq, Sq, Dq, device=dev, dtype=torch.float16, generator=g)
    v = torch.randn(Bq, Hq, Sq, Dq, device=dev, dtype=torch.float16, generator=g)
    k = torch.randn(Bq, Hq, Sq, Dq, device=dev, dtype=torch.float16, generator=g)
    k = torch.where(torch.rand(Bq, Hq, Sq, Dq, device=dev, generator=g) < 0.01, k * 8, k)
    for _ in range(2):
        _ops.quantize_k_int8(k)
    ms = event_time(lambda: _ops.quantize_k_int8(k), 5)
    out["int8_k_quantiser"] = {"ms": ms, "GB/s": k.numel() * 3 / ms / 1e6, "frac_of_measured_hbm": k.numel() * 3 / ms / 1e6 / peaks["hbm"]}
    for causal in (False, True):
        for _ in range(2):
            fa.attention_int8(q, k, v, causal=causal)
        ms = event_time(lambda: fa.attention_int8(q, k, v, causal=causal), 3)
        fl = (2.0 if causal else 4.0) * Bq * Hq * Sq * Sq * Dq
        out["int8_fwd_causal" if causal else "int8_fwd"] = {"ms": ms, "tflops": fl / ms / 1e9, "note": "incl. K and Q quantiser prepasses"}
    del q, k, v
    # config 3: packed varlen fwd+bwd, 32 sequences, H32 D128, causal + window 1024 + ALiBi + softcap 30
    rng = np.random.default_rng(3)
    lens = (64 * rng.integers(4, 65, size=32)).tolist()
    Hh, Dd, T = 32, 128, int(sum(lens))
    g = torch.Generator(device=dev).manual_seed(3)
    q, k, v, do = (torch.randn(T, Hh, Dd, device=dev, dtype=torch.float16, generator=g) for _ in range(4))
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=dev)
    sl = torch.tensor([2.0 ** (-8 * (i + 1) / Hh) for i in range(Hh)], device=dev)
    fa.set_validation(False)

    def vstep():
        qq, kk, vv = (t.detach().requires_grad_() for t in (q, k, v))
        o = fa.flash_attn_varlen_func(qq, kk, vv, cu, cu, max(lens), max(lens), causal=True,
                                      window_size=(1024, 0), alibi_slopes=sl, softcap=30.0)
        torch.autograd.grad(o, (qq, kk, vv), do)
    for _ in range(2):
        vstep()
    ms = event_time(vstep, 3)
    fa.set_validation(True)
    pairs = sum(L * (L + 1) // 2 if L <= 1025 else 1025 * 1026 // 2 + (L - 1025) * 1025 for L in lens)
    fl = 3.5 * 4.0 * Dd * Hh * pairs
    out["varlen_fwd_bwd"] = {"ms": ms, "tflops": fl / ms / 1e9, "tokens": T}
    return out


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist

    import flash_attn_triton_b200 as fa
    from flash_attn_triton_b200 import _native as N
    from flash_attn_triton_b200 import _ops
    from flash_attn_triton_b200 import sharding

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    peaks = measured_peaks()
    scale = 1.0 / math.sqrt(D)

    # this rank's shard: with N ranks the job is N x (B*H) units, each rank owns B*H of them
    lo, hi = sharding.shard_range(B * H * world, rank, world)
    assert hi - lo == B * H
    g = torch.Generator(device=dev).manual_seed(sharding.unit_seed(0, lo))
    mk = lambda: torch.randn(B, S, H, D, device=dev, dtype=torch.float16, generator=g)
    q, k, v, do = mk(), mk(), mk(), mk()

    def fwd_only():
        return _ops.dense_forward(q, k, v, scale, True, -1, -1, 0.0, None, 0, N.IMPL_AUTO, "bshd", True)

    o, lse, _ = fwd_only()

    def step():
        o2, lse2, _ = fwd_only()
        _ops.dense_backward(q, k, v, o2, lse2, do, scale, True, -1, -1, 0.0, None, 0, N.IMPL_AUTO, "bshd")

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()

    sampler = make_sampler(local_rank)
    if world > 1:
        dist.barrier()
    sampler.start()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop()
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    value = world * (FWD_FLOPS + BWD_FLOPS) / ms / 1e9

    # ---- per-kernel timing (rank-local, after the headline measurement) --------------------
    import ctypes as C
    kernels = {}
    kernels["fwd"] = event_time(fwd_only, max(args.steps, 5))
    a = N.AttnArgs()
    dq, dk, dv, delta = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v), torch.empty_like(lse)
    _ops._fill_common(a, q, k, v, o, _ops._BSHD, _ops._BSHD, batch=B, sq=S, sk=S, hq=H, hkv=H, d=D, scale=scale,
                      causal=True, wl=-1, wr=-1, softcap=0.0, alibi=None, q_pos_offset=0, impl=N.IMPL_AUTO)
    a.lse2, a.lse_stride = lse.data_ptr(), N._I64x3(H * S, 1, S)
    a.dout, a.do_stride, a.delta = do.data_ptr(), N.strides3(do, _ops._BSHD), delta.data_ptr()
    a.dq, a.dk, a.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.dq_stride = a.dk_stride = a.dv_stride = N.strides3(dq, _ops._BSHD)
    L, st = N.lib(), N.stream_ptr(dev)
    for name, fn in (("bwd_preprocess", L.fa_bwd_preprocess), ("bwd_dq", L.fa_bwd_dq), ("bwd_dkdv", L.fa_bwd_dkdv)):
        kernels[name] = event_time(lambda fn=fn: N.check(fn(C.byref(a), st), name), max(args.steps, 5))
    # algorithmic FLOPs per launch: fwd = 2 GEMMs, dq = 1 of the 5 backward GEMMs, dkdv = 4
    # (S and dP are recomputed in both backward kernels; recompute is not counted)
    algo = {"fwd": FWD_FLOPS, "bwd_dq": FWD_FLOPS * 0.5, "bwd_dkdv": FWD_FLOPS * 2.0, "bwd_preprocess": 0.0}
    executed = {"fwd": FWD_FLOPS, "bwd_dq": FWD_FLOPS * 1.5, "bwd_dkdv": FWD_FLOPS * 2.0, "bwd_preprocess": 0.0}
    top = max(("fwd", "bwd_dq", "bwd_dkdv"), key=lambda n: kernels[n])
    # DRAM traffic per launch of each kernel from the ncu captures summarised in profiles/
    # (B=2 capture scaled x8 by batch, profiles/fwd_bwd_sm100_B2_H16_S4096_D128_causal.md)
    traffic = {"fwd": 0.94e9, "bwd_dq": 1.24e9, "bwd_dkdv": 1.41e9}
    roofline = {"kernel": top, "bound": "tensor", "achieved": algo[top] / kernels[top] / 1e9,
                "peak": peaks["bf16"], "unit": "TFLOP/s", "frac": algo[top] / kernels[top] / 1e9 / peaks["bf16"],
                "peak_source": peaks["source"] + " cuBLAS bf16 burst", "traffic": traffic[top],
                "executed_tflops": executed[top] / kernels[top] / 1e9,
                "frac_of_2250_datasheet": algo[top] / kernels[top] / 1e9 / 2250.0}
    kern = {n: {"ms": kernels[n], "tflops": (algo[n] / kernels[n] / 1e9 if algo[n] else None),
                "frac_of_measured_peak": (algo[n] / kernels[n] / 1e9 / peaks["bf16"] if algo[n] else None),
                "frac_of_2250": (algo[n] / kernels[n] / 1e9 / 2250.0 if algo[n] else None)} for n in kernels}
    kern["fwd"]["tcgen05"] = bool(L.fa_fwd_uses_tcgen05(C.byref(a)))

    # ---- end to end through the public API with host buffers -------------------------------
    # Every step copies q, k, v, dO (1 GiB) from pinned host memory, runs forward + backward
    # through flash_attn_func / autograd and reads four checksums back.  The batch goes through
    # in NCH chunks so that the copy of chunk c+1 (copy stream) overlaps the kernels of chunk c:
    # (batch x head) units are independent, so chunking changes no result.
    NCH = 4
    hq, hk_, hv, hdo = (t.cpu().pin_memory() for t in (q, k, v, do))
    dq_, dk_, dv_, ddo = (torch.empty_like(q) for _ in range(4))
    host_out = torch.empty(4, dtype=torch.float32).pin_memory()
    copy_stream = torch.cuda.Stream(device=dev)
    cb = B // NCH

    def e2e_step():
        cur = torch.cuda.current_stream(dev)
        copy_stream.wait_stream(cur)          # the previous step's kernels are done with the buffers
        res = torch.zeros(4, device=dev, dtype=torch.float32)
        for c in range(NCH):
            sl = slice(c * cb, (c + 1) * cb)
            with torch.cuda.stream(copy_stream):
                for dst, src in ((dq_, hq), (dk_, hk_), (dv_, hv), (ddo, hdo)):
                    dst[sl].copy_(src[sl], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(copy_stream)
            cur.wait_event(ev)
            qq, kk, vv = (t[sl].detach().requires_grad_() for t in (dq_, dk_, dv_))
            out = fa.flash_attn_func(qq, kk, vv, causal=True)
            gq, gk, gv = torch.autograd.grad(out, (qq, kk, vv), ddo[sl])
            res += torch.stack([(out[0, 0, 0].float() * ddo[sl][0, 0, 0].float()).sum(), gq[0, 0, 0].float().sum(),
                                gk[0, 0, 0].float().sum(), gv[0, 0, 0].float().sum()])
        host_out.copy_(res, non_blocking=True)
    e2e_step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e2e_ms = event_time(e2e_step, max(2, min(args.steps, 5)))
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = t.item()
    e2e = {"value": world * (FWD_FLOPS + BWD_FLOPS) / e2e_ms / 1e9, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": 4 * q.numel() * 2, "d2h_bytes_per_step": 16,
           "note": f"host->device copies in {NCH} chunks on a copy stream, overlapped with the kernels"}
    del hq, hk_, hv, hdo, dq_, dk_, dv_, ddo

    gather_ms = None
    if world > 1:
        # optional: bring every rank's output to every rank (not part of the metric)
        bufs = [torch.empty_like(o) for _ in range(world)]
        torch.cuda.synchronize()
        dist.barrier()
        t0 = time.perf_counter()
        dist.all_gather(bufs, o)
        torch.cuda.synchronize()
        gather_ms = (time.perf_counter() - t0) * 1e3
        del bufs

    wait_status = L.fa_device_wait_status(local_rank)
    if rank != 0:
        return
    decode = decode_bench(dev, peaks)
    del q, k, v, do, o, lse, dq, dk, dv, delta
    torch.cuda.empty_cache()
    extras = extras_bench(dev, peaks)
    cpu_v, cores, sample = cpu_sample(15.0)
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "per_gpu_units": B * H, "global_units": B * H * world,
                   "sharding": "(batch x head) units, no data-path collective",
                   "l2": "inputs (1 GiB per step) are larger than the 126 MB L2",
                   "flops_per_step": FWD_FLOPS + BWD_FLOPS},
        "clocks": clocks, "e2e": e2e, "gpu_launches": 4 * args.steps,
        "roofline": roofline,
        "cpu_baseline": {"value": cpu_v, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "kernels": kern, "decode": decode, "other_configs": extras, "device_wait_status": wait_status,
        "frac_of_2250_datasheet": value / world / 2250.0, "gather_ms": gather_ms,
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--profile-case", action="store_true",
                    help="run only forward+backward steps on a reduced batch (B=2) and exit: the small "
                         "case used for ncu captures")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.profile_case:
        profile_case(args)
        return
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
