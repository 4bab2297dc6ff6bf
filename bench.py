"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (N=1): dense training-shaped forward+backward, B=16 H=16 S=4096 D=128 fp16,
causal, softmax_scale 1/sqrt(128), synthetic N(0,1) inputs.  One step = one forward plus one
backward over that batch.  FLOPs are the algorithmic ones: forward 2*B*H*D*S*(S+1), backward
2.5x forward (five GEMMs; the recompute of the split dQ / dK,dV design is not counted).

Printed keys (one JSON line on rank 0):
  value      fwd+bwd TFLOP/s, inputs resident in HBM, CUDA-event timed, max over ranks
  e2e        the same through the public Python API with pinned HOST buffers: q, k, v, dO are
             copied to the device and out, dq, dk, dv are copied back inside the timed region
  roofline   the kernel with the largest share of the step: algorithmic TFLOP/s of that
             kernel (timed on its own with CUDA events) against the measured cuBLAS bf16 peak
  cpu_baseline  the CPU oracle (fp32 torch restatement of the reference) on this box's host
             cores on a bounded slice of the same workload; torch's CPU SDPA beside it
  kernels    per-kernel ms and TFLOP/s
  decode     paged-KV decode GB/s (batch 64, Hq32/Hkv8, D128, page 256, lengths U[1024,32768])
             against the measured HBM copy bandwidth, with and without the host value checks
  other_configs  INT8 forward, K quantiser and the packed variable-length batch, each with its
             own roofline fraction
  strong     (N > 1) the same 256 (batch, head) units SPLIT over the ranks: ms per step and
             efficiency against the single-GPU step

With N > 1 (torchrun) every rank runs the same per-GPU workload on its own shard of
(batch x head) units -- the units are independent, there is no data-path collective -- so
`value` is weak scaling: N * per-rank FLOPs / max-over-ranks time.

--impl reference times the reference's CPU path (its algorithm restated in oracle/, since the
reference is Triton-on-GPU only and its interpreter needs the reference checkout) on the host cores.
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
WORKLOAD = "dense training step: forward+backward, B16 H16 S4096 D128 fp16 causal"


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


def bind_to_gpu_numa_node(gpu_index):
    """Restrict this process to the CPUs NVML lists as local to its GPU, so that the pinned host
    buffers of the end-to-end leg (first touched by this process) and the copy threads sit on the
    memory node the GPU hangs off.  Harmless on a single-node host.  Returns a short description."""
    try:
        import pynvml
        pynvml.nvmlInit()
        try:
            uuid = str(torch.cuda.get_device_properties(gpu_index).uuid)
            h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
        except Exception:
            h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        ncpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (ncpu + 63) // 64)
        local = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
        allowed = os.sched_getaffinity(0)
        target = (local & allowed) or allowed
        os.sched_setaffinity(0, target)
        return {"cpus_local_to_gpu": len(local), "cpus_allowed": len(allowed), "cpus_bound": len(target)}
    except Exception as e:      # no NVML, no affinity support: keep the default placement
        return {"unavailable": type(e).__name__}


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


def event_time_alone(fn, iters):
    """Median ms of single fn() calls, each bracketed by its own events with a device
    synchronisation in between (a launch timed alone: no neighbour fills its tail, and the clocks
    are those of a burst, which is what the burst peak in MEASURED_PEAKS.json is measured with)."""
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


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
def _cpu_threads():
    torch.set_num_threads(max(torch.get_num_threads(), os.cpu_count() or 1))  # torchrun pins OMP to 1
    return torch.get_num_threads()


def _cpu_slice(bh=1):
    g = torch.Generator().manual_seed(0)
    return [torch.randn(1, S, bh, D, generator=g).half() for _ in range(4)]


def cpu_sample(seconds_budget=20.0):
    """fwd+bwd of (batch, head) slices of the headline workload through the fp32 oracle until
    the budget is used.  Returns (TFLOP/s, threads, description)."""
    from oracle import attention_oracle as orc
    threads = _cpu_threads()
    q, k, v, do = _cpu_slice()
    t0 = time.perf_counter()
    n = 0
    while True:
        orc.attention_grads_ref(q, k, v, do, causal=True)
        n += 1
        if time.perf_counter() - t0 > seconds_budget or n >= 64:
            break
    dt = time.perf_counter() - t0
    flops = n * 3.5 * 2.0 * D * S * (S + 1)
    return flops / dt / 1e12, threads, (
        f"{n} of {B * H} (batch,head) slices of the workload (S={S}, D={D}, causal), fwd+bwd "
        f"through the fp32 oracle, {dt:.1f} s")


def cpu_sdpa_sample(seconds_budget=8.0):
    """The same slices through torch's own CPU scaled_dot_product_attention (fp32, autograd
    backward): the fastest CPU attention on the box, reported beside the oracle."""
    threads = _cpu_threads()
    q, k, v, do = (t.float().transpose(1, 2).contiguous() for t in _cpu_slice(bh=4))   # (1, 4, S, D)
    t0 = time.perf_counter()
    n = 0
    while True:
        qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
        o = torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, is_causal=True)
        torch.autograd.grad(o, (qq, kk, vv), do)
        n += 4
        if time.perf_counter() - t0 > seconds_budget or n >= 64:
            break
    dt = time.perf_counter() - t0
    return {"value": n * 3.5 * 2.0 * D * S * (S + 1) / dt / 1e12, "unit": "TFLOP/s", "cores": threads,
            "kind": "torch_sdpa", "sample": f"{n} (batch,head) slices, fp32 torch CPU SDPA fwd+bwd, {dt:.1f} s"}


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
            "cpu_sdpa": cpu_sdpa_sample(),
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------
def decode_case(dev, batch_lo=0, batch_hi=64):
    """Paged-KV decode workload: batch 64, Hq32/Hkv8, D128, page 256, pool 4096, lengths
    U[1024, 32768], append + rotary.  Returns the tensors of sequences [batch_lo, batch_hi)."""
    import numpy as np
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
    sl = slice(batch_lo, batch_hi)
    bt = torch.from_numpy(bt[sl]).to(dev)
    cl = torch.tensor(lens[sl], dtype=torch.int32, device=dev)
    inv = 1.0 / (10000.0 ** (torch.arange(0, Dd, 2, dtype=torch.float32) / Dd))
    ang = torch.arange(32769 + 8, dtype=torch.float32)[:, None] * inv[None, :]
    cos, sin = torch.cos(ang).half().to(dev), torch.sin(ang).half().to(dev)
    bytes_step = float(np.sum(lens[sl] + 1)) * Hkv * Dd * 2 * 2
    return (q[sl], kc, vc, kn[sl], vn[sl], cos, sin, cl, bt), bytes_step, seed


def decode_bench(dev, peaks, iters=20, batch_lo=0, batch_hi=64):
    """Paged-KV decode; GB/s = K and V bytes of every cached token once / time.  Timed with the
    host value checks off (no synchronisation inside the call) and with the default checks."""
    import flash_attn_triton_b200 as fa
    (q, kc, vc, kn, vn, cos, sin, cl, bt), bytes_step, seed = decode_case(dev, batch_lo, batch_hi)

    def step():
        fa.flash_attn_with_kvcache(q, kc, vc, kn, vn, cos, sin, cache_seqlens=cl, block_table=bt,
                                   rotary_interleaved=False)
    res = {}
    for checks in (False, True):
        fa.set_validation(checks)
        for _ in range(3):
            step()
        res[checks] = event_time(step, iters)
    fa.set_validation(True)
    ms = res[False]
    gbs = bytes_step / ms / 1e6
    return {"metric": "paged-decode HBM GB/s", "value": gbs, "unit": "GB/s", "ms_per_step": ms,
            "ms_per_step_with_value_checks": res[True], "GB/s_with_value_checks": bytes_step / res[True] / 1e6,
            "bytes_per_step": bytes_step, "seed": seed,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm"], "peak_source": peaks["source"] + " copy bandwidth",
                         "frac_of_8TBs": gbs / 8000.0,
                         # ncu on 16 sequences of this workload: 875.7 MB of DRAM traffic for 870.0 MB of K/V
                         "traffic": bytes_step * 875.7 / 870.0,
                         "traffic_source": "ncu capture of 16 of the sequences, scaled by the K/V bytes"},
            "frac_of_measured_hbm": gbs / peaks["hbm"], "frac_of_8TBs": gbs / 8000.0,
            "config": f"sequences [{batch_lo},{batch_hi}) of batch 64, Hq32/Hkv8, D128, page 256, pool 4096, "
                      "lens U[1024,32768], append+rotary"}


def profile_case(args):
    """Small cases for ncu captures (a few hundred MB on the device, more than the 126 MB L2), W+K
    steps of one kernel family each:
      dense     forward + backward, B2 H16 S4096 D128 causal (per-CTA dK/dV kernel)
      dense_nc  the same without the mask (persistent dK/dV kernel)
      varlen    8 packed sequences, H8 D128, causal + window 1024 + ALiBi + soft cap (feature variants)
      decode    16 sequences of the paged-decode workload
      int8      INT8-QK^T forward B1 H8 S8192 D128 and both quantisers"""
    import flash_attn_triton_b200 as fa
    from flash_attn_triton_b200 import _native as N
    from flash_attn_triton_b200 import _ops
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    which = args.profile_case
    scale = 1.0 / math.sqrt(D)
    n = args.warmup + args.steps
    if which in ("dense", "dense_nc"):
        causal = which == "dense"
        q, k, v, do = (torch.randn(2, S, H, D, device=dev, dtype=torch.float16, generator=g) for _ in range(4))
        for _ in range(n):
            o, lse, _ = _ops.dense_forward(q, k, v, scale, causal, -1, -1, 0.0, None, 0, N.IMPL_AUTO, "bshd", True)
            _ops.dense_backward(q, k, v, o, lse, do, scale, causal, -1, -1, 0.0, None, 0, N.IMPL_AUTO, "bshd")
        what = "B2 H16 S4096 D128 fwd+bwd, causal=%d" % causal
    elif which == "varlen":
        import numpy as np
        lens = (64 * np.random.default_rng(3).integers(4, 65, size=8)).tolist()
        Hh, T = 8, int(sum(lens))
        q, k, v, do = (torch.randn(T, Hh, D, device=dev, dtype=torch.float16, generator=g) for _ in range(4))
        cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=dev)
        alibi = torch.tensor([[2.0 ** (-8 * (i + 1) / Hh) for i in range(Hh)]] * 8, device=dev).contiguous()
        cfg = (max(lens), max(lens), scale, True, 1024, 0, 30.0, alibi)
        for _ in range(n):
            o, lse, _ = _ops.varlen_forward(q, k, v, cu, cu, *cfg, N.IMPL_AUTO, True)
            _ops.varlen_backward(q, k, v, o, lse, do, cu, cu, *cfg, N.IMPL_AUTO)
        what = "packed %d tokens in 8 sequences, H8 D128, causal window 1024 ALiBi softcap 30, fwd+bwd" % T
    elif which == "decode":
        (q, kc, vc, kn, vn, cos, sin, cl, bt), bytes_step, _ = decode_case(dev, 0, 16)
        fa.set_validation(False)
        for _ in range(n):
            fa.flash_attn_with_kvcache(q, kc, vc, kn, vn, cos, sin, cache_seqlens=cl, block_table=bt,
                                       rotary_interleaved=False)
        what = "paged decode, sequences [0,16) of the workload, %.0f MB of K/V per step" % (bytes_step / 1e6)
    elif which == "int8":
        q, k, v = (torch.randn(1, 8, 8192, D, device=dev, dtype=torch.float16, generator=g) for _ in range(3))
        for _ in range(n):
            fa.attention_int8(q, k, v, causal=False)
        what = "INT8 forward B1 H8 S8192 D128 non-causal incl. K and Q quantisers"
    else:
        raise SystemExit("unknown profile case " + str(which))
    torch.cuda.synchronize()
    print(json.dumps({"profile_case": which, "what": what, "steps": n,
                      "device_wait_status": N.lib().fa_device_wait_status(0)}))


def varlen_lens():
    import numpy as np
    return (64 * np.random.default_rng(3).integers(4, 65, size=32)).tolist()


def varlen_flops(lens, heads=32, dim=128):
    """Forward FLOPs of the packed batch: 4 * D * H * visible (query, key) pairs (causal, window 1024)."""
    pairs = sum(L * (L + 1) // 2 if L <= 1025 else 1025 * 1026 // 2 + (L - 1025) * 1025 for L in lens)
    return 4.0 * dim * heads * pairs


def varlen_case(dev, owned=None):
    """Packed batch: 32 sequences of 64*U[4,64] tokens, H32 D128, causal + window 1024 + ALiBi +
    soft cap 30.  `owned` selects a subset of the sequences (multi-GPU sharding)."""
    import numpy as np
    lens_all = varlen_lens()
    idx = list(range(32)) if owned is None else list(owned)
    lens = [lens_all[i] for i in idx]
    Hh, Dd, T = 32, 128, int(sum(lens))
    g = torch.Generator(device=dev).manual_seed(3)
    q, k, v, do = (torch.randn(T, Hh, Dd, device=dev, dtype=torch.float16, generator=g) for _ in range(4))
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=dev)
    sl = torch.tensor([2.0 ** (-8 * (i + 1) / Hh) for i in range(Hh)], device=dev)
    return (q, k, v, do, cu, sl, lens), varlen_flops(lens, Hh, Dd), lens_all


def varlen_bench(dev, peaks, owned=None):
    import flash_attn_triton_b200 as fa
    from flash_attn_triton_b200 import _native as N, _ops
    (q, k, v, do, cu, sl, lens), fwd_flops, _ = varlen_case(dev, owned)
    if not lens:
        return {"ms": 0.0, "tflops": 0.0, "tokens": 0}
    fa.set_validation(False)

    def vstep():
        qq, kk, vv = (t.detach().requires_grad_() for t in (q, k, v))
        o = fa.flash_attn_varlen_func(qq, kk, vv, cu, cu, max(lens), max(lens), causal=True,
                                      window_size=(1024, 0), alibi_slopes=sl, softcap=30.0)
        torch.autograd.grad(o, (qq, kk, vv), do)
    for _ in range(2):
        vstep()
    ms = event_time(vstep, 5)
    fa.set_validation(True)
    # per kernel
    alibi = sl.unsqueeze(0).expand(len(lens), -1).contiguous()
    scale = 1.0 / math.sqrt(128)
    cfg = (max(lens), max(lens), scale, True, 1024, 0, 30.0, alibi)
    o, lse, _ = _ops.varlen_forward(q, k, v, cu, cu, *cfg, N.IMPL_AUTO, True)
    kern = {"fwd": event_time(lambda: _ops.varlen_forward(q, k, v, cu, cu, *cfg, N.IMPL_AUTO, True), 5),
            "bwd": event_time(lambda: _ops.varlen_backward(q, k, v, o, lse, do, cu, cu, *cfg, N.IMPL_AUTO), 5)}
    tf = 3.5 * fwd_flops / ms / 1e9
    return {"ms": ms, "tflops": tf, "tokens": int(q.shape[0]), "fwd_ms": kern["fwd"], "bwd_ms": kern["bwd"],
            "fwd_tflops": fwd_flops / kern["fwd"] / 1e9, "bwd_tflops": 2.5 * fwd_flops / kern["bwd"] / 1e9,
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16"], "unit": "TFLOP/s",
                         "frac": tf / peaks["bf16"], "peak_source": peaks["source"] + " cuBLAS bf16 burst",
                         "traffic": None}}


def int8_bench(dev, peaks):
    """INT8-QK^T forward B8 H32 S8192 D128 with 1 % of the K entries x8, and the K quantiser."""
    import flash_attn_triton_b200 as fa
    from flash_attn_triton_b200 import _ops
    out = {}
    Bq, Hq, Sq, Dq = 8, 32, 8192, 128
    g = torch.Generator(device=dev).manual_seed(5)
    q = torch.randn(Bq, Hq, Sq, Dq, device=dev, dtype=torch.float16, generator=g)
    v = torch.randn(Bq, Hq, Sq, Dq, device=dev, dtype=torch.float16, generator=g)
    k = torch.randn(Bq, Hq, Sq, Dq, device=dev, dtype=torch.float16, generator=g)
    k = torch.where(torch.rand(Bq, Hq, Sq, Dq, device=dev, generator=g) < 0.01, k * 8, k)
    for _ in range(2):
        _ops.quantize_k_int8(k)
    ms = event_time(lambda: _ops.quantize_k_int8(k), 5)
    gbs = k.numel() * 3 / ms / 1e6
    out["int8_k_quantiser"] = {"ms": ms, "GB/s": gbs, "frac_of_measured_hbm": gbs / peaks["hbm"],
                               "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s",
                                            "frac": gbs / peaks["hbm"], "traffic": None,
                                            "peak_source": peaks["source"] + " copy bandwidth"}}
    i8_peak = peaks.get("int8")      # measured by the probe below when the library has it
    for causal in (False, True):
        for _ in range(2):
            fa.attention_int8(q, k, v, causal=causal)
        ms = event_time(lambda: fa.attention_int8(q, k, v, causal=causal), 3)
        fl = (2.0 if causal else 4.0) * Bq * Hq * Sq * Sq * Dq
        tf = fl / ms / 1e9
        # half of the FLOPs are int8 (Q K^T), half fp16 (P V): time at peak = F/2/int8_peak + F/2/fp16_peak
        mixed_peak = 1.0 / (0.5 / i8_peak + 0.5 / peaks["bf16"]) if i8_peak else None
        out["int8_fwd_causal" if causal else "int8_fwd"] = {
            "ms": ms, "tflops": tf, "note": "incl. K and Q quantiser prepasses",
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16"], "unit": "TFLOP/s",
                         "frac": tf / peaks["bf16"], "peak_source": peaks["source"] + " cuBLAS bf16 burst",
                         "int8_peak_tops": i8_peak, "mixed_peak": mixed_peak,
                         "frac_of_mixed": tf / mixed_peak if mixed_peak else None, "traffic": None}}
    return out


def fp16_on_int8_shape(dev, peaks):
    """The fp16 forward on the INT8 workload's shape (B8 H32 S8192 D128, [B,H,S,D]): what the INT8
    path has to beat.  Timed after the other workloads: these long launches lower the clocks that
    whatever is timed next sees."""
    from flash_attn_triton_b200 import _native as N, _ops
    out = {}
    Bq, Hq, Sq, Dq = 8, 32, 8192, 128
    g = torch.Generator(device=dev).manual_seed(5)
    q, k, v = (torch.randn(Bq, Hq, Sq, Dq, device=dev, dtype=torch.float16, generator=g) for _ in range(3))
    for causal in (False, True):
        fl = (2.0 if causal else 4.0) * Bq * Hq * Sq * Sq * Dq
        args = (1.0 / math.sqrt(Dq), causal, -1, -1, 0.0, None, 0, N.IMPL_AUTO, "bhsd", False)
        for _ in range(2):
            _ops.dense_forward(q, k, v, *args)
        ms16 = event_time(lambda: _ops.dense_forward(q, k, v, *args), 3)
        out["fp16_fwd_same_shape_causal" if causal else "fp16_fwd_same_shape"] = {
            "ms": ms16, "tflops": fl / ms16 / 1e9, "frac_of_measured_peak": fl / ms16 / 1e9 / peaks["bf16"]}
    return out


def mma_peak_probe(dev):
    """Tensor-pipe rate of back-to-back tcgen05.mma from one CTA per SM, f16 and int8 operands
    (the library's own issue loop): the denominators for the INT8 forward."""
    import ctypes as C

    from flash_attn_triton_b200 import _native as N
    L = N.lib()
    if not hasattr(L, "fa_mma_peak_probe"):
        return {}
    L.fa_mma_peak_probe.restype = C.c_int
    L.fa_mma_peak_probe.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_void_p]
    out = {}
    iters = 20000
    for kind, name, k_per in ((0, "f16", 16), (1, "int8", 32)):
        st = N.stream_ptr(dev)
        L.fa_mma_peak_probe(dev.index or 0, kind, 2000, st)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        r = L.fa_mma_peak_probe(dev.index or 0, kind, iters, st)
        e1.record()
        torch.cuda.synchronize()
        if r != 0:
            continue
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        out[name] = 2.0 * 128 * 128 * k_per * iters * sms / (e0.elapsed_time(e1) * 1e-3) / 1e12
    return out


def run_ours(args, rank, world, local_rank):
    import ctypes as C

    import torch.distributed as dist

    import flash_attn_triton_b200 as fa
    from flash_attn_triton_b200 import _native as N
    from flash_attn_triton_b200 import _ops
    from flash_attn_triton_b200 import sharding

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    numa = bind_to_gpu_numa_node(local_rank)
    peaks = measured_peaks()
    scale = 1.0 / math.sqrt(D)

    # this rank's shard: with N ranks the job is N x (B*H) units, each rank owns B*H of them
    lo, hi = sharding.shard_range(B * H * world, rank, world)
    assert hi - lo == B * H
    g = torch.Generator(device=dev).manual_seed(sharding.unit_seed(0, lo))
    mk = lambda: torch.randn(B, S, H, D, device=dev, dtype=torch.float16, generator=g)
    q, k, v, do = mk(), mk(), mk(), mk()

    def fwd_only(qq=q, kk=k, vv=v):
        return _ops.dense_forward(qq, kk, vv, scale, True, -1, -1, 0.0, None, 0, N.IMPL_AUTO, "bshd", True)

    o, lse, _ = fwd_only()

    def step(qq=q, kk=k, vv=v, dd=do):
        o2, lse2, _ = fwd_only(qq, kk, vv)
        _ops.dense_backward(qq, kk, vv, o2, lse2, dd, scale, True, -1, -1, 0.0, None, 0, N.IMPL_AUTO, "bshd")

    def timed(fn, steps, finish=None):
        """ms per step of fn over `steps` steps: barrier + synchronize on both sides, CUDA events,
        max over ranks.  `finish` (optional) runs once after the last step, inside the timed region."""
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        if finish is not None:
            finish()
        e1.record()
        torch.cuda.synchronize()
        ms_ = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms_], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_ = t.item()
        return ms_

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = make_sampler(local_rank)
    sampler.start()
    ms = timed(step, args.steps)
    clocks = sampler.stop()
    value = world * (FWD_FLOPS + BWD_FLOPS) / ms / 1e9

    # ---- the same units split over the ranks (strong scaling) -------------------------------
    strong = None
    if world > 1:
        ulo, uhi = sharding.shard_range(B, rank, world)        # whole batch entries: 16 heads each
        if uhi > ulo:
            qs, ks, vs, ds = (t[ulo:uhi] for t in (q, k, v, do))
            sstep = lambda: step(qs, ks, vs, ds)
        else:
            sstep = lambda: None
        for _ in range(3):
            sstep()
        sms = timed(sstep, args.steps)
        strong = {"units_total": B * H, "units_per_gpu": (uhi - ulo) * H, "ms_per_step": sms,
                  "tflops": (FWD_FLOPS + BWD_FLOPS) / sms / 1e9, "efficiency_vs_1gpu_step": (ms / world) / sms,
                  "note": "the 256 (batch, head) units of the workload split by batch entry over the ranks; "
                          "efficiency = (single-GPU step / N) / this step"}

    # ---- per-kernel timing (rank-local, after the headline measurement) --------------------
    reps = max(args.steps, 10)
    kernels = {"fwd": event_time(fwd_only, reps)}
    alone = {"fwd": event_time_alone(fwd_only, 10)}
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
        kernels[name] = event_time(lambda fn=fn: N.check(fn(C.byref(a), st), name), reps)
        alone[name] = event_time_alone(lambda fn=fn: N.check(fn(C.byref(a), st), name), 10)
    # algorithmic FLOPs per launch: fwd = 2 GEMMs, dq = 1 of the 5 backward GEMMs, dkdv = 4
    # (S and dP are recomputed in both backward kernels; recompute is not counted)
    algo = {"fwd": FWD_FLOPS, "bwd_dq": FWD_FLOPS * 0.5, "bwd_dkdv": FWD_FLOPS * 2.0, "bwd_preprocess": 0.0}
    executed = {"fwd": FWD_FLOPS, "bwd_dq": FWD_FLOPS * 1.5, "bwd_dkdv": FWD_FLOPS * 2.0, "bwd_preprocess": 0.0}
    top = max(("fwd", "bwd_dq", "bwd_dkdv"), key=lambda n: kernels[n])
    # DRAM bytes per launch (dram__bytes_read + write) from the ncu captures summarised in profiles/:
    # taken on the B=2 profile case and scaled by 8 (the batch ratio); the working set of one launch
    # exceeds L2 at both sizes, so the traffic grows with the batch
    traffic = {"fwd": 0.93e9, "bwd_dq": 1.24e9, "bwd_dkdv": 1.41e9}
    roofline = {"kernel": top, "bound": "tensor", "achieved": algo[top] / kernels[top] / 1e9,
                "peak": peaks["bf16"], "unit": "TFLOP/s", "frac": algo[top] / kernels[top] / 1e9 / peaks["bf16"],
                "peak_source": peaks["source"] + " cuBLAS bf16 burst", "traffic": traffic[top],
                "traffic_source": "ncu capture of the B=2 profile case, x8",
                "executed_tflops": executed[top] / kernels[top] / 1e9,
                "frac_of_2250_datasheet": algo[top] / kernels[top] / 1e9 / 2250.0,
                # `achieved` is the average over `reps` back-to-back launches (tens of ms of sustained load)
                # against the BURST peak; the two like-for-like pairs are given beside it
                "timing": "average of %d back-to-back launches" % reps,
                "frac_of_sustained_peak": (algo[top] / kernels[top] / 1e9 / peaks["bf16_sustained"]
                                           if peaks.get("bf16_sustained") else None),
                "alone": {"ms": alone[top], "achieved": algo[top] / alone[top] / 1e9,
                          "frac_of_burst_peak": algo[top] / alone[top] / 1e9 / peaks["bf16"],
                          "timing": "median of 10 single launches, device synchronised in between"}}
    kern = {n: {"ms": kernels[n], "tflops": (algo[n] / kernels[n] / 1e9 if algo[n] else None),
                "frac_of_measured_peak": (algo[n] / kernels[n] / 1e9 / peaks["bf16"] if algo[n] else None),
                "frac_of_2250": (algo[n] / kernels[n] / 1e9 / 2250.0 if algo[n] else None),
                "ms_alone": alone[n],
                "frac_of_measured_peak_alone": (algo[n] / alone[n] / 1e9 / peaks["bf16"] if algo[n] else None)}
            for n in kernels}
    kern["fwd"]["tcgen05"] = bool(L.fa_fwd_uses_tcgen05(C.byref(a)))
    kern["bwd_preprocess"]["GB/s"] = (2 * q.numel() * 2 + lse.numel() * 4) / kernels["bwd_preprocess"] / 1e6
    del dq, dk, dv, delta

    # ---- end to end through the public API with host buffers -------------------------------
    # Every step copies q, k, v, dO (1 GiB) from pinned host memory, runs forward + backward through
    # flash_attn_func / autograd and copies out, dq, dk, dv (1 GiB) back to pinned host memory.  The
    # batch goes through in NCH chunks: the copy-in of chunk c+1 (copy stream) and the copy-out of
    # chunk c-1 (second copy stream) overlap the kernels of chunk c; (batch x head) units are
    # independent, so chunking changes no result.
    NCH = max(1, min(B, int(os.environ.get("FA_BENCH_E2E_CHUNKS", "16"))))
    while B % NCH:
        NCH -= 1
    hq, hk_, hv, hdo = (t.cpu().pin_memory() for t in (q, k, v, do))
    ho, hdq, hdk, hdv = (torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (q, q, k, v))
    dq_, dk_, dv_, ddo = (torch.empty_like(q) for _ in range(4))
    in_stream, out_stream = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    cb = B // NCH

    consumed = [None] * NCH      # per chunk: the previous step's kernels have read its device input buffers

    def e2e_step():
        # Steps are pipelined like a training loop that prefetches its next batch: the copy-in of
        # chunk c of this step only waits for the kernels that read chunk c in the previous step
        # (copy-outs are ordered by their stream).
        cur = torch.cuda.current_stream(dev)
        for c in range(NCH):
            sl = slice(c * cb, (c + 1) * cb)
            with torch.cuda.stream(in_stream):
                if consumed[c] is not None:
                    in_stream.wait_event(consumed[c])
                for dst, src in ((dq_, hq), (dk_, hk_), (dv_, hv), (ddo, hdo)):
                    dst[sl].copy_(src[sl], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(in_stream)
            cur.wait_event(ev)
            qq, kk, vv = (t[sl].detach().requires_grad_() for t in (dq_, dk_, dv_))
            out = fa.flash_attn_func(qq, kk, vv, causal=True)
            gq, gk, gv = torch.autograd.grad(out, (qq, kk, vv), ddo[sl])
            done = torch.cuda.Event()
            done.record(cur)
            consumed[c] = done
            out_stream.wait_event(done)
            with torch.cuda.stream(out_stream):
                for dst, src in ((ho, out), (hdq, gq), (hdk, gk), (hdv, gv)):
                    dst[sl].copy_(src.detach(), non_blocking=True)
                    src.record_stream(out_stream)

    def e2e_drain():
        torch.cuda.current_stream(dev).wait_stream(out_stream)    # the last results are on the host
    e2e_step()
    e2e_drain()
    torch.cuda.synchronize()
    e2e_ms = timed(e2e_step, max(2, min(args.steps, 5)), finish=e2e_drain)
    h2d = 4 * q.numel() * 2
    d2h = (2 * q.numel() + 2 * k.numel()) * 2
    e2e = {"value": world * (FWD_FLOPS + BWD_FLOPS) / e2e_ms / 1e9, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "h2d_GBs_per_rank": h2d / e2e_ms / 1e6, "d2h_GBs_per_rank": d2h / e2e_ms / 1e6,
           "host_binding": numa,
           "note": f"q,k,v,dO in and out,dq,dk,dv back through pinned host memory, {NCH} chunks, copies on two "
                   "streams overlapped with the kernels; consecutive steps overlap (the next step's first "
                   "chunks are copied in while the last results are copied out), all results on the host "
                   "before the clock stops"}
    # spot check of the round trip (first batch entry of the output against the resident run)
    e2e["roundtrip_ok"] = bool(torch.equal(ho[0], o[0].cpu()))
    del hq, hk_, hv, hdo, dq_, dk_, dv_, ddo, ho, hdq, hdk, hdv

    # ---- the other workloads, split over the ranks like the headline one --------------------
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
    del q, k, v, do, o, lse
    torch.cuda.empty_cache()

    sharded = None
    if world > 1:
        # packed batch by sequence (longest first on visible pairs), decode by batch entry
        lens_all = varlen_lens()
        owned = sharding.balance_sequences(lens_all, world, window_left=1024)[rank]
        vres = varlen_bench(dev, peaks, owned)
        blo, bhi = sharding.shard_range(64, rank, world)
        dres = decode_bench(dev, peaks, iters=10, batch_lo=blo, batch_hi=bhi)
        t = torch.tensor([vres["ms"], dres["ms_per_step"]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        tot = torch.tensor([dres["bytes_per_step"]], device=dev, dtype=torch.float64)
        dist.all_reduce(tot)
        flops_all = varlen_flops(lens_all)
        sharded = {"varlen_fwd_bwd": {"ms_max_over_ranks": t[0].item(), "tflops_aggregate": 3.5 * flops_all / t[0].item() / 1e9,
                                      "sharding": "sequences, longest first on visible (query, key) pairs"},
                   "decode": {"ms_max_over_ranks": t[1].item(), "GB/s_aggregate": tot.item() / t[1].item() / 1e6,
                              "sharding": "batch entries (each rank holds the pages of its sequences)"}}
    if rank != 0:
        return
    peaks.update({k_: v_ for k_, v_ in (("f16_probe", None), ("int8", None))})
    probe = mma_peak_probe(dev)
    if probe:
        peaks["f16_probe"], peaks["int8"] = probe.get("f16"), probe.get("int8")
    decode = decode_bench(dev, peaks)
    extras = int8_bench(dev, peaks)
    extras["varlen_fwd_bwd"] = varlen_bench(dev, peaks)
    extras.update(fp16_on_int8_shape(dev, peaks))
    if probe:
        extras["tensor_pipe_probe_tflops"] = probe
        if probe.get("f16"):
            # the same kernels against the bare MMA loop measured on this box in this run: a fraction
            # that does not move with the box's clocks the way the fixed denominator does
            roofline["probe_peak"] = probe["f16"]
            roofline["frac_of_probe"] = roofline["achieved"] / probe["f16"]
            for n in kern:
                if kern[n].get("tflops"):
                    kern[n]["frac_of_probe"] = kern[n]["tflops"] / probe["f16"]
    return dict(value=value, ms=ms, clocks=clocks, e2e=e2e, roofline=roofline, kern=kern, decode=decode,
                extras=extras, wait_status=wait_status, gather_ms=gather_ms, strong=strong, sharded=sharded)


def print_line(args, world, r):
    cpu_v, cores, sample = cpu_sample(15.0)
    line = {
        "metric": METRIC, "value": r["value"], "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": r["ms"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "per_gpu_units": B * H, "global_units": B * H * world,
                   "sharding": "(batch x head) units, no data-path collective",
                   "l2": "inputs (1 GiB per step) are larger than the 126 MB L2",
                   "flops_per_step": FWD_FLOPS + BWD_FLOPS},
        "clocks": r["clocks"], "e2e": r["e2e"], "gpu_launches": 4 * args.steps,
        "roofline": r["roofline"],
        "cpu_baseline": {"value": cpu_v, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "cpu_sdpa": cpu_sdpa_sample(),
        "kernels": r["kern"], "decode": r["decode"], "other_configs": r["extras"],
        "device_wait_status": r["wait_status"],
        "frac_of_2250_datasheet": r["value"] / world / 2250.0, "gather_ms": r["gather_ms"],
    }
    if r["strong"] is not None:
        line["strong"] = r["strong"]
        line["sharded_other_configs"] = r["sharded"]
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--profile-case", nargs="?", const="dense", default=None,
                    choices=["dense", "dense_nc", "varlen", "decode", "int8"],
                    help="run only W+K steps of one small case and exit (for ncu captures); default: dense")
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
    result = None
    try:
        result = run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
            dist.destroy_process_group()
    # the CPU baselines run after the process group is gone: no rank spins in a collective and
    # takes host cores away from them
    if rank == 0 and result is not None:
        print_line(args, world, result)


if __name__ == "__main__":
    main()
