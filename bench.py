#!/usr/bin/env python
"""Benchmark of the cascading-KV-cache hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload (``config.workload`` = "c2_llama8b_decode"): one decode step at Llama-3.1-8B attention
shapes in bf16 -- batch 16, 32 query / 8 KV heads, head_dim 128, 64 sinks, 8 cascades x 8192 slots
(65536), cache fully populated, EMA admission rule (beta 0.9999, max head reduction).  A step =
attention of one new token per sequence over sinks + cache + itself with cache-position RoPE, the
EMA score update of all slots, and the cascade cache update.  With N > 1 every rank runs the same
workload on its own GPU (lanes are independent: no data-path collective), so scaling is weak.

Reported metric: achieved HBM GB/s = algorithmic bytes per step (K and V read once, score cache
read+written once, q/out/new k,v once) / step time, summed over ranks; ``ms_per_step`` carries the
latency.  ``e2e`` is the same metric with the step's q/k/v copied from pinned host memory and the
output copied back inside the timed region.

``--impl reference`` times the CPU restatement of the reference path (oracle/) on the host cores
on a bounded sample (one sequence of the batch) of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

WORKLOADS = {
    "c2_llama8b_decode": dict(B=16, H=32, KVH=8, D=128, NS=64, W=8192, C=8, theta=500000.0, beta=0.9999,
                              admission="ema", head_reduction="max", seed=1),
    "c4_qwen2_decode": dict(B=32, H=28, KVH=4, D=128, NS=4, W=2048, C=8, theta=1000000.0, beta=0.9999,
                            admission="stride", head_reduction="max", seed=3),
}
METRIC = "decode_attn_cache_update_hbm_gbs"
UNIT = "GB/s"


def measured_peak_hbm():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: through NVML every 5 ms
    (read-only queries), or with one nvidia-smi process per sample when NVML cannot be loaded."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    # NVML clocks-event-reason bits, in the order of `NAMES` (the first four are what nvidia-smi is asked for)
    BITS = (0x8, 0x40, 0x20, 0x4, 0x2, 0x10, 0x80, 0x100)
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap", "applications_clocks_setting",
             "sync_boost", "hw_power_brake_slowdown", "display_clock_setting")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.samples = []          # (sm_mhz, max_mhz, [bool per reason])
        self.power = []            # watts
        self.source = "nvidia-smi"
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None
        self._handle = None
        try:
            import pynvml
            pynvml.nvmlInit()
            try:
                uuid = str(torch.cuda.get_device_properties(gpu_index).uuid)
                self._handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
            except Exception:
                self._handle = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
            self._nvml = pynvml
            self.source = "nvml"
        except Exception:
            self._nvml = None

    def _sample_nvml(self):
        n = self._nvml
        sm = n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM)
        mx = n.nvmlDeviceGetMaxClockInfo(self._handle, n.NVML_CLOCK_SM)
        try:
            mask = n.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
        except Exception:
            mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
        self.samples.append((float(sm), float(mx), [bool(mask & b) for b in self.BITS]))
        try:
            self.power.append(n.nvmlDeviceGetPowerUsage(self._handle) / 1000.0)
        except Exception:
            pass

    def _sample_smi(self):
        out = subprocess.run(["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}",
                              "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
        parts = [p.strip() for p in out.stdout.strip().split(",")]
        if len(parts) >= 6:
            self.samples.append((float(parts[0]), float(parts[1]),
                                 [x.lower().startswith("active") for x in parts[2:6]] + [False] * 4))

    def _run(self):
        while not self._stop.is_set():
            try:
                if self._nvml is not None:
                    self._sample_nvml()
                else:
                    self._sample_smi()
            except Exception:
                pass
            self._stop.wait(0.005 if self._nvml is not None else 0.1)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(s[0] for s in self.samples)
        reasons = [n for i, n in enumerate(self.NAMES) if any(s[2][i] for s in self.samples)]
        out = {"sm_mhz": sm[len(sm) // 2], "sm_min_mhz": sm[0], "sm_max_mhz": self.samples[0][1], "reasons": reasons,
               "samples": len(sm), "source": self.source}
        if self.power:
            out["power_w"] = sorted(self.power)[len(self.power) // 2]
        return out


def algorithmic_bytes(w):
    from cascading_kv_cache_b200.synthetic import decode_algorithmic_bytes
    return decode_algorithmic_bytes(w["B"], w["H"], w["KVH"], w["D"], w["NS"], w["W"] * w["C"],
                                    ema=w["admission"] == "ema")


def time_cpu_port(w, steps, warmup, batch_sample=1):
    """The CPU restatement of the reference path on the host cores: `batch_sample` sequences of the
    workload per step.  Returns (seconds per step, threads, bytes per step)."""
    from oracle.cascade_oracle import OracleCascadingKVCache, cascade_attention_step
    from cascading_kv_cache_b200.synthetic import decode_algorithmic_bytes, populate_steady_state
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    S = w["W"] * w["C"]
    dt = torch.bfloat16
    cache = OracleCascadingKVCache(w["W"], w["NS"], batch_sample, w["KVH"], w["D"], S, dtype=dt,
                                   head_reduction=w["head_reduction"], layers=1, eager_fill=True, beta=w["beta"])
    populate_steady_state(cache, 0, seed=w["seed"], beta=w["beta"])
    g = torch.Generator().manual_seed(w["seed"] + 100)
    times = []
    for it in range(warmup + steps):
        q = torch.randn(batch_sample, w["H"], 1, w["D"], generator=g).to(dt)
        k = torch.randn(batch_sample, w["KVH"], 1, w["D"], generator=g).to(dt)
        v = torch.randn(batch_sample, w["KVH"], 1, w["D"], generator=g).to(dt)
        t0 = time.perf_counter()
        if w["admission"] == "ema":
            cascade_attention_step(q, k, v, cache, 0, w["theta"], w["head_reduction"], False)
        else:
            cascade_attention_step(q, k, v, cache, 0, w["theta"], w["head_reduction"], False, do_update=False)
            cache.update(k, v, 0)
        dtm = time.perf_counter() - t0
        if it >= warmup:
            times.append(dtm)
    nbytes = decode_algorithmic_bytes(batch_sample, w["H"], w["KVH"], w["D"], w["NS"], S,
                                      ema=w["admission"] == "ema")
    return sum(times) / len(times), threads, nbytes


PREFILL = dict(B=1, H=32, KVH=8, D=128, NS=4, W=8192, C=4, K=4096, theta=500000.0, beta=0.9999,
               admission="ema", head_reduction="max", seed=2)


def measured_peak_tflops():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
        except Exception:
            pass
    return 1590.0, 1400.0, "fallback"


def run_prefill_leg(dev, chunks=6, warm=2, admission=None):
    """Chunked prefill at the c3 shapes (batch 1, 32/8 heads, 4 sinks, 4 x 8192 slots, chunk 4096) on a full
    cache: attention of the chunk + fused score/cache update per chunk.  ``admission`` "ema" (c3 itself: two
    passes over the keys, because the column scores need exactly normalised probabilities) or "stride" (the
    other admission rule at the same shapes: no column scores, one pass)."""
    from cascading_kv_cache_b200 import CascadingKVCache, cascade_attention, profiling
    from cascading_kv_cache_b200.synthetic import populate_steady_state, prefill_algorithmic_flops
    w = dict(PREFILL, admission=admission or PREFILL["admission"])
    B, H, KVH, D, NS, W, C, K = (w[k] for k in ("B", "H", "KVH", "D", "NS", "W", "C", "K"))
    S = W * C
    dt = torch.bfloat16
    cache = CascadingKVCache(W, NS, B, KVH, D, S, device=dev, dtype=dt, head_reduction=w["head_reduction"],
                             layers=1, eager_fill=True, admission=w["admission"])
    populate_steady_state(cache, 0, seed=w["seed"], beta=w["beta"])
    g = torch.Generator(device=dev).manual_seed(77)
    pool = 3
    qs = torch.randn(pool, B, H, K, D, generator=g, device=dev).to(dt)
    ks = torch.randn(pool, B, KVH, K, D, generator=g, device=dev).to(dt)
    vs = torch.randn(pool, B, KVH, K, D, generator=g, device=dev).to(dt)
    out = torch.empty(B, H, K, D, device=dev, dtype=dt)

    def step(i):
        j = i % pool
        cascade_attention(qs[j], ks[j], vs[j], cache, 0, rope_theta=w["theta"], out=out)

    for i in range(warm):
        step(i)
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(dev.index or 0) as clocks:
        ev0.record()
        for i in range(chunks):
            step(i)
        ev1.record()
        torch.cuda.synchronize()
    ms_chunk = ev0.elapsed_time(ev1) / chunks
    k_ms, _, k_name = profiling.time_dominant_kernel(step, n_steps=3)
    launches = profiling.last_launch_count()
    torch.cuda.synchronize()
    flops = prefill_algorithmic_flops(B, H, D, K, NS + S)
    burst, sustained, kind = measured_peak_tflops()
    return {"workload": "c3_chunked_prefill_full_cache", "admission": w["admission"], "chunk_tokens": K,
            "tokens_per_s": K / (ms_chunk * 1e-3),
            "ms_per_chunk": ms_chunk, "algorithmic_tflop_per_chunk": flops / 1e12,
            "tflops": flops / (ms_chunk * 1e-3) / 1e12, "kernel": k_name, "kernel_ms": k_ms,
            "kernel_tflops": flops / (k_ms * 1e-3) / 1e12, "peak_tflops": burst, "peak_kind": kind,
            "kernel_frac_of_peak": flops / (k_ms * 1e-3) / 1e12 / burst, "launches_per_chunk": launches,
            "clocks": clocks.summary(), "status": cache.kernel_status()}


def run_reference(args, w, rank, world):
    if rank != 0:
        return
    steps, warmup = max(1, min(args.steps, 3)), max(1, min(args.warmup, 1))
    sec, threads, nbytes = time_cpu_port(w, steps, warmup)
    gbs = nbytes / sec / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "sample": "1 of %d sequences per step" % w["B"]},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "CPU restatement of the reference eager attention + cache update (oracle/), "
                                   "1 of %d sequences per step, full cache length" % w["B"]},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--workload", default="c2_llama8b_decode", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--force-generic", action="store_true")
    ap.add_argument("--batch", type=int, default=0, help="override the batch (smaller cases for profiler captures)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (profiler captures)")
    ap.add_argument("--no-profile", action="store_true", help="skip the per-kernel event timing")
    ap.add_argument("--no-prefill", action="store_true", help="skip the chunked-prefill leg")
    ap.add_argument("--prefill-only", action="store_true", help="run only the chunked-prefill leg (profiler captures)")
    ap.add_argument("--prefill-chunks", type=int, default=6)
    ap.add_argument("--prefill-admission", choices=["ema", "stride"], default="ema")
    args = ap.parse_args()
    w = dict(WORKLOADS[args.workload])
    if args.batch > 0:
        w["B"] = args.batch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, w, rank, world)
        return
    if args.prefill_only:
        torch.cuda.set_device(local_rank)
        print(json.dumps({"prefill": run_prefill_leg(torch.device("cuda", local_rank), chunks=args.prefill_chunks,
                                                     warm=1, admission=args.prefill_admission)}), flush=True)
        return

    import torch.distributed as dist
    from cascading_kv_cache_b200 import CascadingKVCache, cascade_attention
    from cascading_kv_cache_b200.synthetic import populate_steady_state

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    steps, warmup = args.steps, max(args.warmup, 3)
    B, H, KVH, D, NS, W, C = (w[k] for k in ("B", "H", "KVH", "D", "NS", "W", "C"))
    S = W * C
    dt = torch.bfloat16
    cache = CascadingKVCache(W, NS, B, KVH, D, S, device=dev, dtype=dt, head_reduction=w["head_reduction"],
                             layers=1, eager_fill=True, admission=w["admission"])
    populate_steady_state(cache, 0, seed=w["seed"] + rank, beta=w["beta"])

    # fresh N(0,1) q/k/v for every step, resident in HBM before the timed region (a pool that is cycled)
    pool = 64
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    qs = torch.randn(pool, B, H, 1, D, generator=g, device=dev).to(dt)
    ks = torch.randn(pool, B, KVH, 1, D, generator=g, device=dev).to(dt)
    vs = torch.randn(pool, B, KVH, 1, D, generator=g, device=dev).to(dt)
    out = torch.empty(B, H, 1, D, device=dev, dtype=dt)

    def step(i):
        j = i % pool
        cascade_attention(qs[j], ks[j], vs[j], cache, 0, rope_theta=w["theta"], out=out,
                          force_generic=args.force_generic)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(warmup):
        step(i)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        ev0.record()
        for i in range(steps):
            step(warmup + i)
        ev1.record()
        barrier()
    ms_total = ev0.elapsed_time(ev1)

    # end to end: pinned host inputs -> device, step, output -> host, every step
    hq, hk, hv = (t.cpu().pin_memory() for t in (qs, ks, vs))
    hout = torch.empty(B, H, 1, D, dtype=dt).pin_memory()
    dq, dk, dv = (torch.empty_like(t[0]) for t in (qs, ks, vs))
    e2e_steps = max(3, min(steps, 50))

    def e2e_step(i):
        j = i % pool
        dq.copy_(hq[j], non_blocking=True)
        dk.copy_(hk[j], non_blocking=True)
        dv.copy_(hv[j], non_blocking=True)
        cascade_attention(dq, dk, dv, cache, 0, rope_theta=w["theta"], out=out, force_generic=args.force_generic)
        hout.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller reads the result

    ms_e2e_total = float("nan")
    if not args.no_e2e:
        for i in range(3):
            e2e_step(i)
        barrier()
        ev2, ev3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev2.record()
        for i in range(e2e_steps):
            e2e_step(i)
        ev3.record()
        barrier()
        ms_e2e_total = ev2.elapsed_time(ev3)

    from cascading_kv_cache_b200.dist_utils import max_over_ranks
    ms_total, ms_e2e_total = max_over_ranks([ms_total, ms_e2e_total], device=dev)

    nbytes = algorithmic_bytes(w)
    ms_step = ms_total / steps
    ms_e2e = ms_e2e_total / e2e_steps
    value = world * nbytes / (ms_step * 1e-3) / 1e9
    e2e_value = world * nbytes / (ms_e2e * 1e-3) / 1e9
    peak, peak_kind = measured_peak_hbm()

    if rank == 0:
        from cascading_kv_cache_b200 import profiling
        if args.no_profile:
            step(0)
            k_ms, k_name = ms_step, "whole step"
        else:
            k_ms, k_n, k_name = profiling.time_dominant_kernel(step, n_steps=min(steps, 50))
        launches_per_step = profiling.last_launch_count()
        torch.cuda.synchronize()
        prof = {"ms": k_ms, "gbs": nbytes / (k_ms * 1e-3) / 1e9, "kernel": k_name,
                "traffic": profiling.recorded_dram_traffic(args.workload, k_name)}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms_step, "us_per_step": ms_step * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "batch_per_gpu": B, "q_heads": H, "kv_heads": KVH, "head_dim": D,
                       "sinks": NS, "cascades": C, "window": W, "admission": w["admission"],
                       "l2": "inputs larger than L2 (%.2f GB of K/V per step)" % (nbytes / 1e9),
                       "path": "generic" if args.force_generic else "tuned"},
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": int(dq.numel() + dk.numel() + dv.numel()) * 2,
                    "d2h_bytes_per_step": int(out.numel()) * 2},
            "gpu_launches": launches_per_step * steps,
            "clocks": clocks.summary(),
            "roofline": {"bound": "hbm", "achieved": prof["gbs"], "peak": peak, "unit": "GB/s",
                         "frac": prof["gbs"] / peak, "peak_kind": peak_kind, "traffic": prof.get("traffic"),
                         "kernel": prof["kernel"], "kernel_ms": prof["ms"],
                         "step_frac": (nbytes / (ms_step * 1e-3) / 1e9) / peak},
        }
        if not args.no_prefill:
            del qs, ks, vs
            line["prefill"] = run_prefill_leg(dev)
            line["prefill_stride_rule"] = run_prefill_leg(dev, admission="stride")
        if not args.no_cpu_baseline:
            sec, threads, cpu_bytes = time_cpu_port(w, steps=2, warmup=1)
            line["cpu_baseline"] = {
                "value": cpu_bytes / sec / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
                "ms_per_step_full_batch": sec * 1e3 * B,
                "sample": "CPU restatement of the reference path (oracle/), 1 of %d sequences per step, "
                          "2 timed steps after 1 warm-up; full-batch time is the sample x %d" % (B, B)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
