#!/usr/bin/env python
"""Benchmark of the cascading-KV-cache hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Headline workload (``config.workload`` = "c2_llama8b_decode"): one decode step at Llama-3.1-8B attention
shapes in bf16 -- batch 16, 32 query / 8 KV heads, head_dim 128, 64 sinks, 8 cascades x 8192 slots (65536),
cache fully populated, EMA admission rule (beta 0.9999, max head reduction).  A step = attention of one new
token per sequence over sinks + cache + itself with cache-position RoPE, the EMA score update of all slots,
and the cascade cache update.

With N > 1 the GLOBAL workload is partitioned: lanes (sequence, KV head) are independent, so rank r owns
sequences [r*16/N, (r+1)*16/N) with exactly the data a single GPU holds for them (no data-path collective;
``torch.distributed`` only carries the barrier and the max-over-ranks of the times) -> ``"scaling": "strong"``.
The old behaviour, every rank running the whole batch, is reported next to it as ``weak_replicas``.

Reported metric: achieved HBM GB/s = algorithmic bytes of the whole job per step (K and V read once, score
cache read+written once, q/out/new k,v once) / step time (max over ranks); ``ms_per_step`` carries the latency.
The timed loop replays CUDA graphs of several consecutive steps (the kernels take every counter from device
memory, so a step needs nothing from the host).  ``e2e`` is the same metric through the Python call a user
makes, one synchronous host round trip per step: the step's q|k|v copied from pinned host memory, the call, the
output copied back and waited for, all inside the timed region (a one-step graph; the eager figure beside it).

Further keys of the same JSON line: ``sustained`` (1000 steps, as the configuration is written), ``c4`` (the
Qwen2-7B decode configuration, batch 32 split over the ranks), ``prefill`` / ``prefill_stride_rule`` (a
4096-token chunk over the full 4 x 8192 cache at the c3 shapes, KV heads split over the ranks),
``prefill_stream`` (c3 as written: 1,048,576 tokens in 256 chunks from an empty cache), ``host_us_per_call``,
``cpu_baseline`` (the CPU restatement of the reference path under oracle/ on the host cores, bounded samples).

``--impl reference`` times that CPU restatement alone, on all host threads, on a bounded sample of the same
workload (the reference is a Python project and does not travel to the GPU box).
"""
import argparse
import json
import math
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
PREFILL = dict(B=1, H=32, KVH=8, D=128, NS=4, W=8192, C=4, K=4096, theta=500000.0, beta=0.9999,
               admission="ema", head_reduction="max", seed=2)
METRIC = "decode_attn_cache_update_hbm_gbs"
UNIT = "GB/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            return dict(hbm=float(d["hbm_gbs"]), tf=float(d["bf16_tflops"]),
                        tf_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), kind="measured")
        except Exception:
            pass
    return dict(hbm=6650.0, tf=1590.0, tf_sustained=1400.0, kind="fallback")


def recorded_dram_traffic(workload, kernel, lanes):
    """DRAM bytes per launch of ``kernel`` from the committed ncu summary (profiles/dram_traffic.json holds
    bytes per lane of the captured case; traffic grows in proportion to the lanes a launch covers)."""
    try:
        per_lane = json.load(open(os.path.join(ROOT, "profiles", "dram_traffic.json")))[workload][kernel]["bytes_per_lane"]
        return int(per_lane * lanes)
    except Exception:
        return None


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


class Job:
    """Rank bookkeeping: barrier, max over ranks, device."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.dev = None
        self.dist = None

    def start(self):
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, values):
        from cascading_kv_cache_b200.dist_utils import max_over_ranks
        return max_over_ranks(values, device=self.dev)

    def stop(self):
        if self.dist is not None:
            self.dist.barrier()
            self.dist.destroy_process_group()


def steps_per_graph(steps, limit=20):
    """Largest divisor of ``steps`` up to ``limit``: the timed loop replays whole graphs and runs exactly ``steps``."""
    for g in range(min(steps, limit), 0, -1):
        if steps % g == 0:
            return g
    return 1


def timed_steps(job, step, note_seen, steps, warmup, graph=True, sample_clocks=True):
    """``warmup`` untimed steps, then exactly ``steps`` steps bracketed by barrier + synchronize on both sides,
    CUDA events on the launching stream.  Returns (ms for all steps, max over ranks; clock summary)."""
    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    G = steps_per_graph(steps) if graph else 1
    if G > 1:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        cg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(cg, stream=side):
            for j in range(G):
                step(warmup + j)
        note_seen(-G)                      # capturing ran the host mirror forward, not the device
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()

        def run(i):
            cg.replay()
            note_seen(G)
        run(0)                             # one untimed replay
        n_iter = steps // G
    else:
        run, n_iter = (lambda i: step(warmup + i)), steps
    job.barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(job.local_rank) if sample_clocks else None
    if sampler:
        sampler.__enter__()
    job.barrier()
    ev0.record()
    for i in range(n_iter):
        run(i)
    ev1.record()
    job.barrier()
    if sampler:
        sampler.__exit__()
    ms = job.max_over_ranks([ev0.elapsed_time(ev1)])[0]
    return ms, (sampler.summary() if sampler else None), G


def decode_bytes(w, B):
    from cascading_kv_cache_b200.synthetic import decode_algorithmic_bytes
    return decode_algorithmic_bytes(B, w["H"], w["KVH"], w["D"], w["NS"], w["W"] * w["C"], ema=w["admission"] == "ema")


class DecodeCase:
    """One rank's share of a decode workload: cache, a pool of fresh N(0,1) inputs resident in HBM, the step."""

    def __init__(self, job, w, partition=True, force_generic=False):
        from cascading_kv_cache_b200 import CascadingKVCache
        from cascading_kv_cache_b200.dist_utils import shard_lanes
        from cascading_kv_cache_b200.synthetic import populate_steady_state
        self.w, self.job, self.force_generic = w, job, force_generic
        B, H, KVH, D, NS, W, C = (w[k] for k in ("B", "H", "KVH", "D", "NS", "W", "C"))
        b0, b1 = shard_lanes(B, KVH, job.world, job.rank)["batch"] if partition else (0, B)
        self.B_local, self.B_global = b1 - b0, (B if partition else B * job.world)
        dt, dev = torch.bfloat16, job.dev
        self.cache = CascadingKVCache(W, NS, self.B_local, KVH, D, W * C, device=dev, dtype=dt,
                                      head_reduction=w["head_reduction"], layers=1, eager_fill=True,
                                      admission=w["admission"], verbose=False)
        first = b0 if partition else job.rank * B      # replicas: every rank its own sequences
        populate_steady_state(self.cache, 0, seed=w["seed"], beta=w["beta"], first_sequence=first)
        self.pool = 64
        g = torch.Generator(device=dev).manual_seed(1000 + w["seed"])
        full = lambda h: torch.randn(self.pool, B, h, 1, D, generator=g, device=dev).to(dt)
        sl = slice(b0, b1) if partition else slice(0, B)
        self.qs, self.ks, self.vs = (full(h)[:, sl].contiguous() for h in (H, KVH, KVH))
        self.out = torch.empty(self.B_local, H, 1, D, device=dev, dtype=dt)
        self.bytes_local = decode_bytes(w, self.B_local)
        self.bytes_global = decode_bytes(w, self.B_global)

    def step(self, i):
        from cascading_kv_cache_b200 import cascade_attention
        j = i % self.pool
        cascade_attention(self.qs[j], self.ks[j], self.vs[j], self.cache, 0, rope_theta=self.w["theta"], out=self.out,
                          force_generic=self.force_generic)

    def note_seen(self, n):
        self.cache.note_tokens_seen(0, n)

    def run(self, steps, warmup, graph=True):
        ms, clocks, G = timed_steps(self.job, self.step, self.note_seen, steps, warmup, graph=graph)
        ms_step = ms / steps
        return dict(ms_per_step=ms_step, us_per_step=ms_step * 1e3, gbs=self.bytes_global / (ms_step * 1e-3) / 1e9,
                    batch_per_gpu=self.B_local, steps=steps, steps_per_graph=G, clocks=clocks)

    def run_e2e(self, steps):
        """Pinned host q|k|v -> device, the call a user makes, output -> host, and a wait for the result, every
        step.  The three inputs of a step travel as one buffer (they are the output of one fused projection in a
        model) and the call takes them as strided views of it.  Timed twice: issued call by call, and as a graph."""
        from cascading_kv_cache_b200 import cascade_attention
        H, KVH = self.qs.size(2), self.ks.size(2)
        hqkv = torch.cat([self.qs, self.ks, self.vs], dim=2).cpu().pin_memory()      # [pool, B, H + 2 KVH, 1, D]
        hout = torch.empty_like(self.out, device="cpu").pin_memory()
        dqkv = torch.empty_like(hqkv[0], device=self.qs.device)
        dq, dk, dv = dqkv[:, :H], dqkv[:, H:H + KVH], dqkv[:, H + KVH:]

        def e2e_step(i):
            dqkv.copy_(hqkv[i % self.pool], non_blocking=True)
            cascade_attention(dq, dk, dv, self.cache, 0, rope_theta=self.w["theta"], out=self.out,
                              force_generic=self.force_generic)
            hout.copy_(self.out, non_blocking=True)
            torch.cuda.current_stream().synchronize()  # the caller reads the result

        ms, _, _ = timed_steps(self.job, e2e_step, self.note_seen, steps, 3, graph=False, sample_clocks=False)
        eager_ms = ms / steps

        # The same step as a serving loop would issue it: the host writes the step's inputs into one pinned staging
        # buffer, replays a graph of [host -> device copy, the call, device -> host copy] and waits for the result.
        stage = torch.empty_like(hqkv[0]).pin_memory()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        cg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(cg, stream=side):
            dqkv.copy_(stage, non_blocking=True)
            cascade_attention(dq, dk, dv, self.cache, 0, rope_theta=self.w["theta"], out=self.out,
                              force_generic=self.force_generic)
            hout.copy_(self.out, non_blocking=True)
        self.note_seen(-1)                 # capturing ran the host mirror forward, not the device
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()

        def graph_step(i):
            stage.copy_(hqkv[i % self.pool])           # host memory to host memory: this step's inputs
            cg.replay()
            self.note_seen(1)
            torch.cuda.current_stream().synchronize()  # the caller reads the result

        ms, _, _ = timed_steps(self.job, graph_step, lambda n: None, steps, 3, graph=False, sample_clocks=False)
        ms_step = ms / steps
        world = self.job.world
        return {"value": self.bytes_global / (ms_step * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": ms_step,
                "h2d_bytes_per_step": int(dqkv.numel()) * 2 * world,
                "d2h_bytes_per_step": int(self.out.numel()) * 2 * world,
                "launch": "one CUDA graph per step: pinned host q|k|v -> device, the call, output -> pinned host; the host "
                          "waits for every step's result",
                "eager_ms_per_step": eager_ms}

    def host_us_per_call(self, calls=200):
        """Host time to issue one call (marshalling + launches), measured while the GPU keeps up or not: the
        smaller of the enqueue time and the device time bounds what the host adds per step."""
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(calls):
            self.step(i)
        t1 = time.perf_counter()
        torch.cuda.synchronize()
        return (t1 - t0) / calls * 1e6

    def kernel_profile(self, n_steps):
        from cascading_kv_cache_b200 import profiling
        k_ms, k_n, k_name = profiling.time_dominant_kernel(self.step, n_steps=n_steps)
        self.breakdown = {name: ms for name, ms, _ in profiling.kernel_breakdown()}
        launches = profiling.last_launch_count()
        torch.cuda.synchronize()
        return k_ms, k_name, launches


class PrefillCase:
    """One rank's KV heads of the c3 chunked-prefill workload (batch 1: the lanes to split are the heads)."""

    def __init__(self, job, admission, populate=True):
        from cascading_kv_cache_b200 import CascadingKVCache
        from cascading_kv_cache_b200.dist_utils import shard_lanes
        from cascading_kv_cache_b200.synthetic import populate_steady_state
        w = self.w = dict(PREFILL, admission=admission)
        B, H, KVH, D, NS, W, C, K = (w[k] for k in ("B", "H", "KVH", "D", "NS", "W", "C", "K"))
        h0, h1 = shard_lanes(B, KVH, job.world, job.rank)["kv_heads"]
        self.job, self.kvh_local, G = job, h1 - h0, H // KVH
        dt, dev = torch.bfloat16, job.dev
        self.cache = CascadingKVCache(W, NS, B, self.kvh_local, D, W * C, device=dev, dtype=dt,
                                      head_reduction=w["head_reduction"], layers=1, eager_fill=True,
                                      admission=admission, verbose=False)
        if populate:
            populate_steady_state(self.cache, 0, seed=w["seed"], beta=w["beta"], first_kv_head=h0, global_kv_heads=KVH)
        else:
            self.cache.beta = w["beta"]
        g = torch.Generator(device=dev).manual_seed(77)
        self.pool = 3
        full = lambda h: torch.randn(self.pool, B, h, K, D, generator=g, device=dev).to(dt)
        self.qs = full(H)[:, :, h0 * G:h1 * G].contiguous()
        self.ks, self.vs = (full(KVH)[:, :, h0:h1].contiguous() for _ in range(2))
        self.out = torch.empty(B, self.kvh_local * G, K, D, device=dev, dtype=dt)

    def step(self, i):
        from cascading_kv_cache_b200 import cascade_attention
        j = i % self.pool
        cascade_attention(self.qs[j], self.ks[j], self.vs[j], self.cache, 0, rope_theta=self.w["theta"], out=self.out)

    def note_seen(self, n):
        self.cache.note_tokens_seen(0, n * self.w["K"])

    def run_full_cache(self, chunks, warm):
        """Chunks over the fully populated cache: ms per chunk (max over ranks), the attention kernels' share."""
        from cascading_kv_cache_b200 import profiling
        from cascading_kv_cache_b200.synthetic import prefill_algorithmic_flops
        w = self.w
        ms, clocks, _ = timed_steps(self.job, self.step, self.note_seen, chunks, warm, graph=False)
        ms_chunk = ms / chunks
        k_ms, _, k_name = profiling.time_dominant_kernel(self.step, n_steps=3)
        launches = profiling.last_launch_count()
        torch.cuda.synchronize()
        k_ms = self.job.max_over_ranks([k_ms])[0]
        flops = prefill_algorithmic_flops(w["B"], w["H"], w["D"], w["K"], w["NS"] + w["W"] * w["C"])   # whole job
        peaks = measured_peaks()
        n = self.job.world
        return {"workload": "c3_chunked_prefill_full_cache", "admission": w["admission"], "chunk_tokens": w["K"],
                "kv_heads_per_gpu": self.kvh_local, "tokens_per_s": w["K"] / (ms_chunk * 1e-3),
                "ms_per_chunk": ms_chunk, "algorithmic_tflop_per_chunk": flops / 1e12,
                "tflops": flops / (ms_chunk * 1e-3) / 1e12, "kernel": k_name, "kernel_ms": k_ms,
                "kernel_tflops": flops / (k_ms * 1e-3) / 1e12, "peak_tflops": peaks["tf"] * n,
                "peak_kind": peaks["kind"], "kernel_frac_of_peak": flops / (k_ms * 1e-3) / 1e12 / (peaks["tf"] * n),
                "chunk_frac_of_peak": flops / (ms_chunk * 1e-3) / 1e12 / (peaks["tf"] * n),
                "launches_per_chunk": launches, "clocks": clocks, "status": self.cache.kernel_status()}

    def run_stream(self, chunks):
        """The configuration as written: ``chunks`` chunks of 4096 tokens streamed from an EMPTY cache (the
        eager-fill phase, then the steady state).  Tokens per second over the whole stream."""
        from cascading_kv_cache_b200.synthetic import prefill_algorithmic_flops
        w = self.w
        self.cache.reset(verbose=False)
        self.cache.beta = w["beta"]
        ms, clocks, _ = timed_steps(self.job, self.step, self.note_seen, chunks, 0, graph=False)
        S, K, NS = w["W"] * w["C"], w["K"], w["NS"]
        flops = sum(prefill_algorithmic_flops(w["B"], w["H"], w["D"], K, min(max(K * c - NS, 0), S) + (NS if c else 0))
                    for c in range(chunks))
        peaks = measured_peaks()
        n = self.job.world
        return {"workload": "c3_chunked_prefill_stream", "admission": w["admission"], "chunks": chunks,
                "tokens": chunks * K, "seconds": ms * 1e-3, "tokens_per_s": chunks * K / (ms * 1e-3),
                "ms_per_chunk": ms / chunks, "algorithmic_tflop": flops / 1e12,
                "tflops": flops / (ms * 1e-3) / 1e12,
                "frac_of_burst_peak": flops / (ms * 1e-3) / 1e12 / (peaks["tf"] * n),
                "frac_of_sustained_peak": flops / (ms * 1e-3) / 1e12 / (peaks["tf_sustained"] * n),
                "clocks": clocks, "status": self.cache.kernel_status()}


# ------------------------------------------------------------------------- CPU legs (oracle/ is the checker)
def time_cpu_decode(w, steps, warmup, batch_sample):
    """The CPU restatement of the reference path on the host cores: `batch_sample` sequences of the
    workload per step.  Returns (seconds per step, threads, bytes per step)."""
    from oracle.cascade_oracle import OracleCascadingKVCache, cascade_attention_step
    from cascading_kv_cache_b200.synthetic import populate_steady_state
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    S, dt = w["W"] * w["C"], torch.bfloat16
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
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    return sum(times) / len(times), threads, decode_bytes(w, batch_sample)


def time_cpu_prefill_head():
    """One KV head (with its 4 query heads) of one full-cache c3 chunk on the host cores."""
    from oracle.cascade_oracle import OracleCascadingKVCache, cascade_attention_step
    from cascading_kv_cache_b200.synthetic import populate_steady_state
    w = PREFILL
    torch.set_num_threads(os.cpu_count() or 1)
    G, dt = w["H"] // w["KVH"], torch.bfloat16
    cache = OracleCascadingKVCache(w["W"], w["NS"], 1, 1, w["D"], w["W"] * w["C"], dtype=dt,
                                   head_reduction=w["head_reduction"], layers=1, eager_fill=True, beta=w["beta"])
    populate_steady_state(cache, 0, seed=w["seed"], beta=w["beta"])
    g = torch.Generator().manual_seed(5)
    q = torch.randn(1, G, w["K"], w["D"], generator=g).to(dt)
    k = torch.randn(1, 1, w["K"], w["D"], generator=g).to(dt)
    v = torch.randn(1, 1, w["K"], w["D"], generator=g).to(dt)
    t0 = time.perf_counter()
    cascade_attention_step(q, k, v, cache, 0, w["theta"], w["head_reduction"], False)
    return time.perf_counter() - t0


def time_cpu_c1():
    """The reference's own CPU-runnable configuration in full: fp32, B1 H32/KVH8 D128, 4 sinks, 4 x 512 slots,
    stride rule, 16384 tokens in chunks of 512, then 64 decode steps."""
    from oracle.cascade_oracle import OracleCascadingKVCache, cascade_attention_step
    torch.set_num_threads(os.cpu_count() or 1)
    B, H, KVH, D, NS, W, C, theta = 1, 32, 8, 128, 4, 512, 4, 5e5
    ref = OracleCascadingKVCache(W, NS, B, KVH, D, W * C, dtype=torch.float32, layers=1, eager_fill=False)
    g = torch.Generator().manual_seed(0)
    t_prefill = t_decode = 0.0
    for n in [512] * 32 + [1] * 64:
        q = torch.randn(B, H, n, D, generator=g)
        k = torch.randn(B, KVH, n, D, generator=g)
        v = torch.randn(B, KVH, n, D, generator=g)
        t0 = time.perf_counter()
        cascade_attention_step(q, k, v, ref, 0, theta, None, False, do_update=False)
        ref.update(k, v, 0)
        dtm = time.perf_counter() - t0
        if n > 1:
            t_prefill += dtm
        else:
            t_decode += dtm
    return {"prefill_tokens_per_s": 16384 / t_prefill, "decode_us_per_step": t_decode / 64 * 1e6,
            "seconds_total": t_prefill + t_decode}


def run_c5(job, args):
    """End to end (``--workload c5_e2e``): the Llama-3.1-8B architecture with random-init bf16 weights (32 layers,
    hidden 4096, 32 q / 8 KV heads, FFN 14336, vocab 128256; N(0, 0.02) from seed 4, plain RoPE base 500000), a
    prompt of seeded uniform token ids prefilled in strides of 4096 through the cascading cache (window 32768,
    4 cascades, 64 sinks, EMA rule), then greedy decode tokens.  One sequence per GPU (rank r: seed 4 + r); the
    generated ids are gathered at the end, the only collective."""
    from cascading_kv_cache_b200.dist_utils import gather_token_ids
    from cascading_kv_cache_b200.thin_model import CascadeForCausalLM, cascade_config, get_cache
    dev = job.dev
    cfg = cascade_config("llama", num_hidden_layers=args.c5_layers)
    with torch.device(dev):
        model = CascadeForCausalLM(cfg, "llama").to(torch.bfloat16).eval()
    model.init_weights(seed=4)
    if args.c5_fuse:
        model.fuse_projections()       # q|k|v and gate|up as one projection each
    cache = get_cache(model)
    cache.beta = 0.9999
    g = torch.Generator().manual_seed(4 + job.rank)
    prompt = torch.randint(0, cfg.vocab_size, (1, args.c5_prompt), generator=g).to(dev)
    stride, n_new = cfg._cascade_stride, args.c5_new_tokens
    with torch.no_grad():      # warm-up on a scratch cache: kernel attributes, cuBLAS handles, workspaces
        warm = get_cache(model)
        model(prompt[:, :stride], past_key_values=warm, num_logits_to_keep=1)
        model(prompt[:, :1], past_key_values=warm, num_logits_to_keep=1)
        del warm
    torch.cuda.empty_cache()
    job.barrier()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    with ClockSampler(job.local_rank) as clocks, torch.no_grad():
        ev[0].record()
        for i in range(0, prompt.size(1), stride):
            out = model(prompt[:, i:i + stride], past_key_values=cache, num_logits_to_keep=1)
        ids = [out.logits[:, -1].argmax(-1)]
        ev[1].record()
        # the first half of the new tokens one host-driven forward at a time, the second half by replaying a
        # CUDA graph of one whole decode step (32 layers + lm_head + argmax; the kernels read every counter
        # from device memory, the host only advances its mirrors)
        n_eager = (n_new - 1) // 2 if args.c5_graph else n_new - 1
        for _ in range(n_eager):
            out = model(ids[-1][:, None], past_key_values=cache, num_logits_to_keep=1)
            ids.append(out.logits[:, -1].argmax(-1))
        ev[2].record()
        n_graph, graph_note = n_new - 1 - n_eager, None
        if n_graph > 0:
            try:
                tok_in = ids[-1][:, None].clone()
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                cg = torch.cuda.CUDAGraph()
                with torch.cuda.graph(cg, stream=side):
                    tok_out = model(tok_in, past_key_values=cache, num_logits_to_keep=1).logits[:, -1].argmax(-1)
                for l in range(cfg.num_hidden_layers):
                    cache.note_tokens_seen(l, -1)        # capturing ran the host mirrors forward, not the device
                torch.cuda.current_stream().wait_stream(side)
                ev.append(torch.cuda.Event(enable_timing=True))
                ev.append(torch.cuda.Event(enable_timing=True))
                ev[3].record()
                for _ in range(n_graph):
                    cg.replay()
                    for l in range(cfg.num_hidden_layers):
                        cache.note_tokens_seen(l, 1)
                    ids.append(tok_out.clone())
                    tok_in.copy_(tok_out[:, None])
                ev[4].record()
            except Exception as exc:                     # keep the line: finish the tokens without a graph
                graph_note = "graph capture failed: %s" % str(exc)[:200]
                torch.cuda.synchronize()
                for _ in range(n_new - len(ids)):
                    out = model(ids[-1][:, None], past_key_values=cache, num_logits_to_keep=1)
                    ids.append(out.logits[:, -1].argmax(-1))
        job.barrier()
    ids = torch.stack(ids, dim=1)[0]
    all_ids = gather_token_ids(ids)
    ms_prefill, ms_decode = job.max_over_ranks([ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2])])
    ms_graph = job.max_over_ranks([ev[3].elapsed_time(ev[4])])[0] if len(ev) == 5 else None
    if job.rank == 0:
        n = job.world
        line = {"metric": "e2e_prefill_tokens_per_s", "value": n * args.c5_prompt / (ms_prefill * 1e-3), "unit": "tokens/s",
                "n_gpus": n, "steps": 1, "warmup": 1, "ms_per_step": ms_prefill + ms_decode, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": "c5_e2e", "layers": args.c5_layers, "prompt_tokens": args.c5_prompt,
                           "new_tokens": n_new, "stride": stride, "sequences_per_gpu": 1,
                           "rope": "theta 500000, no frequency scaling"},
                "prefill_s": ms_prefill * 1e-3, "decode_s": ms_decode * 1e-3,
                "decode_ms_per_token": ms_decode / max(n_eager, 1), "decode_tokens_timed": n_eager,
                "decode_tokens_per_s": n * n_eager / (ms_decode * 1e-3) if n_eager > 0 else None,
                "decode_graph_ms_per_token": ms_graph / n_graph if ms_graph else None,
                "decode_graph_tokens_per_s": n * n_graph / (ms_graph * 1e-3) if ms_graph else None,
                "decode_graph_tokens_timed": n_graph if ms_graph else 0, "decode_graph_note": graph_note,
                "generated_ids_shape": list(all_ids.shape), "first_ids": all_ids[0, :8].tolist(),
                "cache_tokens": cache.get_seq_length(0), "kernel_status": cache.kernel_status(),
                "clocks": clocks.summary()}
        print(json.dumps(line), flush=True)


def cpu_sample_size(w):
    return max(1, w["B"] // 4)


def run_reference(args, w, job):
    if job.rank != 0:
        return
    steps, warmup = max(1, min(args.steps, 3)), max(1, min(args.warmup, 1))
    sample = cpu_sample_size(w)
    sec, threads, nbytes = time_cpu_decode(w, steps, warmup, sample)
    gbs = nbytes / sec / 1e9
    what = ("CPU restatement of the reference eager attention + cache update (oracle/), %d of %d sequences per step, "
            "full cache length, %d timed steps" % (sample, w["B"], steps))
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": sec * 1e3, "ms_per_step_full_batch": sec * 1e3 * w["B"] / sample,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "sample": "%d of %d sequences per step" % (sample, w["B"])},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port", "sample": what},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--workload", default="c2_llama8b_decode", choices=sorted(WORKLOADS) + ["c5_e2e"])
    ap.add_argument("--c5-layers", type=int, default=32)
    ap.add_argument("--c5-prompt", type=int, default=131072)
    ap.add_argument("--c5-new-tokens", type=int, default=256)
    ap.add_argument("--c5-fuse", type=int, default=1, help="one projection for q|k|v and one for gate|up per layer")
    ap.add_argument("--c5-graph", type=int, default=1, help="decode the second half of the new tokens from a CUDA graph")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="N > 1: partition the global batch (strong, default) or run the whole batch on every rank")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--force-generic", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every step from the host instead of replaying graphs")
    ap.add_argument("--batch", type=int, default=0, help="override the global batch (smaller cases for profiler captures)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (profiler captures)")
    ap.add_argument("--no-profile", action="store_true", help="skip the per-kernel event timing")
    ap.add_argument("--no-extras", action="store_true",
                    help="headline only: skip sustained / c4 / prefill / stream legs (profiler captures)")
    ap.add_argument("--prefill-only", action="store_true", help="run only the chunked-prefill leg (profiler captures)")
    ap.add_argument("--prefill-chunks", type=int, default=6)
    ap.add_argument("--prefill-admission", choices=["ema", "stride"], default="ema")
    ap.add_argument("--sustained-steps", type=int, default=1000)
    ap.add_argument("--stream-chunks", type=int, default=256)
    args = ap.parse_args()
    job = Job()
    if args.workload == "c5_e2e":
        if args.impl == "reference":
            if job.rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": "the end-to-end configuration is timed on the "
                                  "GPU arm only; its CPU baseline is one layer-chunk (cpu_baseline.prefill of the default run)"}))
            return
        job.start()
        run_c5(job, args)
        job.stop()
        return
    w = dict(WORKLOADS[args.workload])
    if args.batch > 0:
        w["B"] = args.batch
    if args.impl == "reference":
        run_reference(args, w, job)
        return
    job.start()
    if args.prefill_only:
        res = PrefillCase(job, args.prefill_admission).run_full_cache(args.prefill_chunks, 1)
        if job.rank == 0:
            print(json.dumps({"prefill": res}), flush=True)
        job.stop()
        return

    steps, warmup = args.steps, max(args.warmup, 3)
    graph = not args.no_graph
    partition = args.scaling == "strong"
    peaks = measured_peaks()
    case = DecodeCase(job, w, partition=partition, force_generic=args.force_generic)
    head = case.run(steps, warmup, graph=graph)
    e2e = None if args.no_e2e else case.run_e2e(max(3, min(steps, 50)))

    if args.no_profile:
        k_ms, k_name, launches = head["ms_per_step"], "whole step", 3
    else:
        k_ms, k_name, launches = case.kernel_profile(min(steps, 50))
    k_ms = job.max_over_ranks([k_ms])[0]
    k_gbs = case.bytes_local / (k_ms * 1e-3) / 1e9
    lanes_local = case.B_local * w["KVH"]
    line = {
        "metric": METRIC, "value": head["gbs"], "unit": UNIT, "n_gpus": job.world, "steps": steps, "warmup": warmup,
        "ms_per_step": head["ms_per_step"], "us_per_step": head["us_per_step"], "higher_is_better": True,
        "scaling": args.scaling if job.world > 1 else "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": args.workload, "global_batch": case.B_global, "batch_per_gpu": case.B_local,
                   "q_heads": w["H"], "kv_heads": w["KVH"], "head_dim": w["D"], "sinks": w["NS"],
                   "cascades": w["C"], "window": w["W"], "admission": w["admission"],
                   "partition": "batch over ranks, no data-path collective" if partition else "replicas",
                   "launch": ("CUDA graphs of %d steps" % head["steps_per_graph"]) if head["steps_per_graph"] > 1
                   else "one host call per step",
                   "l2": "inputs larger than L2 (%.2f GB of K/V per GPU per step)" % (case.bytes_local / 1e9),
                   "path": "generic" if args.force_generic else "tuned"},
        "gpu_launches": launches * steps * job.world,
        "clocks": head["clocks"],
        "roofline": {"bound": "hbm", "achieved": k_gbs, "peak": peaks["hbm"], "unit": "GB/s",
                     "frac": k_gbs / peaks["hbm"], "peak_kind": peaks["kind"],
                     "traffic": recorded_dram_traffic(args.workload, k_name, lanes_local),
                     "kernel": k_name, "kernel_ms": k_ms, "per": "GPU (rank 0's share of the batch)",
                     "kernels_ms": getattr(case, "breakdown", None),
                     "step_frac": head["gbs"] / (peaks["hbm"] * job.world),
                     "step_frac_of_8tbs": head["gbs"] / (8000.0 * job.world)},
    }
    if e2e is not None:
        line["e2e"] = e2e
    line["host_us_per_call"] = job.max_over_ranks([case.host_us_per_call()])[0]

    if not args.no_extras:
        # short legs first, the two seconds-long ones (1000 decode steps, the 256-chunk stream) last: they drive
        # the part into its power cap, which would colour whatever is measured right after them
        if args.workload != "c4_qwen2_decode":
            w4 = dict(WORKLOADS["c4_qwen2_decode"])
            c4 = DecodeCase(job, w4, partition=True)
            r = c4.run(steps, warmup, graph=graph)
            r["step_frac"] = r["gbs"] / (peaks["hbm"] * job.world)
            r["host_us_per_call"] = job.max_over_ranks([c4.host_us_per_call()])[0]
            r["no_graph_ms_per_step"] = c4.run(steps, 3, graph=False)["ms_per_step"]
            r["e2e"] = c4.run_e2e(max(3, min(steps, 50)))
            r["workload"] = "c4_qwen2_decode"
            line["c4"] = r
            del c4
            torch.cuda.empty_cache()
        if job.world > 1 and partition:
            rep = DecodeCase(job, w, partition=False)
            r = rep.run(steps, warmup, graph=graph)
            line["weak_replicas"] = {"value": r["gbs"], "unit": UNIT, "ms_per_step": r["ms_per_step"],
                                     "batch_per_gpu": rep.B_local, "scaling": "weak"}
            del rep
            torch.cuda.empty_cache()
        pf = PrefillCase(job, "ema")
        line["prefill"] = pf.run_full_cache(args.prefill_chunks, 2)
        ps = PrefillCase(job, "stride")
        line["prefill_stride_rule"] = ps.run_full_cache(args.prefill_chunks, 2)
        del ps
        torch.cuda.empty_cache()
        # the configurations as written: 1000 decode steps; 1,048,576 tokens in 256 chunks from an empty cache
        sus = case.run(args.sustained_steps, 3, graph=graph)
        sus["frac_of_copy_peak"] = sus["gbs"] / (peaks["hbm"] * job.world)
        sus["frac_of_8tbs"] = sus["gbs"] / (8000.0 * job.world)
        line["sustained"] = sus
        line["prefill_stream"] = pf.run_stream(args.stream_chunks)
        del pf, case
        torch.cuda.empty_cache()

    if job.rank == 0:
        if not args.no_cpu_baseline and job.world == 1:
            sample = cpu_sample_size(w)
            sec, threads, cpu_bytes = time_cpu_decode(w, steps=2, warmup=1, batch_sample=sample)
            line["cpu_baseline"] = {
                "value": cpu_bytes / sec / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
                "ms_per_step_full_batch": sec * 1e3 * w["B"] / sample,
                "sample": "CPU restatement of the reference path (oracle/), %d of %d sequences per step, 2 timed "
                          "steps after 1 warm-up; full-batch time is the sample x %g" % (sample, w["B"], w["B"] / sample)}
            if not args.no_extras:
                sec_head = time_cpu_prefill_head()
                line["cpu_baseline"]["prefill"] = {
                    "tokens_per_s": PREFILL["K"] / (sec_head * PREFILL["KVH"]), "unit": "tokens/s",
                    "sample": "one KV head (4 query heads) of one full-cache 4096-token chunk: %.2f s; the chunk has "
                              "8 such heads, so the figure divides by 8 x that time" % sec_head}
                line["cpu_baseline"]["c1_fp32_stride_stream_in_full"] = time_cpu_c1()
        print(json.dumps(line), flush=True)
    job.stop()


if __name__ == "__main__":
    main()
