#!/usr/bin/env python
"""Benchmark of the KV-cache hot path: one decode step of 8 attention layers
(fused RMSNorm+RoPE+KV append, then gated GQA decode attention) at batch 128 per
GPU and 4096 keys per sequence, fp16 KV, per-sequence pointer tables.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line (rank 0).  `value` is algorithmic HBM bytes of the whole
job per second (GB/s) with every input resident in HBM; `e2e` is the same metric
through the host-buffer C-ABI entry (q/k/v/gate/tables copied from pinned host
memory and ctx copied back inside the timed region; the KV cache itself is state
that lives on the device).  Under torchrun each rank owns its own 128 sequences
(replicas, no data-path collective); torch.distributed is used only for the
barrier and the max-over-ranks of the device time.

--impl reference runs the reference's own kernels (its PTX, prebuilt into
oracle/_ref/*.cubin) on ONE B200 with the engine's launch sequence: 9 launches
per layer.  The reference has no CPU implementation of this path; the CPU figure
reported in `cpu_baseline` is the scalar oracle port on the host cores.
"""
from __future__ import annotations

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

NQ, NKV, HD = 16, 4, 128
LAYERS, BATCH, CTX = 8, 128, 4096
RAGGED = False  # --ragged: context lengths uniform 1024..4096 instead of 4096 for every sequence
ROW_BYTES = NKV * HD * 2
# algorithmic bytes per (layer, sequence): K and V rows read once per GQA group plus the
# step's q/k/v/gate, norm weights, cos/sin rows, K/V row writes, ctx write, table entries
PER_SEQ_FIXED = 4096 + 1024 + 1024 + 32 + 512 + 512 + 2048 + 4096 + 28


def alg_bytes_layer(seq_lens) -> int:
    return int(sum(2 * ROW_BYTES * int(s) + PER_SEQ_FIXED for s in seq_lens))


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only queries)
    every few milliseconds while a region runs; falls back to nvidia-smi if NVML is absent."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.stop_flag, self.sm, self.reasons, self.max_mhz = index, False, [], set(), None

    def run(self):
        try:
            import pynvml as N
            N.nvmlInit()
            h = N.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = int(N.nvmlDeviceGetMaxClockInfo(h, N.NVML_CLOCK_SM))
            names = {"hw_slowdown": getattr(N, "nvmlClocksEventReasonHwSlowdown", 0x8),
                     "hw_thermal_slowdown": getattr(N, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                     "sw_thermal_slowdown": getattr(N, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                     "sw_power_cap": getattr(N, "nvmlClocksEventReasonSwPowerCap", 0x4)}
            get = getattr(N, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                N.nvmlDeviceGetCurrentClocksThrottleReasons
            while not self.stop_flag:
                mhz, bits = int(N.nvmlDeviceGetClockInfo(h, N.NVML_CLOCK_SM)), int(get(h))
                self.sm.append((time.perf_counter(), mhz, tuple(k for k, v in names.items() if bits & v)))
                time.sleep(0.001)
        except Exception:
            self._run_smi()

    def _run_smi(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        while not self.stop_flag:
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={q}",
                                      "--format=csv,noheader,nounits"], capture_output=True,
                                     text=True, timeout=5).stdout.strip()
                r = [x.strip() for x in out.split(",")]
                if r and r[0].isdigit():
                    self.max_mhz = int(r[1])
                    self.sm.append((time.perf_counter(), int(r[0]),
                                    tuple(n for n, v in zip(("hw_slowdown", "hw_thermal_slowdown",
                                                             "sw_thermal_slowdown", "sw_power_cap"), r[2:6])
                                          if v.lower().startswith("active"))))
            except Exception:
                pass
            time.sleep(0.02)

    def window(self, t0: float, t1: float):
        """Median/min SM clock and the reasons seen between two perf_counter() instants."""
        rows = [r for r in list(self.sm) if t0 <= r[0] <= t1]
        sm = sorted(r[1] for r in rows)
        reasons = sorted({x for r in rows for x in r[2]})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_min_mhz": sm[0] if sm else None,
                "sm_max_mhz": self.max_mhz, "samples": len(sm), "reasons": reasons}

    def wait_ready(self, timeout: float = 3.0):
        """Blocks until the first sample is in (NVML start-up takes longer than a short timed region)."""
        t0 = time.perf_counter()
        while not self.sm and time.perf_counter() - t0 < timeout:
            time.sleep(0.005)

    def stop(self):
        self.stop_flag = True
        self.join(timeout=6)


def gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def build_workload_shape(torch, seq_len, batch, layers, seed):
    """build_workload without the module-level shape overrides (every sequence seq_len keys long)."""
    global RAGGED
    keep, RAGGED = RAGGED, False
    try:
        return build_workload(torch, seq_len, batch, layers, seed)
    finally:
        RAGGED = keep


def build_workload(torch, seq_len: int, batch: int, layers: int, seed: int):
    """Per layer: one K and one V slab [batch][seq_len][4][128] f16 ~N(0,1) (each sequence its
    own contiguous region, addressed through pointer tables), the step's q/k/v/gate ~N(0,1),
    norm weights ~1+N(0,0.02), RoPE theta 1e6 at position seq_len-1."""
    import numpy as np
    from oxide_infer_b200 import rotary_tables
    g = torch.Generator(device="cuda").manual_seed(seed)
    dev = "cuda"
    w = type("W", (), {})()
    w.batch, w.layers, w.seq_len = batch, layers, seq_len
    w.k_slab, w.v_slab, w.k_ptrs, w.v_ptrs = [], [], [], []
    stride = seq_len * ROW_BYTES
    for _ in range(layers):
        k = torch.empty(batch, seq_len, NKV, HD, dtype=torch.float16, device=dev).normal_(generator=g)
        v = torch.empty(batch, seq_len, NKV, HD, dtype=torch.float16, device=dev).normal_(generator=g)
        w.k_slab.append(k)
        w.v_slab.append(v)
        w.k_ptrs.append(torch.tensor([k.data_ptr() + i * stride for i in range(batch)], dtype=torch.int64, device=dev))
        w.v_ptrs.append(torch.tensor([v.data_ptr() + i * stride for i in range(batch)], dtype=torch.int64, device=dev))
    rn = lambda *s: torch.empty(*s, dtype=torch.float16, device=dev).normal_(generator=g)
    w.q0 = rn(layers, batch, NQ, HD)
    w.k = rn(layers, batch, NKV, HD)
    w.v = rn(layers, batch, NKV, HD)
    w.gate = rn(layers, batch, NQ)
    w.q = w.q0.clone()
    w.qw = (1 + 0.02 * torch.randn(layers, HD, device=dev, generator=g)).half()
    w.kw = (1 + 0.02 * torch.randn(layers, HD, device=dev, generator=g)).half()
    cos, sin = rotary_tables(seq_len, 1e6, 0.5)
    w.cos, w.sin = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
    if RAGGED:  # configuration 2's ragged variant: old lengths uniform 1024..4096 (seeded), capacity seq_len each
        lens_np = np.minimum(np.random.default_rng(seed).integers(1024, 4097, batch) + 1, seq_len).astype(np.int64)
    else:
        lens_np = np.full(batch, seq_len, np.int64)
    w.pos = torch.from_numpy((lens_np - 1).astype(np.int32)).to(dev)
    w.lens = torch.from_numpy(lens_np.astype(np.int32)).to(dev)
    w.ctx = torch.zeros(layers, batch, NQ, HD, dtype=torch.float16, device=dev)
    w.seq_lens_host = lens_np
    return w


def cpu_baseline(seq_len: int, batch: int, budget_s: float = 12.0):
    """The oracle's decode sequence for ONE layer of the workload on the host cores."""
    import numpy as np
    from oracle import cpu as O
    O.build()
    O.use_all_cores()
    rng = np.random.default_rng(0)
    f16 = lambda *s: rng.standard_normal(s, dtype=np.float32).astype(np.float16)
    b = batch
    kc = [f16(seq_len, NKV, HD) for _ in range(b)]
    vc = [f16(seq_len, NKV, HD) for _ in range(b)]
    q, k, v, gate = f16(b, NQ, HD), f16(b, NKV, HD), f16(b, NKV, HD), f16(b, NQ)
    w = np.ones(HD, np.float16)
    cos, sin = O.rope_table(seq_len)
    pos = np.full(b, seq_len - 1, np.uint32)
    kp, vp = O.ptr_table(kc), O.ptr_table(vc)
    reps, t0 = 0, time.perf_counter()
    while True:
        O.decode_layer(q.copy(), k.copy(), v, gate, w, w, cos, sin, pos, pos + 1, kp, vp)
        reps += 1
        dt = time.perf_counter() - t0
        if dt > budget_s or reps >= 20:
            break
    gbs = alg_bytes_layer([seq_len] * b) * reps / dt / 1e9
    return {"value": round(gbs, 3), "unit": "GB/s", "cores": O.num_threads(), "kind": "port",
            "sample": f"1 of {LAYERS} layers (append + split/combine + gate), B={b}, ctx={seq_len}, "
                      f"{reps} reps in {dt:.1f} s"}


def _graph_of(torch, fn, warm=1):
    """Captures fn() (already warmed up by the caller) into a CUDA graph on a side stream."""
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    return graph


def _timed_region(torch, fn, steps, barrier):
    """K calls of fn() between two events on the current stream, a barrier + synchronize on both sides."""
    stream = torch.cuda.current_stream()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record(stream)
    for _ in range(steps):
        fn()
    t1.record(stream)
    barrier()
    return t0.elapsed_time(t1)


def read_only_peak(torch, kv, bufs, reps=8):
    """GB/s of the library's read-only stream probe (the decode kernel's bulk-copy pipeline without
    arithmetic): one launch per buffer of `bufs` (each as large as the K + V bytes one decode launch reads, far larger than L2),
    replayed as a CUDA graph like the headline step, with the decode kernel's 4 KB copies and with
    32 KB copies."""
    out = {}
    for name, cb in (("copy_4k", 4096), ("copy_32k", 32768)):
        def launches():
            for b in bufs:
                kv.stream_read(b, cb)
        launches()
        graph = _graph_of(torch, launches)
        graph.replay()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(reps):
            graph.replay()
        t1.record()
        torch.cuda.synchronize()
        nbytes = reps * sum(b.numel() * b.element_size() for b in bufs)
        out[name] = round(nbytes / (t0.elapsed_time(t1) * 1e-3) / 1e9, 1)
    return out


def run_ours(args, torch, rank, world, local_rank):
    from oxide_infer_b200 import KvPath
    kv = KvPath(local_rank, max_batch=BATCH, max_seq_len=CTX, max_prefill_rows=16)
    w = build_workload(torch, CTX, BATCH, LAYERS, seed=1234 + rank)
    stream = torch.cuda.current_stream()

    def step(events=None):
        # one fused launch pair per layer: decode_attn_kernel<fused> (RMSNorm + RoPE + KV append +
        # split-KV attention) and decode_merge_kernel (merge + gate); q is read-only
        for l in range(LAYERS):
            if events is not None:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
            kv.append_decode(w.ctx[l], w.q0[l], w.k[l], w.v[l], w.gate[l], w.qw[l], w.kw[l], w.cos, w.sin, w.pos,
                             w.lens, w.k_ptrs[l], w.v_ptrs[l])
            if events is not None:
                e1.record(stream)
                events.append((e0, e1))

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(gpu_index(local_rank))
    sampler.start()
    sampler.wait_ready()
    for _ in range(args.warmup):
        step()
    ev = []
    w0 = time.perf_counter()
    ms = _timed_region(torch, lambda: step(ev), args.steps, barrier)
    w1 = time.perf_counter()
    pair_ms_stream = sum(a.elapsed_time(b) for a, b in ev) / len(ev)

    # the same K steps as replays of ONE captured 8-layer step (what an engine that captures its
    # decode step sees): identical kernels and work, no host launch gaps; timed like the stream run
    ms_graph = float("inf")
    graph = graph_h = None
    try:
        graph = _graph_of(torch, step)
        for _ in range(3):
            graph.replay()
        ms_graph = _timed_region(torch, graph.replay, args.steps, barrier)
    except Exception as exc:  # every rank must take the same path below
        if rank == 0:
            print(f"cuda graph capture failed: {exc}", file=sys.stderr)
    clocks = sampler.window(w0, time.perf_counter())  # both timed regions of the headline
    if args.no_e2e:
        sampler.stop()
        if rank == 0:
            attn_gbs = alg_bytes_layer(w.seq_lens_host) / (pair_ms_stream * 1e-3) / 1e9
            return {"profiling_case": True, "layers": LAYERS, "batch": BATCH, "ctx": CTX,
                    "ms_per_step": round(ms / args.steps, 4), "decode_attn_us": round(pair_ms_stream * 1e3, 2),
                    "decode_attn_gbs": round(attn_gbs, 1), "clocks": clocks}
        return None

    # ---- end to end through the host-buffer entry
    pin = lambda t: t.cpu().pin_memory()
    hq, hk, hv, hg = pin(w.q0), pin(w.k), pin(w.v), pin(w.gate)
    hctx = torch.zeros(LAYERS, BATCH, NQ, HD, dtype=torch.float16).pin_memory()
    hpos = pin(w.pos)
    hkp, hvp = pin(torch.stack(w.k_ptrs)), pin(torch.stack(w.v_ptrs))
    h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv, hg, hkp, hvp)) + hpos.numel() * 4
    d2h = hctx.numel() * 2

    def step_host():
        kv.decode_step_host(hctx, hq, hk, hv, hg, w.qw, w.kw, w.cos, w.sin, hpos, hkp, hvp, BATCH, LAYERS)

    # host-to-device bandwidth of this box (pinned memory), for context: boxes of one pool differ by more than 2x
    pcie_src = torch.empty(64 << 20, dtype=torch.uint8).pin_memory()
    pcie_dst = torch.empty(64 << 20, dtype=torch.uint8, device="cuda")
    pcie_dst.copy_(pcie_src, non_blocking=True)
    torch.cuda.synchronize()
    pe0, pe1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    pe0.record()
    for _ in range(4):
        pcie_dst.copy_(pcie_src, non_blocking=True)
    pe1.record()
    torch.cuda.synchronize()
    h2d_gbs = 4 * (64 << 20) / (pe0.elapsed_time(pe1) * 1e-3) / 1e9
    del pcie_src, pcie_dst

    for _ in range(max(3, args.warmup)):
        step_host()
    ms_e2e = _timed_region(torch, step_host, args.steps, barrier)
    e2e_mode = "stream launches"
    ms_e2e_graph = float("inf")
    try:  # the same host-buffer step captured once (copies from the same pinned buffers included) and replayed
        graph_h = _graph_of(torch, step_host)
        for _ in range(3):
            graph_h.replay()
        ms_e2e_graph = _timed_region(torch, graph_h.replay, args.steps, barrier)
    except Exception as exc:
        if rank == 0:
            print(f"cuda graph capture of the host-buffer step failed: {exc}", file=sys.stderr)
    step()  # untimed: same inputs as the host-buffer path, for the equality check
    status = kv.device_status()
    ctx_ok = bool(torch.isfinite(w.ctx.float()).all().item()) and bool(torch.isfinite(hctx.float()).all().item())
    same = bool((hctx.cuda() == w.ctx).all().item())
    # two buffers of one decode launch's K + V bytes each (1.07 GB at the default shape), read alternately
    probe_bytes = int(BATCH) * int(CTX) * 2 * ROW_BYTES
    probe_bufs = [torch.empty(probe_bytes, dtype=torch.uint8, device="cuda").zero_() for _ in range(2)]
    ro_peak = read_only_peak(torch, kv, probe_bufs)
    del probe_bufs
    status |= kv.device_status()
    layer_bytes = alg_bytes_layer(w.seq_lens_host)

    # ---- the other configurations, every rank on its own GPU (rank 0 reports); config 5 is partitioned
    secondary = {}
    if not args.no_secondary:
        secondary["decode_ragged"] = leg_decode_ragged(args, torch, "ours", w, kv)
        if (LAYERS, BATCH, CTX) == (8, 128, 4096):
            secondary["decode_paged"] = leg_decode_paged(args, torch, w, kv)
        del w, graph, graph_h
        kv.close()
        torch.cuda.empty_cache()
        # the tensor-bound legs before the long streaming leg: right after half a minute of HBM streaming the same wave
        # measured 7 % slower (0.66 instead of 0.71 of the tensor peak)
        secondary["prefill"] = leg_prefill(args, torch, "ours")
        secondary["project_append"] = leg_project_append(args, torch, "ours")
        secondary["layer_step"] = leg_layer_step(args, torch, "ours")
        torch.cuda.empty_cache()
        secondary["decode_small"] = leg_decode_small(args, torch, "ours")
        secondary["conv"] = leg_conv(args, torch, "ours")
        secondary["sample"] = leg_sample(args, torch)
        torch.cuda.empty_cache()
        secondary["serving_mix"] = leg_serving_mix(args, torch, "ours", rank, world, local_rank)
        torch.cuda.empty_cache()
    sampler.stop()

    times = torch.tensor([ms, ms_e2e, pair_ms_stream, ms_graph, ms_e2e_graph], dtype=torch.float64, device="cuda")
    if world > 1:
        torch.distributed.all_reduce(times, op=torch.distributed.ReduceOp.MAX)
    ms, ms_e2e, pair_ms_stream, ms_graph, ms_e2e_graph = (float(x) for x in times.tolist())
    ms_e2e_stream = ms_e2e
    if ms_e2e_graph < ms_e2e:
        ms_e2e, e2e_mode = ms_e2e_graph, "cuda graph replay of the captured host-buffer step"
    if rank != 0:
        return None

    step_bytes = LAYERS * layer_bytes * world
    peak, peak_kind = measured_peak_gbs()
    ms_stream = ms  # K steps launched one call at a time on the stream
    launch_mode = "stream launches (one C-ABI call per layer)"
    if ms_graph < ms:
        ms = ms_graph
        launch_mode = "cuda graph replay of the captured 8-layer step"
    # the dominant kernel pair (fused decode_attn_kernel + decode_merge_kernel) is the whole timed region:
    # its average duration in the SAME launch mode as `value` is region time / launches
    pair_us = ms / args.steps / LAYERS * 1e3
    attn_gbs = layer_bytes / (pair_us * 1e-6) / 1e9
    line = {
        "metric": "gqa_decode_step_hbm_gbs", "value": round(step_bytes * args.steps / (ms * 1e-3) / 1e9, 1),
        "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms / args.steps, 4), "us_per_layer": round(ms / args.steps / LAYERS * 1e3, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": f"decode_step_{LAYERS}_attention_layers_B{BATCH}_per_gpu_ctx{CTX}" +
                               ("_ragged_lengths_uniform_1024_4096" if RAGGED else ""),
                   "layers": LAYERS, "batch_per_gpu": BATCH, "seq_len": CTX},
        "notes": {"heads": "16q/4kv x128", "kv_bytes_per_gpu": int(LAYERS * BATCH * CTX * 2 * ROW_BYTES),
                  "l2": "inputs larger than L2 (1.07 GB of KV per layer, 8 distinct layers)",
                  "launch": launch_mode,
                  "parallelism": f"replicas x{world}, sequences partitioned, no collective"},
        "e2e": {"value": round(step_bytes * args.steps / (ms_e2e * 1e-3) / 1e9, 1), "unit": "GB/s",
                "ms_per_step": round(ms_e2e / args.steps, 4), "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h), "launch": e2e_mode, "h2d_gbs_of_this_box": round(h2d_gbs, 1),
                "stream_launch_ms_per_step": round(ms_e2e_stream / args.steps, 4),
                "cuda_graph_replay_ms_per_step": round(ms_e2e_graph / args.steps, 4) if ms_e2e_graph != float("inf") else None},
        "gpu_launches": 2 * LAYERS * args.steps,  # fused append+decode_attn, decode_merge per layer
        "roofline": {"kernel": "decode_attn_kernel<fused append> + decode_merge_kernel", "bound": "hbm",
                     "achieved": round(attn_gbs, 1), "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                     "frac": round(attn_gbs / peak, 4), "frac_of_8TBs_nominal": round(attn_gbs / 8000.0, 4),
                     "us_per_launch": round(pair_us, 2),
                     "us_per_launch_mode": launch_mode + ": timed region / (steps x layers), one kernel pair per layer",
                     "us_per_launch_stream_events": round(pair_ms_stream * 1e3, 2),
                     "read_only_peak": ro_peak["copy_32k"], "read_only_peak_4k_copies": ro_peak["copy_4k"],
                     "frac_of_read_only_peak": round(attn_gbs / ro_peak["copy_32k"], 4),
                     "read_only_peak_kind": "measured in this run: the decode kernel's bulk-copy ring without arithmetic "
                                            "(oxi_debug_stream_read), one launch per buffer of a decode launch's K + V bytes, graph replay, 32 KB copies; "
                                            "the decode kernel copies 4 KB",
                     # the ncu capture was taken at the default sizes only
                     "traffic": TRAFFIC_PER_LAUNCH if (not RAGGED and (LAYERS, BATCH, CTX) == (8, 128, 4096)) else None,
                     "traffic_source": "constant: dram bytes read + written of one launch from the ncu capture summarised in "
                                       "profiles/decode_attn_kernel_B128_ctx4096.md, not measured in this run"},
        "clocks": clocks, "device_status": status, "finite": ctx_ok, "e2e_equals_device_path": same,
        "cuda_graph_replay_ms_per_step": round(ms_graph / args.steps, 4) if ms_graph != float("inf") else None,
        "stream_launch_ms_per_step": round(ms_stream / args.steps, 4),
    }
    if secondary:
        line["secondary"] = secondary
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(CTX, BATCH)
    return line


# dram__bytes_read.sum + dram__bytes_write.sum of one decode_attn_kernel launch at the bench
# workload, from the ncu capture summarised in profiles/decode_attn_kernel_B128_ctx4096.md
TRAFFIC_PER_LAUNCH = 1074318000 + 3661568


def run_reference(args, torch, rank, world, local_rank):
    """The reference's kernels on one B200 (rank 0 only), engine launch order, 9 per layer."""
    if rank != 0:
        return None
    from oracle import refptx
    cfg = {"workload": f"decode_step_{LAYERS}_attention_layers_B{BATCH}_per_gpu_ctx{CTX}", "layers": LAYERS,
           "batch_per_gpu": BATCH, "seq_len": CTX}
    if not refptx.available():
        cb = cpu_baseline(CTX, BATCH)
        return {"impl": "reference", "metric": "gqa_decode_step_hbm_gbs", "value": cb["value"], "unit": "GB/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True,
                "scaling": "weak", "dtype": "f16", "data": "synthetic", "config": cfg,
                "notes": {"what": "reference cubins absent: CPU oracle port timed instead"},
                "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    ref = refptx.RefPtx()
    w = build_workload(torch, CTX, BATCH, LAYERS, seed=1234)
    nch = ref.nchunks_for(CTX, 0)
    acc = torch.empty(BATCH * nch * NQ * HD, dtype=torch.float32, device="cuda")
    stats = torch.empty(BATCH * nch * NQ * 2, dtype=torch.float32, device="cuda")
    kbuf = w.k.clone()

    def step():
        for l in range(LAYERS):  # q and k are normalised in place; the timed steps re-normalise them
            ref.append(w.q[l], kbuf[l], w.v[l], w.qw[l], w.kw[l], w.cos, w.sin, w.pos, w.k_ptrs[l], w.v_ptrs[l], BATCH)
            ref.decode_attention(w.ctx[l], w.q[l], w.gate[l], w.k_ptrs[l], w.v_ptrs[l], w.lens, BATCH, 0, CTX, acc, stats)

    barrier = torch.cuda.synchronize
    sampler = ClockSampler(gpu_index(local_rank))
    sampler.start()
    sampler.wait_ready()
    for _ in range(args.warmup):
        step()
    w0 = time.perf_counter()
    ms_stream = _timed_region(torch, step, args.steps, barrier)
    w1 = time.perf_counter()
    clocks = sampler.window(w0, w1)
    # the same 72-launch step captured once and replayed, like our arm's graph mode
    ms_graph = float("inf")
    try:
        graph = _graph_of(torch, step)
        for _ in range(3):
            graph.replay()
        ms_graph = _timed_region(torch, graph.replay, args.steps, barrier)
    except Exception as exc:
        print(f"cuda graph capture of the reference step failed: {exc}", file=sys.stderr)
    ms = min(ms_stream, ms_graph)
    launch_mode = "cuda graph replay of the captured 72-launch step" if ms_graph < ms_stream else "stream launches"

    # end to end with the same host traffic as our arm: upload q/k/v/gate + tables, download ctx
    pin = lambda t: t.cpu().pin_memory()
    hq, hk, hv, hg = pin(w.q0), pin(w.k), pin(w.v), pin(w.gate)
    hkp, hvp = pin(torch.stack(w.k_ptrs)), pin(torch.stack(w.v_ptrs))
    hctx = torch.zeros(LAYERS, BATCH, NQ, HD, dtype=torch.float16).pin_memory()
    dkp, dvp = torch.stack(w.k_ptrs).clone(), torch.stack(w.v_ptrs).clone()

    def step_host():
        for l in range(LAYERS):
            w.q[l].copy_(hq[l], non_blocking=True)
            kbuf[l].copy_(hk[l], non_blocking=True)
            w.v[l].copy_(hv[l], non_blocking=True)
            w.gate[l].copy_(hg[l], non_blocking=True)
            dkp[l].copy_(hkp[l], non_blocking=True)
            dvp[l].copy_(hvp[l], non_blocking=True)
            ref.append(w.q[l], kbuf[l], w.v[l], w.qw[l], w.kw[l], w.cos, w.sin, w.pos, dkp[l], dvp[l], BATCH)
            ref.decode_attention(w.ctx[l], w.q[l], w.gate[l], dkp[l], dvp[l], w.lens, BATCH, 0, CTX, acc, stats)
            hctx[l].copy_(w.ctx[l], non_blocking=True)

    for _ in range(3):
        step_host()
    ms_e2e_stream = _timed_region(torch, step_host, args.steps, barrier)
    ms_e2e_graph = float("inf")
    try:
        graph_h = _graph_of(torch, step_host)
        for _ in range(3):
            graph_h.replay()
        ms_e2e_graph = _timed_region(torch, graph_h.replay, args.steps, barrier)
    except Exception as exc:
        print(f"cuda graph capture of the reference host-buffer step failed: {exc}", file=sys.stderr)
    ms_e2e = min(ms_e2e_stream, ms_e2e_graph)
    h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv, hg, hkp, hvp))
    step_bytes = LAYERS * alg_bytes_layer(w.seq_lens_host)

    secondary = {}
    if not args.no_secondary:
        secondary["decode_ragged"] = leg_decode_ragged(args, torch, "reference", w, ref)
        del w, acc, stats, kbuf
        torch.cuda.empty_cache()
        secondary["prefill"] = leg_prefill(args, torch, "reference")
        secondary["project_append"] = leg_project_append(args, torch, "reference")
        secondary["layer_step"] = leg_layer_step(args, torch, "reference")
        torch.cuda.empty_cache()
        secondary["decode_small"] = leg_decode_small(args, torch, "reference")
        secondary["conv"] = leg_conv(args, torch, "reference")
        torch.cuda.empty_cache()
        secondary["serving_mix"] = leg_serving_mix(args, torch, "reference", 0, 1, local_rank)
    sampler.stop()
    line = {
        "impl": "reference", "metric": "gqa_decode_step_hbm_gbs",
        "value": round(step_bytes * args.steps / (ms * 1e-3) / 1e9, 1), "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 4),
        "us_per_layer": round(ms / args.steps / LAYERS * 1e3, 2), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": cfg,
        "notes": {"what": "reference PTX kernels (sm_80 text assembled for sm_100a) on one B200, "
                          "engine launch sequence: 2 norm, 2 rope, 2 copy, split4, combine, gate",
                  "launch": launch_mode,
                  "parallelism": "single GPU (the reference has no multi-GPU path)"},
        "stream_launch_ms_per_step": round(ms_stream / args.steps, 4),
        "cuda_graph_replay_ms_per_step": round(ms_graph / args.steps, 4) if ms_graph != float("inf") else None,
        "e2e": {"value": round(step_bytes * args.steps / (ms_e2e * 1e-3) / 1e9, 1), "unit": "GB/s",
                "ms_per_step": round(ms_e2e / args.steps, 4), "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(hctx.numel() * 2),
                "stream_launch_ms_per_step": round(ms_e2e_stream / args.steps, 4),
                "cuda_graph_replay_ms_per_step": round(ms_e2e_graph / args.steps, 4) if ms_e2e_graph != float("inf") else None},
        "gpu_launches": 9 * LAYERS * args.steps, "clocks": clocks,
    }
    if secondary:
        line["secondary"] = secondary
    if not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(CTX, BATCH)
    return line


# ---------------------------------------------------------------------------
# The other configurations as short legs of the default run (key "secondary" of the line).  impl =
# "ours" runs this library, impl = "reference" (only under --impl reference) the reference's kernels.

def _tensor_peak():
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        try:
            return float(json.load(open(pk))["bf16_tflops_sustained"]), "measured"
        except Exception:
            pass
    return 1400.0, "fallback"


def leg_decode_ragged(args, torch, impl, w, eng):
    """Configuration 2's lengths: old context uniform 1024..4096 (seeded) on the headline's caches."""
    import numpy as np
    lens_np = np.minimum(np.random.default_rng(2).integers(1024, 4097, BATCH) + 1, CTX).astype(np.int64)
    pos = torch.from_numpy((lens_np - 1).astype(np.int32)).cuda()
    lens = torch.from_numpy(lens_np.astype(np.int32)).cuda()
    if impl == "ours":
        def step():
            for l in range(LAYERS):
                eng.append_decode(w.ctx[l], w.q0[l], w.k[l], w.v[l], w.gate[l], w.qw[l], w.kw[l], w.cos, w.sin, pos, lens,
                                  w.k_ptrs[l], w.v_ptrs[l])
    else:
        nch = eng.nchunks_for(CTX, 0)
        acc = torch.empty(BATCH * nch * NQ * HD, dtype=torch.float32, device="cuda")
        stats = torch.empty(BATCH * nch * NQ * 2, dtype=torch.float32, device="cuda")
        kb = w.k.clone()

        def step():
            for l in range(LAYERS):
                eng.append(w.q[l], kb[l], w.v[l], w.qw[l], w.kw[l], w.cos, w.sin, pos, w.k_ptrs[l], w.v_ptrs[l], BATCH)
                eng.decode_attention(w.ctx[l], w.q[l], w.gate[l], w.k_ptrs[l], w.v_ptrs[l], lens, BATCH, 0, CTX, acc, stats)
    for _ in range(3):
        step()
    graph = _graph_of(torch, step)
    ms = _time_loop(torch, graph.replay, args.steps, 3)
    step_bytes = LAYERS * alg_bytes_layer(lens_np)
    peak, kind = measured_peak_gbs()
    gbs = step_bytes / (ms * 1e-3) / 1e9
    return {"workload": f"decode_step_{LAYERS}_layers_B{BATCH}_ctx_uniform_1024_4096", "ms_per_step": round(ms, 4),
            "us_per_layer": round(ms / LAYERS * 1e3, 2), "gbs": round(gbs, 1), "frac": round(gbs / peak, 4),
            "peak": peak, "peak_kind": kind, "launch": "cuda graph replay", "mean_keys": float(lens_np.mean())}


def leg_decode_small(args, torch, impl):
    """Small and skewed decode shapes, one layer step, CUDA-graph replay in both arms (like for like): 8 sequences of 512 keys
    (launch / latency bound) and one sequence of 32,768 keys (128 work items, one per SM)."""
    out = {}
    for name, batch, ctx in (("B8_ctx512", 8, 512), ("B1_ctx32768", 1, 32768)):
        w = build_workload_shape(torch, ctx, batch, 4, seed=77)
        if impl == "ours":
            from oxide_infer_b200 import KvPath
            kv = KvPath(torch.cuda.current_device(), max_batch=batch, max_seq_len=ctx, max_prefill_rows=0)

            def step():
                for l in range(4):
                    kv.append_decode(w.ctx[l], w.q0[l], w.k[l], w.v[l], w.gate[l], w.qw[l], w.kw[l], w.cos, w.sin, w.pos, w.lens,
                                     w.k_ptrs[l], w.v_ptrs[l])
        else:
            from oracle import refptx
            ref = refptx.RefPtx()
            nch = ref.nchunks_for(ctx, 0)
            acc = torch.empty(batch * nch * NQ * HD, dtype=torch.float32, device="cuda")
            stats = torch.empty(batch * nch * NQ * 2, dtype=torch.float32, device="cuda")
            kb = w.k.clone()

            def step():
                for l in range(4):
                    ref.append(w.q[l], kb[l], w.v[l], w.qw[l], w.kw[l], w.cos, w.sin, w.pos, w.k_ptrs[l], w.v_ptrs[l], batch)
                    ref.decode_attention(w.ctx[l], w.q[l], w.gate[l], w.k_ptrs[l], w.v_ptrs[l], w.lens, batch, 0, ctx, acc, stats)
        for _ in range(3):
            step()
        graph = _graph_of(torch, step)
        ms = _time_loop(torch, graph.replay, max(args.steps, 50), 3) / 4
        byts = batch * (2 * ROW_BYTES * ctx + PER_SEQ_FIXED)
        out[name] = {"us_per_layer": round(ms * 1e3, 2), "gbs": round(byts / (ms * 1e-3) / 1e9, 1)}
        if impl == "ours":
            out[name]["device_status"] = kv.device_status()
            kv.close()
    out["launch"] = "cuda graph replay of 4 layers (4 distinct caches)"
    return out


def leg_decode_paged(args, torch, w, kv):
    """The headline step over a paged layout: the same slabs seen as pools of 16-token blocks, every
    sequence's pages scattered over the pool by a seeded permutation (CUDA-graph replay)."""
    import numpy as np
    from oxide_infer_b200 import PagedLayout
    bs = 16
    per_seq = CTX // bs
    nblk = BATCH * per_seq
    table = torch.from_numpy(np.random.default_rng(7).permutation(nblk).astype(np.int32).reshape(BATCH, per_seq)).cuda()
    lays = [PagedLayout.of(w.k_slab[l].view(nblk, bs, NKV, HD), w.v_slab[l].view(nblk, bs, NKV, HD), table, bs)
            for l in range(LAYERS)]

    def paged():
        for l in range(LAYERS):
            kv.append_decode_paged(w.ctx[l], w.q0[l], w.k[l], w.v[l], w.gate[l], w.qw[l], w.kw[l], w.cos, w.sin,
                                   w.lens, lays[l])
    for _ in range(3):
        paged()
    graph = _graph_of(torch, paged)
    ms = _time_loop(torch, graph.replay, args.steps, 3)
    step_bytes = LAYERS * alg_bytes_layer(w.seq_lens_host)
    peak, kind = measured_peak_gbs()
    gbs = step_bytes / (ms * 1e-3) / 1e9
    return {"workload": "decode_step_8_layers_B128_ctx4096_paged_kv_16_token_blocks", "ms_per_step": round(ms, 4),
            "us_per_layer": round(ms / LAYERS * 1e3, 2), "gbs": round(gbs, 1), "frac": round(gbs / peak, 4),
            "peak": peak, "peak_kind": kind, "launch": "cuda graph replay"}


def leg_prefill(args, torch, impl):
    """Configuration 4: one wave of 128 new tokens for each of 32 sequences, prefixes uniform 0..8192
    (seeded), one attention layer.  ours: append of the 4,096 rows + causal gated attention;
    reference: its non-GEMM path, the online kernel over all rows + the gate kernel
    (batch_engine.rs:1214-1239) - its cuBLASLt path cannot be driven without the engine."""
    import numpy as np
    from oxide_infer_b200 import rotary_tables
    nseq, new = 32, 128
    rows = nseq * new
    prefix = np.random.default_rng(4).integers(0, 8193, nseq)
    g = torch.Generator(device="cuda").manual_seed(4)
    rn = lambda *s: torch.empty(*s, dtype=torch.float16, device="cuda").normal_(generator=g)
    cap = [int(p) + new for p in prefix]
    slab = rn(2 * sum(cap), NKV, HD)
    offs = np.concatenate([[0], np.cumsum(cap)])
    kc = [slab[offs[i]:offs[i + 1]] for i in range(nseq)]
    vc = [slab[sum(cap) + offs[i]:sum(cap) + offs[i + 1]] for i in range(nseq)]
    q, k, v, gate = rn(rows, NQ, HD), rn(rows, NKV, HD), rn(rows, NKV, HD), rn(rows, NQ)
    qw = (1 + 0.02 * torch.randn(HD, device="cuda", generator=g)).half()
    kw = (1 + 0.02 * torch.randn(HD, device="cuda", generator=g)).half()
    cos, sin = rotary_tables(8192 + new, 1e6, 0.5)
    cos, sin = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
    owner = np.repeat(np.arange(nseq), new)
    pos = (prefix[owner] + np.tile(np.arange(new), nseq)).astype(np.int32)
    kp = torch.tensor([kc[i].data_ptr() for i in owner], dtype=torch.int64, device="cuda")
    vp = torch.tensor([vc[i].data_ptr() for i in owner], dtype=torch.int64, device="cuda")
    dpos, dlen = torch.from_numpy(pos).cuda(), torch.from_numpy(pos + 1).cuda()
    ctx = torch.zeros(rows, NQ, HD, dtype=torch.float16, device="cuda")
    flops = float(sum(8192 * (128 * int(p) + 8256) for p in prefix))
    peak_tf, kind = _tensor_peak()
    out = {"workload": "prefill_wave_32seq_x128tok_prefix_U0_8192_one_layer", "rows": rows, "causal_exact_gflop": round(flops / 1e9, 1)}
    if impl == "ours":
        from oxide_infer_b200 import KvPath
        kv = KvPath(torch.cuda.current_device(), max_batch=128, max_seq_len=8192 + new, max_prefill_rows=rows)
        ms_attn = _time_loop(torch, lambda: kv.prefill_attn(ctx, q, gate, kp, vp, dlen, 0), args.steps, 3)

        def wave():
            kv.append(q, k, v, qw, kw, cos, sin, dpos, kp, vp, batch=rows)
            kv.prefill_attn(ctx, q, gate, kp, vp, dlen, 0)
        ms_wave = _time_loop(torch, wave, args.steps, 3)
        tf = flops / (ms_attn * 1e-3) / 1e12
        out.update({"ms_attention": round(ms_attn, 4), "ms_append_plus_attention": round(ms_wave, 4), "tflops": round(tf, 1),
                    "frac": round(tf / peak_tf, 4), "peak": peak_tf, "peak_kind": kind + " (sustained bf16 GEMM)",
                    "bound": "tensor", "device_status": kv.device_status()})
        kv.close()
    else:
        from oracle import refptx
        ref = refptx.RefPtx()

        def ref_attn():
            ref.attn_online(ctx, q, kp, vp, dlen, rows, 0)
            ref.sigmoid_gate(ctx, gate, rows)
        ms = _time_loop(torch, ref_attn, 3, 3)
        out.update({"ms_attention": round(ms, 4), "tflops": round(flops / (ms * 1e-3) / 1e12, 2),
                    "what": "online kernel over all wave rows + gate kernel"})
    return out


def leg_conv(args, torch, impl):
    """Configuration 3: 16 conv layers, batch 128, one decode update per layer (CUDA-graph replay of the
    16 launches), and configuration 4's wave (32 x 128 rows) through one conv layer."""
    import numpy as np
    nl, b, hid = 16, 128, 2048
    g = torch.Generator(device="cuda").manual_seed(3)
    rn = lambda *s, sc=1.0: (torch.randn(*s, device="cuda", generator=g) * sc).half()
    state, bcx, w = rn(nl, b, hid, 6), rn(nl, b, 3 * hid), rn(nl, hid, 7, sc=0.1)
    y = torch.zeros(nl, b, hid, dtype=torch.float16, device="cuda")
    ptrs = torch.tensor([[state[l, i].data_ptr() for i in range(b)] for l in range(nl)], dtype=torch.int64, device="cuda")
    nseq, new = 32, 128
    rows = nseq * new
    carry, pbcx = rn(nseq, hid, 6), rn(rows, 3 * hid)
    py = torch.zeros(rows, hid, dtype=torch.float16, device="cuda")
    origin = torch.from_numpy(np.repeat(np.arange(nseq) * new, new).astype(np.int32)).cuda()
    lpos = torch.from_numpy(np.tile(np.arange(new), nseq).astype(np.int32)).cuda()
    cptr = torch.tensor([carry[i // new].data_ptr() for i in range(rows)], dtype=torch.int64, device="cuda")
    step_bytes = nl * (b * 65536 + 28672)
    pf_bytes = nseq * (16384 * new + 49152)
    peak, kind = measured_peak_gbs()
    out = {"workload": "conv_decode_16_layers_B128_2048ch_K7"}
    if impl == "ours":
        from oxide_infer_b200 import KvPath
        kv = KvPath(torch.cuda.current_device(), max_batch=b, max_seq_len=4096, max_prefill_rows=rows)

        def dec():
            for l in range(nl):
                kv.conv_decode(y[l], ptrs[l], bcx[l], w[l])
        pf = lambda: kv.conv_prefill(py, cptr, origin, lpos, pbcx, w[0])
    else:
        from oracle import refptx
        ref = refptx.RefPtx()
        pool = torch.zeros(rows, hid, 6, dtype=torch.float16, device="cuda")
        pool_ptrs = torch.tensor([pool.data_ptr() + r * hid * 12 for r in range(rows)], dtype=torch.int64, device="cuda")

        def dec():
            for l in range(nl):
                ref.conv_decode(y[l], ptrs[l], bcx[l], w[l], b)

        def pf():  # batch_engine.rs:847-899 on the device; the per-chunk copy-back (server.rs:1192-1224) as 32 device copies
            ref.conv_state_prefill(pool, cptr, origin, lpos, pbcx, rows)
            ref.conv_decode(py, pool_ptrs, pbcx, w[0], rows)
            for i in range(nseq):
                carry[i].copy_(pool[(i + 1) * new - 1])
    for _ in range(3):
        dec()
    graph = _graph_of(torch, dec)
    ms = _time_loop(torch, graph.replay, max(args.steps, 50), 3)
    for _ in range(3):
        pf()
    graph_pf = _graph_of(torch, pf)
    ms_pf = _time_loop(torch, graph_pf.replay, max(args.steps, 20), 3)
    gbs = step_bytes / (ms * 1e-3) / 1e9
    out.update({"us_per_layer": round(ms / nl * 1e3, 2), "gbs": round(gbs, 1), "frac": round(gbs / peak, 4), "peak": peak,
                "peak_kind": kind, "launch": "cuda graph replay of the 16 launches",
                "note": "8.4 MB per launch: bound by launch and memory latency, not bandwidth",
                "prefill_wave_one_layer": {"rows": rows, "us": round(ms_pf * 1e3, 2),
                                           "gbs": round(pf_bytes / (ms_pf * 1e-3) / 1e9, 1)}})
    if impl == "ours":
        out["device_status"] = kv.device_status()
        kv.close()
    return out


def leg_project_append(args, torch, impl):
    """The steps in front of the path fused into it: q/k/v/gate projections ([rows][2048] x [2048][3088]) with
    RMSNorm + RoPE + KV append as the GEMM's epilogue, at the decode shape (128 rows) and at configuration 4's
    wave (4,096 rows).  ours: oxi_project_append (one kernel).  reference: four library GEMMs (torch.matmul
    standing in for the engine's cuBLASLt calls, batch_engine.rs:914-926) + its six append kernels."""
    import numpy as np
    from oxide_infer_b200 import rotary_tables
    hid, nout = 2048, 3088
    g = torch.Generator(device="cuda").manual_seed(8)
    rn = lambda *s, sc=1.0: (torch.randn(*s, device="cuda", generator=g) * sc).half()
    ws = [rn(o, hid, sc=hid ** -0.5) for o in (2048, 512, 512, 16)]
    qw = (1 + 0.02 * torch.randn(HD, device="cuda", generator=g)).half()
    kw = (1 + 0.02 * torch.randn(HD, device="cuda", generator=g)).half()
    cos, sin = rotary_tables(4096 + 256, 1e6, 0.5)
    cos, sin = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
    peak_tf, kind = _tensor_peak()
    peak_gbs, kind_g = measured_peak_gbs()
    out = {"workload": "qkvg_projection_plus_append_rows128_and_rows4096"}
    if impl == "ours":
        from oxide_infer_b200 import KvPath, Linear
        kv = KvPath(torch.cuda.current_device(), max_batch=128, max_seq_len=8192, max_prefill_rows=4096)
        lin = Linear(*ws)
    else:
        from oracle import refptx
        ref = refptx.RefPtx()
    for rows, nseq in ((128, 128), (4096, 32)):
        new = rows // nseq
        cache_k = torch.zeros(nseq, 4096 + new, NKV, HD, dtype=torch.float16, device="cuda")
        cache_v = torch.zeros_like(cache_k)
        owner = np.repeat(np.arange(nseq), new)
        pos = torch.from_numpy((4000 + np.tile(np.arange(new), nseq)).astype(np.int32)).cuda()
        kp = torch.tensor([cache_k[i].data_ptr() for i in owner], dtype=torch.int64, device="cuda")
        vp = torch.tensor([cache_v[i].data_ptr() for i in owner], dtype=torch.int64, device="cuda")
        xs = [rn(rows, hid) for _ in range(4)]   # rotate inputs; the 12.6 MB of weights stay in L2, as in a real layer loop they do not
        q_out = torch.zeros(rows, NQ, HD, dtype=torch.float16, device="cuda")
        gate_out = torch.zeros(rows, NQ, dtype=torch.float16, device="cuda")
        if impl == "ours":
            def fn():
                for x in xs:
                    kv.project_append(lin, x, q_out, gate_out, qw, kw, cos, sin, pos, kp, vp, rows=rows)
        else:
            k_out = torch.zeros(rows, NKV, HD, dtype=torch.float16, device="cuda")
            v_out = torch.zeros(rows, NKV, HD, dtype=torch.float16, device="cuda")

            def fn():
                for x in xs:
                    torch.matmul(x, ws[0].t(), out=q_out.view(rows, 2048))
                    torch.matmul(x, ws[1].t(), out=k_out.view(rows, 512))
                    torch.matmul(x, ws[2].t(), out=v_out.view(rows, 512))
                    torch.matmul(x, ws[3].t(), out=gate_out)
                    ref.append(q_out, k_out, v_out, qw, kw, cos, sin, pos, kp, vp, rows)
        for _ in range(3):
            fn()
        graph = _graph_of(torch, fn)
        ms = _time_loop(torch, graph.replay, max(args.steps, 20), 3) / len(xs)
        flops = 2.0 * rows * hid * nout
        byts = nout * hid * 2 + rows * (hid * 2 + 4096 + 2048 + 32)   # weights, x, q out, K/V rows, gate
        out[f"rows{rows}"] = {"us": round(ms * 1e3, 2), "tflops": round(flops / (ms * 1e-3) / 1e12, 1),
                              "frac_of_tensor_peak": round(flops / (ms * 1e-3) / 1e12 / peak_tf, 4),
                              "gbs": round(byts / (ms * 1e-3) / 1e9, 1), "launches": 1 if impl == "ours" else 10}
        if impl == "ours":
            # context only: ONE library GEMM of the same shape (weights concatenated, no epilogue, no append), i.e. what
            # the vendor's kernel reaches on [rows][2048] x [2048][3088] when the peak was measured on a large square GEMM
            wcat = torch.cat(ws, 0).contiguous()
            y = torch.empty(rows, nout, dtype=torch.float16, device="cuda")

            def lib():
                for x in xs:
                    torch.matmul(x, wcat.t(), out=y)
            for _ in range(3):
                lib()
            lg = _graph_of(torch, lib)
            lms = _time_loop(torch, lg.replay, max(args.steps, 20), 3) / len(xs)
            out[f"rows{rows}"]["library_gemm_same_shape"] = {
                "us": round(lms * 1e3, 2), "frac_of_tensor_peak": round(flops / (lms * 1e-3) / 1e12 / peak_tf, 4),
                "what": "one torch.matmul, no epilogue: context for the fraction above, not a path of this library"}
    out.update({"tensor_peak": peak_tf, "tensor_peak_kind": kind + " (sustained bf16 GEMM)", "launch": "cuda graph replay",
                "bound": "rows128: weight read (12.6 MB) and latency; rows4096: tensor"})
    if impl == "ours":
        out["device_status"] = kv.device_status()
        kv.close()
    return out


def leg_layer_step(args, torch, impl):
    """An attention layer of a decode step from the normed hidden state to the context, 8 layers, batch 128, 4096 keys:
    ours = oxi_project_append + oxi_decode_attn (3 launches per layer); reference = four library GEMMs (torch.matmul for the
    engine's cuBLASLt calls) + its nine kernels (13 launches per layer).  CUDA-graph replay in both arms."""
    layers, batch, ctx_len, hid = 8, 128, 4096, 2048
    w = build_workload_shape(torch, ctx_len, batch, layers, seed=99)
    g = torch.Generator(device="cuda").manual_seed(9)
    rn = lambda *s, sc=1.0: (torch.randn(*s, device="cuda", generator=g) * sc).half()
    ws = [[rn(o, hid, sc=hid ** -0.5) for o in (2048, 512, 512, 16)] for _ in range(layers)]
    x = rn(layers, batch, hid)
    q_out = torch.zeros(batch, NQ, HD, dtype=torch.float16, device="cuda")
    gate_out = torch.zeros(batch, NQ, dtype=torch.float16, device="cuda")
    if impl == "ours":
        from oxide_infer_b200 import KvPath, Linear
        kv = KvPath(torch.cuda.current_device(), max_batch=batch, max_seq_len=ctx_len, max_prefill_rows=0)
        lins = [Linear(*ws[l]) for l in range(layers)]

        def step():
            for l in range(layers):
                kv.project_append(lins[l], x[l], q_out, gate_out, w.qw[l], w.kw[l], w.cos, w.sin, w.pos, w.k_ptrs[l], w.v_ptrs[l])
                kv.decode_attn(w.ctx[l], q_out, gate_out, w.k_ptrs[l], w.v_ptrs[l], w.lens)
        launches = 3
    else:
        from oracle import refptx
        ref = refptx.RefPtx()
        nch = ref.nchunks_for(ctx_len, 0)
        acc = torch.empty(batch * nch * NQ * HD, dtype=torch.float32, device="cuda")
        stats = torch.empty(batch * nch * NQ * 2, dtype=torch.float32, device="cuda")
        k_out = torch.zeros(batch, NKV, HD, dtype=torch.float16, device="cuda")
        v_out = torch.zeros(batch, NKV, HD, dtype=torch.float16, device="cuda")

        def step():
            for l in range(layers):
                torch.matmul(x[l], ws[l][0].t(), out=q_out.view(batch, 2048))
                torch.matmul(x[l], ws[l][1].t(), out=k_out.view(batch, 512))
                torch.matmul(x[l], ws[l][2].t(), out=v_out.view(batch, 512))
                torch.matmul(x[l], ws[l][3].t(), out=gate_out)
                ref.append(q_out, k_out, v_out, w.qw[l], w.kw[l], w.cos, w.sin, w.pos, w.k_ptrs[l], w.v_ptrs[l], batch)
                ref.decode_attention(w.ctx[l], q_out, gate_out, w.k_ptrs[l], w.v_ptrs[l], w.lens, batch, 0, ctx_len, acc, stats)
        launches = 13
    for _ in range(3):
        step()
    graph = _graph_of(torch, step)
    ms = _time_loop(torch, graph.replay, args.steps, 3)
    out = {"workload": "projection_append_attention_8_layers_B128_ctx4096", "ms_per_step": round(ms, 4),
           "us_per_layer": round(ms / layers * 1e3, 2), "launches_per_layer": launches, "launch": "cuda graph replay"}
    if impl == "ours":
        out["device_status"] = kv.device_status()
        kv.close()
    return out


def leg_sample(args, torch):
    """Argmax over 128 x 128,000 f16 logits + the embedding gather of the chosen rows (hidden 2048); eight logits
    buffers (262 MB) rotate; CUDA-graph replay of the eight pairs."""
    from oxide_infer_b200 import KvPath
    b, vocab, hid, nbuf = 128, 128000, 2048, 8
    kv = KvPath(torch.cuda.current_device(), max_batch=b, max_seq_len=256, max_prefill_rows=0)
    g = torch.Generator(device="cuda").manual_seed(6)
    logits = [torch.empty(b, vocab, dtype=torch.float16, device="cuda").normal_(generator=g) for _ in range(nbuf)]
    table = torch.empty(vocab, hid, dtype=torch.float16, device="cuda").normal_(generator=g)
    tok = torch.zeros(nbuf, b, dtype=torch.int32, device="cuda")
    hidden = torch.zeros(b, hid, dtype=torch.float16, device="cuda")

    def pairs():
        for i in range(nbuf):
            kv.argmax(tok[i], logits[i])
            kv.embed_lookup(hidden, table, tok[i])
    for _ in range(3):
        pairs()
    graph = _graph_of(torch, pairs)
    ms = _time_loop(torch, graph.replay, max(args.steps, 50), 3)
    am_bytes = b * vocab * 2 + b * 4
    peak, kind = measured_peak_gbs()
    gbs = nbuf * am_bytes / (ms * 1e-3) / 1e9
    out = {"workload": "argmax_B128_vocab128000_plus_embed_gather_hidden2048", "us_per_pair": round(ms / nbuf * 1e3, 2),
           "gbs_lower_bound_of_argmax": round(gbs, 1), "frac": round(gbs / peak, 4), "peak": peak, "peak_kind": kind,
           "device_status": kv.device_status()}
    kv.close()
    return out


def _fill_normal_tiled(torch, t, g):
    """N(0,1) values for a large tensor: one 256 MB random block tiled (far larger than L2, so the
    timing sees fresh HBM lines; generating tens of GB of fresh normals takes longer than the bench)."""
    flat = t.view(-1)
    blk = min(flat.numel(), 128 * 1024 * 1024)
    flat[:blk].normal_(generator=g)
    off = blk
    while off < flat.numel():
        n = min(blk, flat.numel() - off)
        flat[off:off + n].copy_(flat[:n])
        off += n


def leg_serving_mix(args, torch, impl, rank, world, local_rank):
    """Configuration 5: 1,024 sequences with lognormal context lengths (median 2048, sigma 1.0 - the
    spread is not given by the configuration and is chosen here -, clipped to [16, 32704]), 8 attention
    layers, 64 consecutive decode steps with advancing positions.  The FIXED set is partitioned over
    the ranks by oxide_infer_b200.shard.assign_sequences: strong scaling, replicas, no collective.
    The reference arm runs all 1,024 sequences on one GPU (it has no multi-GPU path)."""
    import numpy as np
    from oxide_infer_b200 import rotary_tables
    from oxide_infer_b200.shard import assign_sequences, shard_keys
    nseq, layers, steps = 1024, 8, 64
    rng = np.random.default_rng(5)
    lens_all = np.clip(np.round(np.exp(rng.normal(np.log(2048), 1.0, nseq))), 16, 32768 - 64).astype(np.int64)
    parts = assign_sequences(lens_all, world)
    lens = lens_all[parts[rank]]
    b = len(lens)
    cap = lens + steps + 1
    g = torch.Generator(device="cuda").manual_seed(50 + rank)
    total_rows = int(cap.sum())
    offs = np.concatenate([[0], np.cumsum(cap)[:-1]]) * ROW_BYTES
    k_ptrs, v_ptrs, slabs = [], [], []
    for _ in range(layers):
        ks = torch.empty(total_rows, NKV, HD, dtype=torch.float16, device="cuda")
        vs = torch.empty(total_rows, NKV, HD, dtype=torch.float16, device="cuda")
        _fill_normal_tiled(torch, ks, g)
        _fill_normal_tiled(torch, vs, g)
        slabs.append((ks, vs))
        k_ptrs.append(torch.from_numpy(ks.data_ptr() + offs).cuda())
        v_ptrs.append(torch.from_numpy(vs.data_ptr() + offs).cuda())
    rn = lambda *s: torch.empty(*s, dtype=torch.float16, device="cuda").normal_(generator=g)
    q, k, v, gate = rn(layers, b, NQ, HD), rn(layers, b, NKV, HD), rn(layers, b, NKV, HD), rn(layers, b, NQ)
    qw = torch.ones(HD, dtype=torch.float16, device="cuda")
    cos, sin = rotary_tables(32768 + steps, 1e6, 0.5)
    cos, sin = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
    ctx = torch.zeros(layers, b, NQ, HD, dtype=torch.float16, device="cuda")
    pos_steps = [torch.from_numpy((lens + s_).astype(np.int32)).cuda() for s_ in range(steps)]
    len_steps = [p + 1 for p in pos_steps]
    status = None
    if impl == "ours":
        from oxide_infer_b200 import KvPath
        kv = KvPath(local_rank, max_batch=max(b, 1), max_seq_len=32768 + steps, max_prefill_rows=0)

        def one(s_):
            for l in range(layers):
                kv.append_decode(ctx[l], q[l], k[l], v[l], gate[l], qw, qw, cos, sin, pos_steps[s_], len_steps[s_],
                                 k_ptrs[l], v_ptrs[l])
    else:
        from oracle import refptx
        ref = refptx.RefPtx()
        max_len = int(lens.max()) + steps + 1
        nch = ref.nchunks_for(max_len, 0)
        acc = torch.empty(b * nch * NQ * HD, dtype=torch.float32, device="cuda")
        stats = torch.empty(b * nch * NQ * 2, dtype=torch.float32, device="cuda")
        qb, kb = q.clone(), k.clone()

        def one(s_):
            for l in range(layers):
                ref.append(qb[l], kb[l], v[l], qw, qw, cos, sin, pos_steps[s_], k_ptrs[l], v_ptrs[l], b)
                ref.decode_attention(ctx[l], qb[l], gate[l], k_ptrs[l], v_ptrs[l], len_steps[s_], b, 0,
                                     int(lens.max()) + s_ + 1, acc, stats)

    def run64():
        for s_ in range(steps):
            one(s_)

    def barrier():
        if world > 1 and impl == "ours":
            torch.distributed.barrier()
        torch.cuda.synchronize()

    for s_ in range(4):  # warm-up steps (W >= 3)
        one(s_)
    launch = "stream launches"
    fn = run64
    try:  # the 64 steps as one captured graph: no host launch gaps at 8 GPUs, where a layer takes ~70 us
        graph = _graph_of(torch, run64)
        graph.replay()
        fn, launch = graph.replay, "cuda graph replay of the 64 captured steps"
    except Exception as exc:
        if rank == 0:
            print(f"serving mix: cuda graph capture failed ({exc}); stream launches", file=sys.stderr)
    ms = _timed_region(torch, fn, 1, barrier)
    if impl == "ours":
        status = kv.device_status()
    finite = bool(torch.isfinite(ctx.float()).all().item())
    tt = torch.tensor([ms], dtype=torch.float64, device="cuda")
    if world > 1 and impl == "ours":
        torch.distributed.all_reduce(tt, op=torch.distributed.ReduceOp.MAX)
    ms = float(tt.item())
    if impl == "ours":
        kv.close()
    total_bytes = sum(layers * alg_bytes_layer(lens_all + s_ + 1) for s_ in range(steps))
    keys = shard_keys(lens_all, parts)
    peak, kind = measured_peak_gbs()
    gbs = total_bytes / (ms * 1e-3) / 1e9
    return {"workload": "serving_mix_1024seq_lognormal_median2048_sigma1_8layers_64steps", "scaling": "strong",
            "n_gpus": world, "ms_per_64_steps": round(ms, 3), "tokens_per_s": round(nseq * steps / (ms * 1e-3), 1),
            "gbs": round(gbs, 1), "gbs_per_gpu": round(gbs / world, 1), "frac_per_gpu": round(gbs / world / peak, 4),
            "peak": peak, "peak_kind": kind, "launch": launch, "sequences": nseq,
            "kv_bytes_total": int(lens_all.sum()) * layers * 2 * ROW_BYTES,
            "keys_per_gpu_min_max": [int(min(keys)), int(max(keys))], "longest_row_keys": int(lens_all.max()) + steps,
            "device_status": status, "finite": finite}


# ---------------------------------------------------------------------------
# Detailed single-workload lines (--workload ...), this library only.

def _time_loop(torch, fn, steps, warmup):
    stream = torch.cuda.current_stream()
    for _ in range(max(3, warmup)):
        fn()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record(stream)
    for _ in range(steps):
        fn()
    t1.record(stream)
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) / steps


def run_sample(args, torch):
    """Sampling side of a decode step at the reference's sizes: argmax over 128,000 f16 logits for
    each of 128 rows (batch_engine.rs:75, :1367-1378) and the embedding gather of the 128 chosen
    rows of a [128000][2048] table.  Eight distinct logits buffers (262 MB) rotate so that no launch
    finds its input in L2."""
    from oxide_infer_b200 import KvPath
    b, vocab, hid, nbuf = 128, 128000, 2048, 8
    kv = KvPath(0, max_batch=b, max_seq_len=256, max_prefill_rows=0)
    g = torch.Generator(device="cuda").manual_seed(6)
    logits = [torch.empty(b, vocab, dtype=torch.float16, device="cuda").normal_(generator=g) for _ in range(nbuf)]
    table = torch.empty(vocab, hid, dtype=torch.float16, device="cuda").normal_(generator=g)
    tok = torch.zeros(nbuf, b, dtype=torch.int32, device="cuda")
    hidden = torch.zeros(b, hid, dtype=torch.float16, device="cuda")
    sampler = ClockSampler(0)
    sampler.start()
    sampler.wait_ready()

    def ours():
        for i in range(nbuf):
            kv.argmax(tok[i], logits[i])
            kv.embed_lookup(hidden, table, tok[i])
    w0 = time.perf_counter()
    ms = _time_loop(torch, ours, args.steps, args.warmup)
    ms_am = _time_loop(torch, lambda: [kv.argmax(tok[i], logits[i]) for i in range(nbuf)], args.steps, args.warmup)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ours()
    ms_graph = _time_loop(torch, graph.replay, max(args.steps, 200), args.warmup)
    graph_am = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph_am):
        for i in range(nbuf):
            kv.argmax(tok[i], logits[i])
    ms_am_graph = _time_loop(torch, graph_am.replay, max(args.steps, 200), args.warmup)
    clocks = sampler.window(w0, time.perf_counter())
    want = torch.stack([x.float().argmax(1) for x in logits]).int()  # random normal f16 logits: ties are possible but
    agree = float((want == tok).float().mean().item())              # rare; parity proper is in tests/test_gpu_sample.py
    sampler.stop()
    pair_bytes = b * vocab * 2 + b * 4 + b * (4 + 2 * hid * 2)   # logits once, ids out; ids in, row in, row out
    am_bytes = b * vocab * 2 + b * 4
    peak, kind = measured_peak_gbs()
    gbs = nbuf * pair_bytes / (ms_graph * 1e-3) / 1e9
    am_gbs = nbuf * am_bytes / (ms_am_graph * 1e-3) / 1e9
    return {"metric": "argmax_embed_hbm_gbs", "value": round(gbs, 1), "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_graph, 4), "us_per_pair": round(ms_graph / nbuf * 1e3, 2),
            "us_per_pair_stream_launches": round(ms / nbuf * 1e3, 2), "us_per_argmax_stream_launches": round(ms_am / nbuf * 1e3, 2), "us_per_argmax": round(ms_am_graph / nbuf * 1e3, 2),
            "higher_is_better": True, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "argmax_B128_vocab128000_plus_embed_gather_hidden2048", "buffers": nbuf,
                       "l2": "8 distinct logits buffers (262 MB) rotate", "note": "value is the 8 pairs replayed as a CUDA graph"},
            "roofline": {"kernel": "argmax_kernel", "bound": "hbm", "achieved": round(am_gbs, 1), "peak": peak, "peak_kind": kind,
                         "unit": "GB/s", "frac": round(am_gbs / peak, 4), "bytes_per_launch": am_bytes},
            "agreement_with_torch_argmax": agree,
            "gpu_launches": 2 * nbuf * args.steps, "clocks": clocks, "device_status": kv.device_status()}


def run_decode_paged(args, torch):
    """The headline decode step (8 layers, batch 128, context 4096, fused append + attention) with
    the K/V rows behind block tables: the same slabs seen as pools of 16- or 256-token blocks, every
    sequence's pages scattered over the pool by a seeded permutation.  Contiguous step timed beside
    it in the same process; all as CUDA-graph replays."""
    import numpy as np
    from oxide_infer_b200 import KvPath, PagedLayout
    w = build_workload(torch, CTX, BATCH, LAYERS, 1)
    kv = KvPath(0, max_batch=BATCH, max_seq_len=CTX, max_prefill_rows=0)
    sampler = ClockSampler(0)
    sampler.start()
    sampler.wait_ready()
    w0 = time.perf_counter()

    def timed(step):
        for _ in range(3):
            step()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        return _time_loop(torch, graph.replay, args.steps, args.warmup)

    def contiguous():
        for l in range(LAYERS):
            kv.append_decode(w.ctx[l], w.q[l], w.k[l], w.v[l], w.gate[l], w.qw[l], w.kw[l], w.cos, w.sin, w.pos, w.lens,
                             w.k_ptrs[l], w.v_ptrs[l])
    res = {"contiguous": timed(contiguous)}
    rng = np.random.default_rng(7)
    for bs in (16, 256):
        per_seq = CTX // bs
        nblk = BATCH * per_seq
        table = torch.from_numpy(rng.permutation(nblk).astype(np.int32).reshape(BATCH, per_seq)).cuda()
        lays = [PagedLayout.of(w.k_slab[l].view(nblk, bs, NKV, HD), w.v_slab[l].view(nblk, bs, NKV, HD), table, bs)
                for l in range(LAYERS)]

        def paged():
            for l in range(LAYERS):
                kv.append_decode_paged(w.ctx[l], w.q[l], w.k[l], w.v[l], w.gate[l], w.qw[l], w.kw[l], w.cos, w.sin,
                                       w.lens, lays[l])
        res[f"paged_{bs}"] = timed(paged)
    clocks = sampler.window(w0, time.perf_counter())
    sampler.stop()
    step_bytes = LAYERS * alg_bytes_layer(w.seq_lens_host)
    peak, kind = measured_peak_gbs()
    gbs = {k: step_bytes / (ms * 1e-3) / 1e9 for k, ms in res.items()}
    return {"metric": "gqa_decode_step_paged_hbm_gbs", "value": round(gbs["paged_16"], 1), "unit": "GB/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(res["paged_16"], 4),
            "us_per_layer": {k: round(ms / LAYERS * 1e3, 2) for k, ms in res.items()},
            "gbs": {k: round(v, 1) for k, v in gbs.items()}, "higher_is_better": True, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "decode_step_8_attention_layers_B128_ctx4096_paged_kv", "block_sizes": [16, 256],
                       "tables": "seeded permutation of all blocks of the pool", "launch": "cuda graph replay"},
            "roofline": {"kernel": "decode_attn_kernel<fused append, paged> + decode_merge_kernel", "bound": "hbm",
                         "achieved": round(gbs["paged_16"], 1), "peak": peak, "peak_kind": kind, "unit": "GB/s",
                         "frac": round(gbs["paged_16"] / peak, 4)},
            "gpu_launches": 2 * LAYERS * args.steps, "clocks": clocks, "device_status": kv.device_status()}


def _prefill_long_prompt_leg(args, torch, rn):
    """A small wave of long prompts (2 requests, 128 new rows each, 32,768 keys of prefix): 16 work
    items for 148 SMs unless the key-range split (the handle's default) cuts the blocks into parts."""
    import numpy as np
    from oxide_infer_b200 import KvPath
    nseq, new, prefix = 2, 128, 32768
    rows = nseq * new
    kc = [rn(prefix + new, NKV, HD) for _ in range(nseq)]
    vc = [rn(prefix + new, NKV, HD) for _ in range(nseq)]
    q, gate = rn(rows, NQ, HD), rn(rows, NQ)
    owner = np.repeat(np.arange(nseq), new)
    lens = (prefix + 1 + np.tile(np.arange(new), nseq)).astype(np.int32)
    kp = torch.tensor([kc[i].data_ptr() for i in owner], dtype=torch.int64, device="cuda")
    vp = torch.tensor([vc[i].data_ptr() for i in owner], dtype=torch.int64, device="cuda")
    dlen = torch.from_numpy(lens).cuda()
    ctx = torch.zeros(rows, NQ, HD, dtype=torch.float16, device="cuda")
    out = {"rows": rows, "prefix": prefix}
    for name, part_keys in (("unsplit", 0), ("split", 512)):
        kv = KvPath(0, max_batch=8, max_seq_len=prefix + new, max_prefill_rows=rows)
        if not part_keys:
            kv.prefill_split_configure(0, 0)  # a new handle splits small waves by default
        ms = _time_loop(torch, lambda: kv.prefill_attn(ctx, q, gate, kp, vp, dlen, 0), args.steps, args.warmup)
        out["us_" + name] = round(ms * 1e3, 1)
        out["status_" + name] = kv.device_status()
        del kv
    flops = 4.0 * rows * NQ * HD * (prefix + (new + 1) / 2.0)
    out["tflops_best"] = round(flops / (min(v for k, v in out.items() if k.startswith("us_")) * 1e-6) / 1e12, 1)
    return out


def run_prefill(args, torch):
    """Config 4: one wave of 128 new tokens for each of 32 sequences, prefixes uniform 0..8192
    (seeded), one attention layer: append of the 4096 wave rows, then causal gated GQA attention."""
    import numpy as np
    from oxide_infer_b200 import KvPath, rotary_tables
    nseq, new = 32, 128
    rows = nseq * new
    rng = np.random.default_rng(4)
    prefix = rng.integers(0, 8193, nseq)
    kv = KvPath(0, max_batch=128, max_seq_len=8192 + new, max_prefill_rows=rows)
    g = torch.Generator(device="cuda").manual_seed(4)
    rn = lambda *s: torch.empty(*s, dtype=torch.float16, device="cuda").normal_(generator=g)
    # every sequence's K and V rows live in one slab, as in the reference's KvPool (kv_pool.rs:31-61)
    cap = [int(p) + new for p in prefix]
    slab = rn(2 * sum(cap), NKV, HD)
    offs = np.concatenate([[0], np.cumsum(cap)])
    kc = [slab[offs[i]:offs[i + 1]] for i in range(nseq)]
    vc = [slab[sum(cap) + offs[i]:sum(cap) + offs[i + 1]] for i in range(nseq)]
    q0, k, v, gate = rn(rows, NQ, HD), rn(rows, NKV, HD), rn(rows, NKV, HD), rn(rows, NQ)
    q = q0.clone()
    qw = (1 + 0.02 * torch.randn(HD, device="cuda", generator=g)).half()
    kw = (1 + 0.02 * torch.randn(HD, device="cuda", generator=g)).half()
    cos, sin = rotary_tables(8192 + new, 1e6, 0.5)
    cos, sin = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
    owner = np.repeat(np.arange(nseq), new)
    pos = (prefix[owner] + np.tile(np.arange(new), nseq)).astype(np.int32)
    kp = torch.tensor([kc[i].data_ptr() for i in owner], dtype=torch.int64, device="cuda")
    vp = torch.tensor([vc[i].data_ptr() for i in owner], dtype=torch.int64, device="cuda")
    dpos = torch.from_numpy(pos).cuda()
    dlen = torch.from_numpy(pos + 1).cuda()
    ctx = torch.zeros(rows, NQ, HD, dtype=torch.float16, device="cuda")
    sampler = ClockSampler(0)
    sampler.start()
    sampler.wait_ready()

    def attn():
        kv.prefill_attn(ctx, q, gate, kp, vp, dlen, 0)

    def wave():
        kv.append(q, k, v, qw, kw, cos, sin, dpos, kp, vp, batch=rows)
        attn()
    w0 = time.perf_counter()
    ms_wave = _time_loop(torch, wave, args.steps, args.warmup)
    ms_attn = _time_loop(torch, attn, args.steps, args.warmup)
    clocks = sampler.window(w0, time.perf_counter())
    # the same wave through a sliding-window layer (the reference's model has 5 of them, window 256)
    ms_attn_w256 = _time_loop(torch, lambda: kv.prefill_attn(ctx, q, gate, kp, vp, dlen, 256), args.steps, args.warmup)
    kv.register_kv_slab(slab)  # the same wave with TMA tile copies instead of per-thread 16-byte copies
    ms_attn_tma = _time_loop(torch, attn, args.steps, args.warmup)
    kv.register_kv_slab(None)
    long_wave = _prefill_long_prompt_leg(args, torch, rn)
    sampler.stop()
    flops = float(sum(8192 * (128 * int(p) + 8256) for p in prefix))
    kv_bytes = float(sum(2048 * (int(p) + new) for p in prefix)) + rows * (4096 + 4096 + 32)
    peak_tf = 1354.7
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    kind = "fallback"
    if os.path.exists(pk):
        try:
            peak_tf, kind = float(json.load(open(pk))["bf16_tflops_sustained"]), "measured"
        except Exception:
            pass
    tf = flops / (ms_attn * 1e-3) / 1e12
    return {"metric": "prefill_attention_tflops", "value": round(tf, 2), "unit": "TFLOP/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_wave, 4),
            "ms_attention_only": round(ms_attn, 4), "ms_attention_only_registered_slab_tma": round(ms_attn_tma, 4),
            "ms_attention_only_window_256": round(ms_attn_w256, 4),
            "higher_is_better": True, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "prefill_wave_32seq_x128tok_prefix_U0_8192_one_layer", "rows": rows,
                       "prefix_sum": int(prefix.sum()), "causal_exact_flops": flops, "algorithmic_bytes": kv_bytes},
            "roofline": {"kernel": "prefill_attn_kernel", "bound": "tensor", "achieved": round(tf, 2), "peak": peak_tf,
                         "peak_kind": kind, "unit": "TFLOP/s", "frac": round(tf / peak_tf, 4)},
            "long_prompt_wave": long_wave,
            "gpu_launches": 3 * args.steps, "clocks": clocks, "device_status": kv.device_status()}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-secondary", action="store_true", help="headline workload only (skip the other configurations)")
    ap.add_argument("--layers", type=int, default=LAYERS, help="override for small profiling cases")
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--ctx", type=int, default=CTX)
    ap.add_argument("--ragged", action="store_true",
                    help="decode workload with context lengths uniform 1024..4096 (configuration 2's ragged variant)")
    ap.add_argument("--workload", default="decode", choices=["decode", "conv", "prefill", "serving_mix", "sample", "decode_paged", "project"],
                    help="decode = the headline line; conv / prefill / sample = secondary single-GPU lines")
    args = ap.parse_args()
    globals().update(LAYERS=args.layers, BATCH=args.batch, CTX=args.ctx, RAGGED=args.ragged)
    args.warmup = max(args.warmup, 3)
    if (args.layers, args.batch, args.ctx) != (8, 128, 4096) or args.ragged or args.no_e2e:
        args.no_secondary = True  # the other configurations ride along with the default headline only

    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference" and rank != 0:
        return 0
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1 and args.impl == "ours":
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        if args.workload == "conv":
            line = leg_conv(args, torch, args.impl) if rank == 0 else None
        elif args.workload == "prefill":
            line = (run_prefill(args, torch) if args.impl == "ours" else leg_prefill(args, torch, "reference")) if rank == 0 else None
        elif args.workload == "project":
            line = leg_project_append(args, torch, args.impl) if rank == 0 else None
        elif args.workload == "sample":
            line = run_sample(args, torch) if rank == 0 else None
        elif args.workload == "decode_paged":
            line = run_decode_paged(args, torch) if rank == 0 else None
        elif args.workload == "serving_mix":
            line = leg_serving_mix(args, torch, args.impl, rank, world, local_rank)
            line = line if rank == 0 else None
        else:
            line = (run_ours if args.impl == "ours" else run_reference)(args, torch, rank, world, local_rank)
        if line is not None:
            print(json.dumps(line), flush=True)
    finally:
        if world > 1 and args.impl == "ours" and torch.distributed.is_initialized():
            torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
