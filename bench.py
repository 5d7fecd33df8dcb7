#!/usr/bin/env python
"""Benchmark of the block-masked MHA hot path (and, with --workload encoder, the BERT encoder forward).

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload attention|encoder]

N > 1 is launched with torchrun, one rank per GPU; ranks own independent shards (weak scaling for
attention: every rank runs the full configuration on its own seeded batch; the encoder shards the
configuration's batch).  No collective runs inside the timed region.  Rank 0 prints ONE JSON line.

A step = one pass of the hot path over one batch of synthetic input: one attention launch over all
(batch, head) problems of the configuration with the block index already built (the reference
benchmark builds the index outside its timed loop too, src/benchmk_attn_unified.py:315-346).
Between timed steps a 256 MiB buffer is written to flush L2; each step is timed with its own CUDA
event pair on the launching stream, and the sum over the K steps is reduced with max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "sc25-stof-ad_b200"))
sys.path.insert(0, ROOT)

import torch  # noqa: E402


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"], "tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _loop(self):
        nv = self._nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4)}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


# --------------------------------------------------------------------------------------------
# CPU baseline: the reference's PyTorch-native path (oracle port) on the host cores
# --------------------------------------------------------------------------------------------
def cpu_attention_pass(cfg, n_load_blocks, elements=None):
    """One pass of the reference's dense `torch_attn_std` path in fp32 over `elements` batch elements (default: the whole
    configuration), one element at a time on all host threads; returns (seconds, effective FLOPs of the pass)."""
    from oracle import attention as oa
    from stof_b200 import workloads as wl
    torch.set_num_threads(os.cpu_count() or 1)
    elements = cfg.batch if elements is None else elements
    g = torch.Generator().manual_seed(cfg.seed)
    q, k, v = (torch.randn(1, cfg.heads, cfg.seq_len, cfg.head_dim, generator=g).half().float() for _ in range(3))
    mask = wl.config_mask(cfg).float()
    t0 = time.perf_counter()
    for _ in range(elements):
        oa.torch_attn_std(q, k, v, mask)
    return time.perf_counter() - t0, wl.attention_flops(n_load_blocks, elements, cfg.heads)


def cpu_attention_sample(cfg, n_load_blocks, budget_s: float = 10.0):
    """CPU baseline of the GPU arm: whole-configuration passes of `cpu_attention_pass` until about `budget_s` seconds of
    CPU work have been spent (at least one pass); returns (effective TFLOP/s, seconds, description)."""
    cpu_attention_pass(cfg, n_load_blocks, 1)                                   # warm the thread pool
    secs, flops, passes = 0.0, 0.0, 0
    while passes == 0 or secs < budget_s:
        dt, fl = cpu_attention_pass(cfg, n_load_blocks)
        secs += dt
        flops += fl
        passes += 1
    return flops / secs / 1e12, secs, (f"{passes} pass(es) over all {cfg.batch} batch elements ({cfg.heads} heads, S={cfg.seq_len}), "
                                       f"dense fp32 torch_attn_std on {torch.get_num_threads()} threads")


def run_reference(args):
    """Reference arm: the reference's own PyTorch-native path (`torch_attn_std`, the dense masked attention its verify scripts
    compare against) on the host cores; one step = the whole configuration 2 once."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from stof_b200 import workloads as wl
    cfg = wl.ATTENTION_CONFIGS["cfg2"]
    nb = int(wl.block_matrix(cfg.mask, cfg.seq_len // cfg.block, cfg.seed).sum().item())
    for _ in range(max(args.warmup, 1)):
        cpu_attention_pass(cfg, nb, 2)
    t0 = time.perf_counter()
    vals = [cpu_attention_pass(cfg, nb) for _ in range(args.steps)]
    wall = time.perf_counter() - t0
    secs = sum(v[0] for v in vals) / len(vals)
    tflops = vals[0][1] / secs / 1e12
    cores = torch.get_num_threads()
    sample = f"every step: all {cfg.batch} batch elements ({cfg.heads} heads, S={cfg.seq_len}) dense fp32 torch_attn_std on {cores} threads"
    line = {"impl": "reference", "metric": "masked-MHA effective TFLOP/s", "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": cfg.name, "batch": cfg.batch, "heads": cfg.heads, "seq_len": cfg.seq_len, "head_dim": 64,
                       "mask": "bigbird block 64: 3 sliding + 2 global + 3 random per row (seed 1)", "load_blocks": nb},
            "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0, "wall_s": wall}
    print(json.dumps(line))
    return 0


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
def run_attention(args, rank, world, local):
    import stof_b200
    from stof_b200 import _lib, dist as sd, workloads as wl
    dev = torch.device("cuda", local)
    cfg = wl.ATTENTION_CONFIGS[args.config]
    if args.batch:
        cfg = wl.AttentionConfig(cfg.name + f"_batch{args.batch}", args.batch, cfg.heads, cfg.seq_len, cfg.seed, cfg.mask)
    peaks = measured_peaks()

    # weak scaling: every rank runs the whole configuration on its own draw (seed + rank)
    cfg_rank = cfg if rank == 0 else wl.AttentionConfig(cfg.name, cfg.batch, cfg.heads, cfg.seq_len, cfg.seed + 100 * rank, cfg.mask)
    q_h, k_h, v_h = (t.pin_memory() for t in wl.attention_inputs(cfg_rank))
    q, k, v = (t.to(dev, non_blocking=True) for t in (q_h, k_h, v_h))
    out = torch.empty_like(q)
    out_h = torch.empty_like(q_h).pin_memory()
    mask = wl.config_mask(cfg).to(dev)

    # block index (once, outside the timed loop) + its own timing
    idx = stof_b200.get_sparse_storage(mask, cfg.block, cfg.block)
    torch.cuda.synchronize(dev)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    comp_ms = []
    for _ in range(5):
        ev0.record()
        idx = stof_b200.get_sparse_storage(mask, cfg.block, cfg.block)
        ev1.record()
        torch.cuda.synchronize(dev)
        comp_ms.append(ev0.elapsed_time(ev1))
    nnz, frp, fci, prp, pci, pbm, lrp, lci = idx
    n_load = int(lrp[-1].item())
    # the two compaction kernels alone (sizes known, no host read in between): enqueued back to back, and as a CUDA graph replay
    refresher = stof_b200.SparseStorageRefresher(mask, cfg.block, cfg.block)
    reps = 50
    for _ in range(5):
        refresher.refresh()
    torch.cuda.synchronize(dev)
    ev0.record()
    for _ in range(reps):
        refresher.refresh()
    ev1.record()
    torch.cuda.synchronize(dev)
    comp_eager_us = ev0.elapsed_time(ev1) / reps * 1e3
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        refresher.refresh()
    torch.cuda.current_stream(dev).wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        refresher.refresh()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize(dev)
    ev0.record()
    for _ in range(reps):
        graph.replay()
    ev1.record()
    torch.cuda.synchronize(dev)
    comp_graph_us = ev0.elapsed_time(ev1) / reps * 1e3
    refresher.check()
    del graph
    flops = wl.attention_flops(n_load, cfg.batch, cfg.heads, cfg.block, cfg.block, cfg.head_dim)

    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def step():
        stof_b200.block_attention(q, k, v, out, frp, fci, prp, pci, pbm, lrp, lci, cfg.block, cfg.block)

    for _ in range(max(args.warmup, 3)):
        flush.zero_()
        step()
    torch.cuda.synchronize(dev)
    _lib.check_status(dev, "warm-up")

    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize(dev)
    with ClockSampler(physical_gpu_index(local)) as clocks:
        t_wall = time.perf_counter()
        for i in range(args.steps):
            flush.zero_()
            starts[i].record()
            step()
            ends[i].record()
        torch.cuda.synchronize(dev)
        wall = time.perf_counter() - t_wall
        # keep the GPU under the same load a little longer so that the clock sampler sees it
        t_end = time.perf_counter() + (0.0 if args.kernel_only else 0.25)
        while time.perf_counter() < t_end:
            step()
        torch.cuda.synchronize(dev)
    if world > 1:
        torch.distributed.barrier()
    _lib.check_status(dev, "timed region")
    dev_ms = sum(s.elapsed_time(e) for s, e in zip(starts, ends))
    dev_ms_max = sd.max_over_ranks(dev_ms, dev)
    ms_per_step = dev_ms_max / args.steps
    total_flops = flops * world
    value = total_flops / (ms_per_step * 1e-3) / 1e12

    if args.kernel_only:
        args.no_encoder = True
        if rank == 0:
            print(json.dumps({"metric": "masked-MHA effective TFLOP/s", "value": value, "unit": "TFLOP/s", "ms_per_step": ms_per_step,
                              "config": {"workload": cfg.name, "load_blocks": n_load}, "note": "kernel-only run (profiling aid)"}))
        return 0
    # end to end with host buffers through the host-buffer form of the operator: H2D of q, k, v, the kernel (in place on q, as
    # the reference operator does) and D2H of the result, batch chunks pipelined over three streams
    e2e_steps = args.steps
    def e2e_step():
        stof_b200.block_attention_host(q_h, k_h, v_h, out_h, frp, fci, prp, pci, pbm, lrp, lci, cfg.block, cfg.block)
    for _ in range(2):
        e2e_step()
    torch.cuda.synchronize(dev)
    if world > 1:
        torch.distributed.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    torch.cuda.synchronize(dev)
    _lib.check_status(dev, "end-to-end region")
    e2e_ms = sd.max_over_ranks(e0.elapsed_time(e1), dev) / e2e_steps
    e2e_value = total_flops / (e2e_ms * 1e-3) / 1e12
    h2d = 3 * q_h.numel() * 2
    d2h = out_h.numel() * 2

    encoder = None
    alg_bytes = 4 * q.numel() * 2
    if not args.no_encoder:
        q = k = v = out = flush = None
        torch.cuda.empty_cache()
        encoder = encoder_measure(args, rank, world, local, steps=max(2, min(args.steps, 3)), warmup=3)
    if rank != 0:
        return 0
    # parity spot check of the timed output against the oracle is the job of the tests; here only sanity
    finite = bool(torch.isfinite(out_h.float()).all())
    cpu_val, cpu_s, cpu_desc = cpu_attention_sample(cfg, n_load, 10.0)
    mask_bytes = mask.numel() * 2
    comp_best = min(comp_ms)
    achieved = flops / (dev_ms / args.steps * 1e-3) / 1e12       # this rank's kernel
    # DRAM read+write bytes of one launch from an ncu capture at batch 8 of the same mask (86.2 MB), scaled by batch
    traffic = 86.230e6 * cfg.batch / 8 if cfg.mask == "bigbird" and cfg.seq_len == 2048 and cfg.heads == 12 else None
    line = {
        "metric": "masked-MHA effective TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": cfg.name, "batch_per_gpu": cfg.batch, "heads": cfg.heads, "seq_len": cfg.seq_len, "head_dim": cfg.head_dim,
                   "mask": f"{cfg.mask} block {cfg.block}", "load_blocks": n_load, "flops_per_step_per_gpu": flops,
                   "l2": "256 MiB flush write between timed steps", "parallelism": f"independent batch shards x{world}"},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": achieved / peaks["tflops"],
                     "traffic": traffic, "traffic_unit": "bytes per launch (ncu dram read+write, batch-8 capture scaled)",
                     "algorithmic_bytes": alg_bytes, "peak_source": peaks["source"] + " bf16 burst",
                     "frac_of_sustained": achieved / peaks["tflops_sustained"], "kernel": "block_attn_kernel"},
        "cpu_baseline": {"value": cpu_val, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port", "sample": cpu_desc,
                         "seconds": cpu_s},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                "api": "stof_b200.block_attention_host: pinned host q/k/v in, host result out, four batch chunks over three streams"},
        "gpu_launches": args.steps,
        "clocks": clocks.summary(),
        "compaction": {"ms": comp_best, "mask_bytes": mask_bytes, "gbs": mask_bytes / (comp_best * 1e-3) / 1e9,
                       "note": "classify + fill + host read of the three totals, S=%d" % cfg.seq_len,
                       "kernels_back_to_back_us": comp_eager_us, "kernels_graph_replay_us": comp_graph_us,
                       "kernels_gbs": mask_bytes / (comp_graph_us * 1e-6) / 1e9},
        "wall_s_timed_region": wall, "output_finite": finite,
    }
    if encoder is not None:
        line["encoder"] = encoder
    print(json.dumps(line))
    return 0


def encoder_measure(args, rank, world, local, steps, warmup):
    """BERT-large 24-layer forward (config 5), the configuration's batch of 64 sharded over the ranks (strong scaling);
    returns the dict that the attention line carries under "encoder" (None on ranks other than 0)."""
    import stof_b200
    from stof_b200 import _lib, dist as sd, workloads as wl
    dev = torch.device("cuda", local)
    cfg = wl.ENCODER_CONFIGS["cfg5"]
    lo, hi = sd.shard_range(cfg.batch, rank, world)
    x = wl.encoder_input(cfg, (lo, hi)).to(dev)
    layers = [stof_b200.EncoderWeights.from_dict(p, dev) for p in wl.encoder_weights(cfg)]
    enc = stof_b200.BertEncoder(layers, cfg.heads, cfg.eps, "erf", cfg.block, cfg.block)
    idx = enc.set_mask(wl.config_mask(cfg).to(dev))
    n_load = int(idx[5][-1].item())
    for _ in range(warmup):
        enc(x)
    torch.cuda.synchronize(dev)
    _lib.check_status(dev, "encoder warm-up")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize(dev)
    e0.record()
    for _ in range(steps):
        enc(x)
    e1.record()
    torch.cuda.synchronize(dev)
    if world > 1:
        torch.distributed.barrier()
    _lib.check_status(dev, "encoder timed region")
    ms = sd.max_over_ranks(e0.elapsed_time(e1), dev) / steps
    if rank != 0:
        return None
    peaks = measured_peaks()
    tflops = wl.encoder_flops(cfg, n_load, cfg.batch) / (ms * 1e-3) / 1e12
    return {"metric": "BERT encoder tokens/s", "value": cfg.batch * cfg.seq_len / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
            "steps": steps, "warmup": warmup, "scaling": "strong", "workload": cfg.name, "global_batch": cfg.batch, "seq_len": cfg.seq_len,
            "layers": cfg.layers, "load_blocks": n_load, "tflops_all_gpus": tflops,
            "frac_of_sustained_peak_per_gpu": tflops / world / peaks["tflops_sustained"], "gpu_launches": steps * cfg.layers * 7}


def run_encoder(args, rank, world, local):
    import stof_b200
    from stof_b200 import _lib, dist as sd, workloads as wl
    dev = torch.device("cuda", local)
    cfg = wl.ENCODER_CONFIGS[args.config if args.config in wl.ENCODER_CONFIGS else "cfg5"]
    peaks = measured_peaks()
    lo, hi = sd.shard_range(cfg.batch, rank, world)          # strong scaling: the configuration's batch is sharded
    x_h = wl.encoder_input(cfg, (lo, hi)).pin_memory()
    x = x_h.to(dev)
    layers = [stof_b200.EncoderWeights.from_dict(p, dev) for p in wl.encoder_weights(cfg)]
    enc = stof_b200.BertEncoder(layers, cfg.heads, cfg.eps, "erf", cfg.block, cfg.block)
    idx = enc.set_mask(wl.config_mask(cfg).to(dev))
    n_load = int(idx[5][-1].item())
    for _ in range(max(args.warmup, 3)):
        y = enc(x)
    torch.cuda.synchronize(dev)
    _lib.check_status(dev, "warm-up")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize(dev)
    with ClockSampler(physical_gpu_index(local)) as clocks:
        e0.record()
        for _ in range(args.steps):
            y = enc(x)
        e1.record()
        torch.cuda.synchronize(dev)
    if world > 1:
        torch.distributed.barrier()
    _lib.check_status(dev, "timed region")
    ms = sd.max_over_ranks(e0.elapsed_time(e1), dev) / args.steps
    tokens = cfg.batch * cfg.seq_len
    value = tokens / (ms * 1e-3)
    # end to end: hidden states from pinned host memory, one fp16 row block of the result back
    y_h = torch.empty(hi - lo, cfg.seq_len, cfg.hidden, dtype=torch.float16).pin_memory()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for _ in range(args.steps):
        x.copy_(x_h, non_blocking=True)
        y = enc(x)
        y_h.copy_(y, non_blocking=True)
    s1.record()
    torch.cuda.synchronize(dev)
    e2e_ms = sd.max_over_ranks(s0.elapsed_time(s1), dev) / args.steps
    # the same forward as one CUDA-graph launch per pass (all kernel launches recorded once)
    replay = enc.capture(x)
    for _ in range(2):
        replay()
    torch.cuda.synchronize(dev)
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record()
    for _ in range(args.steps):
        replay()
    g1.record()
    torch.cuda.synchronize(dev)
    _lib.check_status(dev, "graph replay")
    graph_ms = sd.max_over_ranks(g0.elapsed_time(g1), dev) / args.steps
    if rank != 0:
        return 0
    flops = wl.encoder_flops(cfg, n_load, cfg.batch)
    achieved = wl.encoder_flops(cfg, n_load, hi - lo) / (ms * 1e-3) / 1e12
    line = {
        "metric": "BERT encoder tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": cfg.name, "global_batch": cfg.batch, "seq_len": cfg.seq_len, "hidden": cfg.hidden, "heads": cfg.heads,
                   "ffn": cfg.ffn, "layers": cfg.layers, "mask": f"{cfg.mask} block {cfg.block}", "load_blocks": n_load,
                   "l2": "activations per layer (>= 0.5 GB) exceed L2", "parallelism": f"batch shards x{world}", "flops_per_step": flops},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops_sustained"], "unit": "TFLOP/s",
                     "frac": achieved / peaks["tflops_sustained"], "traffic": None, "peak_source": peaks["source"] + " bf16 sustained",
                     "kernel": "whole forward (GEMMs + attention + LayerNorm)"},
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": x_h.numel() * 2, "d2h_bytes_per_step": y_h.numel() * 2,
                "ms_per_step": e2e_ms},
        "gpu_launches": args.steps * cfg.layers * 7,
        "clocks": clocks.summary(),
        "graph_replay": {"ms_per_step": graph_ms, "value": tokens / (graph_ms * 1e-3), "unit": "tokens/s",
                         "note": "the same forward replayed as one CUDA graph (BertEncoder.capture)"},
    }
    print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="stof", choices=["stof", "reference"])
    ap.add_argument("--workload", default="attention", choices=["attention", "encoder"])
    ap.add_argument("--batch", type=int, default=0, help="override the batch size (profiling aid: smaller captures)")
    ap.add_argument("--no-encoder", action="store_true", help="skip the BERT-large encoder forward that the attention run reports under 'encoder'")
    ap.add_argument("--kernel-only", action="store_true", help="skip the end-to-end and CPU-baseline legs (profiling aid)")
    ap.add_argument("--config", default=None, help="cfg2 (default) or cfg3 for attention; cfg5 (default) or cfg4 for the encoder")
    args = ap.parse_args()
    if args.config is None:
        args.config = "cfg2" if args.workload == "attention" else "cfg5"
    if args.impl == "reference":
        return run_reference(args)
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: the hot path has no CPU fallback"}))
        return 1
    from stof_b200 import dist as sd
    rank, world, local = sd.init_from_env("nccl")
    torch.cuda.set_device(local)
    try:
        if args.workload == "attention":
            return run_attention(args, rank, world, local)
        return run_encoder(args, rank, world, local)
    finally:
        if world > 1 and torch.distributed.is_initialized():
            torch.distributed.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
