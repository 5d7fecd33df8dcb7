#!/usr/bin/env python
"""Benchmark of the block-masked MHA hot path (and, with --workload encoder, the BERT encoder forward).

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload attention|encoder]

N > 1 is launched with torchrun, one rank per GPU; ranks own independent shards.  The headline attention
number weak-scales (every rank runs the full configuration on its own seeded batch); the same line carries
the strong-scaled forms: configurations 2 and 3 sharded over batch x heads ("attention_sharded", every rank a
slice of the SAME seeded tensors, outputs gathered over NCCL after the timing and compared on rank 0) and the
encoder with its batch sharded.  No collective runs inside a timed region.  Rank 0 prints ONE JSON line.

A step = one pass of the hot path over one batch of synthetic input: one attention launch over all
(batch, head) problems of the configuration with the block index already built (the reference
benchmark builds the index outside its timed loop too, src/benchmk_attn_unified.py:315-346).
Between timed steps a 256 MiB buffer is written to flush L2; each step is timed with its own CUDA
event pair on the launching stream.  Blocks of exactly K such steps are repeated until a quarter of a
second of timed steps has run (so that the clock samples fall inside the timed region); the figure is the
median block, reduced with max over ranks, and the fastest block is reported beside it.  The output of
the last timed step is then compared with the CPU oracle on four (batch, head) pairs.
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


def attention_config_dict(cfg, n_load_blocks, flops, parallelism):
    """The `config` object of an attention line; both arms print exactly these keys for the same workload."""
    return {"workload": cfg.name, "batch_per_gpu": cfg.batch, "heads": cfg.heads, "seq_len": cfg.seq_len, "head_dim": cfg.head_dim,
            "mask": f"{cfg.mask} block {cfg.block}", "load_blocks": n_load_blocks, "flops_per_step_per_gpu": flops,
            "l2": "256 MiB flush write between timed steps", "parallelism": parallelism}


# DRAM read + write bytes of one block_attn_kernel launch, from the ncu capture summarised under profiles/ (file named per
# entry), with the batch that capture ran at: every (batch, head) pair is an independent set of work items, so the traffic
# of a launch grows in proportion to the batch.
NCU_TRAFFIC = {
    "mha_bigbird_b16_h12_s2048": {"bytes": 86.25e6, "batch": 8, "profile": "profiles/block_attn_kernel_cfg2_batch8.md"},
}


def timed_step_blocks(step, flush, steps, dev, min_ms=250.0, max_blocks=400, est_ms=None):
    """Runs blocks of exactly `steps` steps, each step after an L2 flush and inside its own CUDA event pair on the current
    stream, until `min_ms` of timed device time has been spent; returns the per-block sums in ms.  The number of blocks is
    fixed beforehand from `est_ms` (an estimate of one step) so that every rank runs the same count."""
    n_blocks = 1 if not est_ms else max(1, min(max_blocks, int(min_ms / (est_ms * steps)) + 1))
    sums = []
    for _ in range(n_blocks):
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        for i in range(steps):
            flush.zero_()
            starts[i].record()
            step()
            ends[i].record()
        torch.cuda.synchronize(dev)
        sums.append(sum(a.elapsed_time(b) for a, b in zip(starts, ends)))
    return sums


def median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2] if len(xs) % 2 else 0.5 * (xs[len(xs) // 2 - 1] + xs[len(xs) // 2])


def attention_parity(out, q, k, v, mask, pairs):
    """Largest |difference| between the kernel output `out` (device) and the oracle's fp32 dense masked attention on the given
    (batch, head) pairs; q, k, v (B,H,S,D) and mask (1,S,S) are the CPU tensors the device inputs were made from."""
    from oracle import attention as oa
    worst = 0.0
    for b, h in pairs:
        want = oa.masked_attention_fp32(q[b:b + 1, h:h + 1], k[b:b + 1, h:h + 1], v[b:b + 1, h:h + 1], mask.float())
        worst = max(worst, (out[b:b + 1, h:h + 1].float().cpu() - want).abs().max().item())
    return worst


PARITY_TOL = 2e-3          # max-abs against the fp32 oracle, fp16 inputs with fp32 accumulation


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
            "config": attention_config_dict(cfg, nb, wl.attention_flops(nb, cfg.batch, cfg.heads), f"independent batch shards x{args.gpus}"),
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
    ev0.record()
    step()
    ev1.record()
    torch.cuda.synchronize(dev)
    est_ms = sd.max_over_ranks(ev0.elapsed_time(ev1), dev)

    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize(dev)
    with ClockSampler(physical_gpu_index(local)) as clocks:
        t_wall = time.perf_counter()
        block_ms = timed_step_blocks(step, flush, args.steps, dev, min_ms=0.0 if args.kernel_only else 250.0, est_ms=est_ms)
        wall = time.perf_counter() - t_wall
    if world > 1:
        torch.distributed.barrier()
    _lib.check_status(dev, "timed region")
    dev_ms = median(block_ms)                                  # K steps of this rank
    ms_per_step = sd.max_over_ranks(dev_ms, dev) / args.steps
    ms_per_step_min = sd.max_over_ranks(min(block_ms), dev) / args.steps
    total_flops = flops * world
    value = total_flops / (ms_per_step * 1e-3) / 1e12

    if args.kernel_only:
        args.no_encoder = True
        if rank == 0:
            print(json.dumps({"metric": "masked-MHA effective TFLOP/s", "value": value, "unit": "TFLOP/s", "ms_per_step": ms_per_step,
                              "config": {"workload": cfg.name, "load_blocks": n_load}, "note": "kernel-only run (profiling aid)"}))
        return 0
    # parity of what was timed: the output of the last timed step against the fp32 oracle on four (batch, head) pairs
    pairs = sorted({(0, 0), (cfg.batch // 2, cfg.heads // 3), (cfg.batch - 1, cfg.heads - 1), (min(1, cfg.batch - 1), 5 % cfg.heads)})
    parity = attention_parity(out, q_h, k_h, v_h, wl.config_mask(cfg), pairs) if rank == 0 else 0.0
    out_full = out.clone() if (world > 1 and rank == 0 and args.config == "cfg2" and not args.batch) else None

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
    e2e_parity = attention_parity(out_h, q_h, k_h, v_h, wl.config_mask(cfg), pairs[:2]) if rank == 0 else 0.0

    alg_bytes = 4 * q.numel() * 2
    q = k = v = out = None
    sharded = None
    if world > 1:
        # strong scaling: configurations 2 and 3 split over batch x heads, every rank a slice of the same seeded tensors
        sharded = [attention_sharded(args, rank, world, local, wl.ATTENTION_CONFIGS[c], flush, out_full if c == "cfg2" else None)
                   for c in ("cfg2", "cfg3")]
    encoder = None
    if not args.no_encoder:
        out_full = flush = None
        torch.cuda.empty_cache()
        encoder = encoder_measure(args, rank, world, local, steps=max(args.steps, 20) if world > 1 else max(8, min(args.steps, 20)), warmup=3)
    if rank != 0:
        return 0
    cpu_val, cpu_s, cpu_desc = cpu_attention_sample(cfg, n_load, 10.0)
    mask_bytes = mask.numel() * 2
    comp_best = min(comp_ms)
    achieved = flops / (dev_ms / args.steps * 1e-3) / 1e12       # this rank's kernel
    tr = NCU_TRAFFIC.get(cfg.name.split("_batch")[0])
    traffic = tr["bytes"] * cfg.batch / tr["batch"] if tr else None
    line = {
        "metric": "masked-MHA effective TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": attention_config_dict(cfg, n_load, flops, f"independent batch shards x{world}"),
        "timed_blocks": {"blocks_of_k_steps": len(block_ms), "ms_per_step_median": ms_per_step, "ms_per_step_min": ms_per_step_min,
                         "timed_device_ms": sum(block_ms)},
        "parity": {"max_abs_vs_fp32_oracle": parity, "tolerance": PARITY_TOL, "batch_head_pairs": [list(x) for x in pairs],
                   "of": "output of the last timed step", "e2e_max_abs": e2e_parity},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": achieved / peaks["tflops"],
                     "traffic": traffic, "traffic_unit": "bytes per launch (ncu dram read+write of a smaller batch, scaled by batch)",
                     "traffic_source": tr["profile"] if tr else None,
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
        "wall_s_timed_region": wall,
    }
    if sharded is not None:
        line["attention_sharded"] = sharded
    if encoder is not None:
        line["encoder"] = encoder
    ok = parity <= PARITY_TOL and e2e_parity <= PARITY_TOL and all(r is None or r.get("ok", True) for r in (sharded or [])) and \
        (encoder is None or encoder.get("parity_first_layer", {}).get("ok", True))
    if not ok:
        line["error"] = "parity check failed"
    print(json.dumps(line))
    return 0 if ok else 1


def attention_sharded(args, rank, world, local, cfg, flush, full_out_rank0):
    """One attention configuration split over batch x heads (`dist.attention_shard`): every rank runs its slice of the SAME
    seeded q, k, v; aggregate effective TFLOP/s = FLOPs of the whole configuration / the slowest rank's time.  After the timing the
    slices are gathered over NCCL (the one collective of this path, verification only) and rank 0 compares the whole tensor
    with the fp32 oracle on (batch, head) pairs from different ranks' slices - and bit for bit with its own single-GPU result of
    the same configuration when it has one (`full_out_rank0`)."""
    import stof_b200
    from stof_b200 import _lib, dist as sd, workloads as wl
    dev = torch.device("cuda", local)
    (b0, b1), (h0, h1) = sd.attention_shard(cfg.batch, cfg.heads, rank, world)
    q_h, k_h, v_h = wl.attention_inputs(cfg)
    q, k, v = (t[b0:b1, h0:h1].contiguous().to(dev) for t in (q_h, k_h, v_h))
    out = torch.empty_like(q)
    idx = stof_b200.get_sparse_storage(wl.config_mask(cfg).to(dev), cfg.block, cfg.block)[1:]
    n_load = int(idx[5][-1].item())

    def step():
        stof_b200.block_attention(q, k, v, out, *idx, cfg.block, cfg.block)

    for _ in range(max(args.warmup, 3)):
        flush.zero_()
        step()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    step()
    ev1.record()
    torch.cuda.synchronize(dev)
    est_ms = sd.max_over_ranks(ev0.elapsed_time(ev1), dev)
    torch.distributed.barrier()
    block_ms = timed_step_blocks(step, flush, args.steps, dev, min_ms=100.0, est_ms=est_ms)
    torch.distributed.barrier()
    _lib.check_status(dev, "sharded attention")
    ms = sd.max_over_ranks(median(block_ms), dev) / args.steps
    split_dim = 1 if (h1 - h0) < cfg.heads else 0
    whole = sd.gather_shards(out, cfg.batch if split_dim == 0 else cfg.heads, dim=split_dim)
    if rank != 0:
        return None
    flops = wl.attention_flops(n_load, cfg.batch, cfg.heads, cfg.block, cfg.block, cfg.head_dim)
    pairs = sorted({(0, 0), (cfg.batch - 1, cfg.heads - 1), (cfg.batch // 2, cfg.heads // 2), (cfg.batch // 2 + cfg.batch // 4, 1 % cfg.heads)})
    parity = attention_parity(whole, q_h, k_h, v_h, wl.config_mask(cfg), pairs)
    same = bool(torch.equal(whole, full_out_rank0)) if full_out_rank0 is not None else None
    return {"workload": cfg.name, "scaling": "strong", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms,
            "shard": f"batch {b1 - b0} x heads {h1 - h0} per GPU", "load_blocks": n_load, "timed_blocks": len(block_ms),
            "gathered_over_nccl": {"max_abs_vs_fp32_oracle": parity, "batch_head_pairs": [list(x) for x in pairs],
                                   "bit_identical_to_single_gpu_result": same},
            "ok": parity <= PARITY_TOL and same is not False}


def encoder_parity(enc_layers, cfg, x_first_seq, dev, depth_report: bool):
    """Parity of the encoder on sequence 0 of the batch against the fp32 oracle (dense masked attention on the CPU):
    the first layer alone, and - when `depth_report` - the whole stack, with the error of the reference's own fp16 path
    (PyTorch eager on the same GPU: fp16 matmuls, softmax, layer_norm, erf GELU, src/benchmk_end2end.py:31-88) beside it, so that
    the growth of rounding error through the layers is on record for both."""
    import stof_b200
    from oracle import fused as of
    from stof_b200 import workloads as wl
    mask_cpu = wl.config_mask(cfg)
    params = wl.encoder_weights(cfg)
    one = stof_b200.BertEncoder(enc_layers[:1], cfg.heads, cfg.eps, "erf", cfg.block, cfg.block)
    one.set_mask(mask_cpu.to(dev))
    got1 = one(x_first_seq.to(dev)).float().cpu()
    want1 = of.bert_layer(x_first_seq, params[0], mask_cpu.float(), cfg.heads, eps=cfg.eps)
    err1 = (got1 - want1).abs().max().item()
    scale1 = max(1.0, want1.abs().max().item())
    rec = {"max_abs_vs_fp32_oracle": err1, "tolerance": PARITY_TOL * scale1, "output_max_abs": want1.abs().max().item(),
           "of": "layer 1 on sequence 0 (tolerance = 2e-3 x the output magnitude: one fp16 step grows with it)",
           "ok": err1 <= PARITY_TOL * scale1}
    if depth_report:
        full = stof_b200.BertEncoder(enc_layers, cfg.heads, cfg.eps, "erf", cfg.block, cfg.block)
        full.set_mask(mask_cpu.to(dev))
        got = full(x_first_seq.to(dev)).float().cpu()
        want = of.encoder_forward(x_first_seq, params, mask_cpu.float(), cfg.heads, cfg.eps)
        eager = torch_eager_fp16_encoder(x_first_seq.to(dev), enc_layers, mask_cpu.to(dev), cfg.heads, cfg.eps).float().cpu()
        rec["all_layers"] = {"layers": cfg.layers, "max_abs_vs_fp32_oracle": (got - want).abs().max().item(),
                             "mean_abs_vs_fp32_oracle": (got - want).abs().mean().item(),
                             "torch_eager_fp16_max_abs_vs_fp32_oracle": (eager - want).abs().max().item(),
                             "torch_eager_fp16_mean_abs_vs_fp32_oracle": (eager - want).abs().mean().item(),
                             "output_max_abs": want.abs().max().item(),
                             "note": "last layer's output of sequence 0, as the reference's end-to-end check compares it"}
    return rec


def torch_eager_fp16_encoder(x, layers, mask, heads, eps):
    """The reference's PyTorch-native fp16 forward on the GPU (library kernels; a comparison figure for the parity report only)."""
    import torch.nn.functional as F
    B, S, hid = x.shape
    d = hid // heads
    add_mask = (1.0 - mask[:, None].half()) * -10000.0
    h = x
    for w in layers:
        qkv = torch.matmul(h, w.Wqkv) + w.bqkv
        q, k, v = (t.view(B, S, heads, d).permute(0, 2, 1, 3) for t in qkv.chunk(3, dim=-1))
        scores = torch.matmul(q, k.transpose(-2, -1)) / (d ** 0.5) + add_mask
        ctx = torch.matmul(F.softmax(scores, dim=-1), v).permute(0, 2, 1, 3).contiguous().view(B, S, hid)
        h = F.layer_norm(torch.matmul(ctx, w.Wo) + w.bo + h, (hid,), w.g1, w.b1, eps)
        f = F.gelu(torch.matmul(h, w.W1) + w.bi1)
        h = F.layer_norm(torch.matmul(f, w.W2) + w.bi2 + h, (hid,), w.g2, w.b2, eps)
    return h


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
    with ClockSampler(physical_gpu_index(local)) as clocks:
        e0.record()
        for _ in range(steps):
            enc(x)
        e1.record()
        torch.cuda.synchronize(dev)
    if world > 1:
        torch.distributed.barrier()
    _lib.check_status(dev, "encoder timed region")
    my_ms = e0.elapsed_time(e1) / steps
    ms = sd.max_over_ranks(my_ms, dev)
    # per-rank time and SM clock: time x MHz tells a slow-clocked GPU from an uneven split of the work
    mine = torch.tensor([my_ms, float(clocks.summary()["sm_mhz"] or 0)], dtype=torch.float64, device=dev)
    per_rank = [mine.clone() for _ in range(world)]
    if world > 1:
        torch.distributed.all_gather(per_rank, mine)
    if rank != 0:
        return None
    peaks = measured_peaks()
    tflops = wl.encoder_flops(cfg, n_load, cfg.batch) / (ms * 1e-3) / 1e12
    parity = encoder_parity(layers, cfg, wl.encoder_input(cfg, (0, 1)), dev, depth_report=(world == 1 and not args.no_depth_report))
    return {"metric": "BERT encoder tokens/s", "value": cfg.batch * cfg.seq_len / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
            "steps": steps, "warmup": warmup, "scaling": "strong", "workload": cfg.name, "global_batch": cfg.batch, "seq_len": cfg.seq_len,
            "layers": cfg.layers, "load_blocks": n_load, "tflops_all_gpus": tflops,
            "frac_of_sustained_peak_per_gpu": tflops / world / peaks["tflops_sustained"], "gpu_launches": steps * cfg.layers * 6,
            "per_rank": [{"ms_per_step": float(t[0]), "sm_mhz_median": float(t[1]), "ms_x_ghz": float(t[0] * t[1] / 1e3)} for t in per_rank],
            "clocks": clocks.summary(), "parity_first_layer": parity}


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
        "gpu_launches": args.steps * cfg.layers * 6,
        "clocks": clocks.summary(),
        "graph_replay": {"ms_per_step": graph_ms, "value": tokens / (graph_ms * 1e-3), "unit": "tokens/s",
                         "note": "the same forward replayed as one CUDA graph (BertEncoder.capture)"},
    }
    print(json.dumps(line))
    return 0


def run_micro(args, local):
    """Every kernel of the library once over, each on its own at a size where its roofline means something (inputs beyond L2
    for the HBM-bound ones), timed with CUDA events over a loop; prints one JSON object.  This is also the command the ncu
    summaries under profiles/ are taken from (`--only <name>` runs a single entry a few times)."""
    import stof_b200
    from stof_b200 import _lib, workloads as wl
    dev = torch.device("cuda", local)
    peaks = measured_peaks()
    g = torch.Generator().manual_seed(7)
    reps = max(args.steps, 1)

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, generator=g) * scale).half().to(dev)

    def timed(fn):
        for _ in range(max(args.warmup, 1)):
            fn()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        _lib.check_status(dev, "micro")
        return e0.elapsed_time(e1) / reps

    T = args.rows
    out = {}

    def gemm_entry(name, K, N, fn_name, extra=()):
        a, w, b = rnd(T, K), rnd(K, N, scale=0.02), rnd(N)
        y = torch.empty(T, N, dtype=torch.float16, device=dev)
        r = rnd(T, N) if "residual" in fn_name else None
        gam, bet = (rnd(N), rnd(N)) if "layernorm" in fn_name else (None, None)
        f = getattr(stof_b200, fn_name)
        if fn_name == "gemm_bias":
            call = lambda: f(a, w, b, out=y)
        elif fn_name == "gemm_bias_gelu":
            call = lambda: f(a, w, b, "erf", out=y)
        elif fn_name == "gemm_bias_residual":
            call = lambda: f(a, w, b, r, out=y)
        else:
            call = lambda: f(a, w, b, r, gam, bet, 1e-12, out=y)
        ms = timed(call)
        tf = 2.0 * T * K * N / (ms * 1e-3) / 1e12
        out[name] = {"rows": T, "k": K, "n": N, "us": ms * 1e3, "tflops": tf, "frac_of_burst_peak": tf / peaks["tflops"]}

    def ln_entry(name, hidden, residual):
        x = rnd(T, hidden)
        r = rnd(T, hidden) if residual else None
        gam, bet = rnd(hidden), rnd(hidden)
        ms = timed(lambda: stof_b200.bias_residual_layernorm(x, None, r, gam, bet, 1e-12, out=x))
        nbytes = T * hidden * 2 * (3 if residual else 2)
        out[name] = {"rows": T, "hidden": hidden, "us": ms * 1e3, "gbs": nbytes / (ms * 1e-3) / 1e9,
                     "frac_of_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}

    def compaction_entry(name, S):
        mask = wl.expand_block_mask(wl.block_bigbird(S // 64, 1)).to(dev)
        refresher = stof_b200.SparseStorageRefresher(mask, 64, 64)
        eager_ms = timed(refresher.refresh)
        # the two kernels (and the two 16-byte clears before them) replayed as a CUDA graph: no host work between them
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            refresher.refresh()
        torch.cuda.current_stream(dev).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            refresher.refresh()
        ms = timed(graph.replay)
        refresher.check()
        out[name] = {"seq_len": S, "us": ms * 1e3, "gbs": mask.numel() * 2 / (ms * 1e-3) / 1e9,
                     "frac_of_hbm_peak": mask.numel() * 2 / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "eager_us": eager_ms * 1e3,
                     "kernels": "classify_kernel + fill_bounded_kernel, CUDA-graph replay"}

    entries = {
        "gemm_qkv_1024": lambda: gemm_entry("gemm_qkv_1024", 1024, 3072, "gemm_bias"),
        "gemm_outproj_residual_1024": lambda: gemm_entry("gemm_outproj_residual_1024", 1024, 1024, "gemm_bias_residual"),
        "gemm_outproj_layernorm_1024": lambda: gemm_entry("gemm_outproj_layernorm_1024", 1024, 1024, "gemm_bias_residual_layernorm"),
        "gemm_ffn1_gelu_1024": lambda: gemm_entry("gemm_ffn1_gelu_1024", 1024, 4096, "gemm_bias_gelu"),
        "gemm_ffn2_residual_1024": lambda: gemm_entry("gemm_ffn2_residual_1024", 4096, 1024, "gemm_bias_residual"),
        "gemm_ffn2_layernorm_1024": lambda: gemm_entry("gemm_ffn2_layernorm_1024", 4096, 1024, "gemm_bias_residual_layernorm"),
        "gemm_outproj_residual_768": lambda: gemm_entry("gemm_outproj_residual_768", 768, 768, "gemm_bias_residual"),
        "gemm_outproj_layernorm_768": lambda: gemm_entry("gemm_outproj_layernorm_768", 768, 768, "gemm_bias_residual_layernorm"),
        "gemm_one_block_small": lambda: gemm_entry("gemm_one_block_small", 768, 768, "gemm_bias"),
        "layernorm_1024": lambda: ln_entry("layernorm_1024", 1024, False),
        "layernorm_residual_1024": lambda: ln_entry("layernorm_residual_1024", 1024, True),
        "layernorm_768": lambda: ln_entry("layernorm_768", 768, False),
        "compaction_S2048": lambda: compaction_entry("compaction_S2048", 2048),
        "compaction_S4096": lambda: compaction_entry("compaction_S4096", 4096),
    }
    for name, fn in entries.items():
        if args.only and name not in args.only.split(","):
            continue
        if name == "gemm_one_block_small":
            T_saved, T = T, 4096
            fn()
            T = T_saved
        else:
            fn()
    print(json.dumps({"metric": "per-kernel timings", "rows": args.rows, "steps": reps, "peaks": peaks, "kernels": out}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="stof", choices=["stof", "reference"])
    ap.add_argument("--workload", default="attention", choices=["attention", "encoder", "micro"])
    ap.add_argument("--rows", type=int, default=65536, help="micro: rows (tokens) of the GEMM / LayerNorm entries")
    ap.add_argument("--only", default="", help="micro: comma-separated entry names to run (default: all)")
    ap.add_argument("--batch", type=int, default=0, help="override the batch size (profiling aid: smaller captures)")
    ap.add_argument("--no-encoder", action="store_true", help="skip the BERT-large encoder forward that the attention run reports under 'encoder'")
    ap.add_argument("--no-depth-report", action="store_true", help="skip the 24-layer parity figure of the encoder sub-record (a minute of CPU work)")
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
        if args.workload == "micro":
            return run_micro(args, local) if rank == 0 else 0
        return run_encoder(args, rank, world, local)
    finally:
        if world > 1 and torch.distributed.is_initialized():
            torch.distributed.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
