"""Block-masked multi-head attention (host side of `stof_block_attn`)."""
from __future__ import annotations

import math
from collections import OrderedDict

import torch

from . import _lib


_PLAN_CACHE = OrderedDict()
_PLAN_CACHE_MAX = 16


_INDEX_GENERATION = {}               # data pointer of an index tensor -> number of in-place rewrites announced by its owner


def index_rewritten(*tensors):
    """Tells the plan cache that these index tensors were rewritten in place by something torch does not see (a C-ABI
    call such as `stof_mask_compact_static`): their version counters did not move, so the cache key carries a
    generation number per storage that this call advances.  Plans and schedules made from the old contents are then
    never found again (they age out of the caches)."""
    for t in tensors:
        if t is not None:
            _INDEX_GENERATION[t.data_ptr()] = _INDEX_GENERATION.get(t.data_ptr(), 0) + 1


_PAIR_MIN_GAIN = 0.06                # re-pair the halves only when that lowers the estimated cost by at least this share
_PAIR_LOAD_WEIGHT = 0.25             # cost of loading one K/V tile pair, in units of one step of the softmax warps
_HOT_PLANS = set()                   # data pointers of plans that were used more than once (see attention_schedule)


def pair_halves(full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, seq_len: int, block_m: int, block_n: int):
    """Chooses, for `stof_block_attn_plan_paired`, which two 64-row halves of the sequence form each work item.
    The two halves of an item walk their own key-tile lists side by side, so an item takes max(len A, len B) steps and
    loads |A union B| tiles: halves with equally long lists belong together, and among those the ones whose lists agree.
    Greedy matching on cost = steps + `_PAIR_LOAD_WEIGHT` * loads: the halves with the longest lists choose first and
    take the free half that is cheapest to pair with (ties: the neighbour 2t / 2t + 1, then the nearest); then pairs of
    items exchange partners while that lowers the total.
    Takes the index as host sequences or CPU tensors.  Returns (pairs, cost_default, cost_paired); pairs is a list of
    ceil(seq_len / 128) (half, half-or--1) tuples, or None when pairing gains less than `_PAIR_MIN_GAIN`.  Pure host code."""
    import numpy as np
    frp, fci, prp, pci = (np.asarray(t, dtype=np.int64) for t in (full_row_ptr, full_col_idx, part_row_ptr, part_col_idx))
    n_half, n_kt, n_rb = (seq_len + 63) // 64, (seq_len + 63) // 64, seq_len // block_m
    lists = np.zeros((n_half, n_kt), dtype=bool)
    for rb in range(n_rb):
        cols = np.concatenate((fci[frp[rb]:frp[rb + 1]], pci[prp[rb]:prp[rb + 1]]))
        if cols.size == 0:
            continue
        h0, h1 = (rb * block_m) // 64, (rb * block_m + block_m - 1) // 64
        for t in range(block_n // 64 if block_n > 64 else 1):
            lists[h0:h1 + 1, np.minimum((cols * block_n) // 64 + t, n_kt - 1)] = True
    if n_half % 2:                                       # an empty dummy half makes the count even; its partner stays alone
        lists = np.concatenate((lists, np.zeros((1, n_kt), dtype=bool)))
    n = lists.shape[0]
    size = lists.sum(axis=1).astype(np.int64)
    both = lists.astype(np.int64) @ lists.astype(np.int64).T
    union = size[:, None] + size[None, :] - both
    cost = np.maximum(size[:, None], size[None, :]) + _PAIR_LOAD_WEIGHT * union
    cost_default = float(sum(cost[2 * t, 2 * t + 1] for t in range(n // 2)))
    free = np.ones(n, dtype=bool)
    idx = np.arange(n)
    pairs = []
    for a in np.argsort(-size, kind="stable"):
        if not free[a]:
            continue
        free[a] = False
        # cheapest partner first; among equals the default neighbour, then the nearest half
        key = cost[a] * (4 * n) + np.where(idx == (a ^ 1), 0, 2 * np.abs(idx - a) + 1)
        b = int(np.argmin(np.where(free, key, np.inf)))
        free[b] = False
        pairs.append([int(a), b])
    # pairwise exchange: swap partners between two items while that lowers the total
    cost = cost.tolist()                                 # plain lists: the loop below is scalar work
    improved, rounds = True, 0
    while improved and rounds < 16:
        improved, rounds = False, rounds + 1
        for i in range(len(pairs)):
            for j in range(i + 1, len(pairs)):
                (a, b), (c, d) = pairs[i], pairs[j]
                now, swap1, swap2 = cost[a][b] + cost[c][d], cost[a][c] + cost[b][d], cost[a][d] + cost[b][c]
                if swap1 < now - 1e-9 and swap1 <= swap2:
                    pairs[i], pairs[j], improved = [a, c], [b, d], True
                elif swap2 < now - 1e-9:
                    pairs[i], pairs[j], improved = [a, d], [b, c], True
    cost_paired = float(sum(cost[a][b] for a, b in pairs))
    if cost_default == 0 or cost_paired > (1.0 - _PAIR_MIN_GAIN) * cost_default:
        return None, cost_default, cost_paired
    out = []
    for a, b in pairs:
        a, b = (a, b) if a < b else (b, a)
        out.append((a, b if b < n_half else -1))
    out.sort()
    return out, cost_default, cost_paired


def plan_halves(plan, seq_len: int):
    """View of a plan's half table: int32 (items, 2), the first sequence row of the two 64-row halves of each work item
    (-1: no second half)."""
    nqt, maxt = (seq_len + 127) // 128, (seq_len + 63) // 64
    a16 = lambda x: (x + 15) & ~15
    off = 32 + a16(4 * nqt) + a16(8 * nqt) + a16(4 * nqt * maxt) + 64 * nqt * maxt
    return plan[off:off + 8 * nqt].view(torch.int32).view(nqt, 2)


def _build_plan(tensors, pairs, seq_len, block_m, block_n):
    full_row_ptr, full_col_idx, part_row_ptr, part_col_idx = tensors
    dev = full_row_ptr.device
    L = _lib.lib()
    nbytes = int(L.stof_block_attn_plan_bytes(seq_len, block_m, block_n))
    with torch.cuda.device(dev):
        plan = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        common = (seq_len, int(block_m), int(block_n), _lib.ptr(plan), nbytes, _lib.ptr(_lib.status_word(dev)), _lib.current_stream_ptr(dev))
        if pairs is None:
            rc = L.stof_block_attn_plan(_lib.ptr(full_row_ptr), _lib.ptr(full_col_idx), _lib.ptr(part_row_ptr), _lib.ptr(part_col_idx), *common)
        else:
            pairs_dev = torch.tensor(pairs, dtype=torch.int32).reshape(-1).to(dev)
            rc = L.stof_block_attn_plan_paired(_lib.ptr(full_row_ptr), _lib.ptr(full_col_idx), _lib.ptr(part_row_ptr),
                                               _lib.ptr(part_col_idx), _lib.ptr(pairs_dev), *common)
    _lib.check(rc, "stof_block_attn_plan")
    return plan


def attention_plan(full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, seq_len: int, block_m: int, block_n: int,
                   pairing: str = "auto"):
    """Kernel-side plan of a block index (`stof_block_attn_plan`), cached per index: the key holds the four
    index tensors themselves (their storage cannot be recycled while the entry lives) and their versions.
    `pairing`: "auto" builds the default plan at the first use of an index and, at its second use, reads the index back
    once and re-plans with `pair_halves` when that spares tile steps (an index used once is not worth the host read);
    "eager" does so at once, "off" never."""
    tensors = (full_row_ptr, full_col_idx, part_row_ptr, part_col_idx)
    key = _plan_key(tensors, seq_len, block_m, block_n)
    hit = _PLAN_CACHE.get(key)
    if hit is not None:
        _PLAN_CACHE.move_to_end(key)
        if hit[2] or pairing == "off":
            return hit[0]
    elif pairing != "eager":
        return _cache_plan(key, _build_plan(tensors, None, seq_len, block_m, block_n), tensors, False)
    # second use (or "eager"): decide about the pairing, once
    plan = hit[0] if hit is not None else None
    if plan is not None and torch.cuda.is_current_stream_capturing():
        return plan                                          # the decision reads the index back: not inside a graph capture
    pairs = None
    if seq_len > 128 and block_m <= 64:
        pairs, _, _ = pair_halves(*(t.cpu() for t in tensors), seq_len, block_m, block_n)
    if pairs is not None or plan is None:
        plan = _build_plan(tensors, pairs, seq_len, block_m, block_n)
    _HOT_PLANS.add(plan.data_ptr())
    return _cache_plan(key, plan, tensors, True)


def _plan_key(tensors, seq_len, block_m, block_n):
    """Identity of a block index for the plan cache: storage address, torch's version counter, length and the generation that
    `index_rewritten` advances for writes torch does not see."""
    return tuple((t.data_ptr(), t._version, t.numel(), _INDEX_GENERATION.get(t.data_ptr(), 0)) for t in tensors) + \
        (seq_len, block_m, block_n, str(tensors[0].device))


def _cache_plan(key, plan, tensors, decided):
    _PLAN_CACHE[key] = (plan, tensors, decided)
    while len(_PLAN_CACHE) > _PLAN_CACHE_MAX:
        _HOT_PLANS.discard(_PLAN_CACHE.popitem(last=False)[1][0].data_ptr())
    return plan


_SCHED_CACHE = OrderedDict()
_SCHED_OVERHEAD_STEPS = 1.5          # per-item fixed work (prologue, epilogue, pipeline refill) in units of one tile step
_SCHED_GROUP_BH = 40                 # (batch, head) pairs whose K/V are kept together in time (L2 residency)


def lpt_schedule(tile_counts, batch_heads: int, blocks: int):
    """Longest-processing-time deal of the work items (query tile x (batch, head)) to `blocks` thread blocks: items in
    descending cost (tile count + a fixed per-item overhead) each go to the block with the least work so far; inside a
    block the items are then ordered by (batch, head) group, heaviest first.  Returns the int32 table that
    `stof_block_attn_scheduled` takes.  Pure host code (used by `attention_schedule` and tested on the CPU)."""
    import heapq
    nqt = len(tile_counts)
    cost = [float(n) + _SCHED_OVERHEAD_STEPS if n > 0 else 0.25 for n in tile_counts]
    order = sorted(range(nqt), key=lambda t: (-cost[t], t))
    total = nqt * batch_heads
    blocks = max(1, min(int(blocks), total))
    heap = [(0.0, b) for b in range(blocks)]
    lists = [[] for _ in range(blocks)]
    for t in order:
        c = cost[t]
        for bh in range(batch_heads):
            load, b = heapq.heappop(heap)
            lists[b].append((bh // _SCHED_GROUP_BH, -c, bh * nqt + t))
            heapq.heappush(heap, (load + c, b))
    table = [blocks, 0]
    ids = []
    for lst in lists:
        lst.sort()
        ids.extend(x[2] for x in lst)
        table.append(len(ids))
    return torch.tensor(table + ids, dtype=torch.int32), blocks


def attention_schedule(plan, seq_len: int, batch: int, heads: int, eager: bool = False):
    """Balanced deal of the work items for this plan and (batch, heads), cached; None when every item gets its own block
    and, unless `eager`, on the first use of a plan (the table is built at the second use: it costs a small synchronising
    read of the plan's per-tile counts and a few milliseconds of host work)."""
    dev = plan.device
    nqt = (seq_len + 127) // 128
    blocks = 2 * torch.cuda.get_device_properties(dev).multi_processor_count
    if nqt * batch * heads <= blocks:
        return None, 0
    key = (plan.data_ptr(), plan._version, seq_len, batch, heads, str(dev))
    hit = _SCHED_CACHE.get(key)
    if hit is not None:
        _SCHED_CACHE.move_to_end(key)
        if hit[0] is None and not torch.cuda.is_current_stream_capturing():   # second use of this plan and shape: now the table pays off
            counts = plan[32:32 + 4 * nqt].view(torch.int32).cpu().tolist()
            table, blocks = lpt_schedule(counts, batch * heads, blocks)
            hit = _SCHED_CACHE[key] = (table.to(dev), blocks, plan)
        return hit[0], hit[1]
    if not eager or torch.cuda.is_current_stream_capturing():
        # first use: an index that is used once (a caller-supplied row mask, a test) is not worth a host read and a few
        # milliseconds of host work; remember it and run the default deal
        _SCHED_CACHE[key] = (None, 0, plan)
        while len(_SCHED_CACHE) > 4 * _PLAN_CACHE_MAX:
            _SCHED_CACHE.popitem(last=False)
        return None, 0
    counts = plan[32:32 + 4 * nqt].view(torch.int32).cpu().tolist()          # the plan's tile count per query tile
    table, blocks = lpt_schedule(counts, batch * heads, blocks)
    table = table.to(dev)
    _SCHED_CACHE[key] = (table, blocks, plan)
    while len(_SCHED_CACHE) > 4 * _PLAN_CACHE_MAX:
        _SCHED_CACHE.popitem(last=False)
    return table, blocks


def block_attention(q, k, v, out, full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, part_block_mask,
                    load_row_ptr, load_col_idx, block_m: int, block_n: int, num_warps: int = 4, softmax_scale=None):
    """Runs the attention kernel on (B,H,S,64)-shaped *views*: q, k, v and out may be arbitrary
    strided views with a contiguous last dimension (for instance slices of a fused (B,S,3*hidden)
    QKV activation permuted to (B,H,S,64), or a merged-head (B,S,hidden) output viewed the same
    way), so no transposing copy is needed around the kernel.  `out` may be `q` itself.
    `load_row_ptr` / `load_col_idx` are accepted for signature compatibility (they are the merge of
    the full and partial lists, which is what the kernel's plan is built from)."""
    _lib.require_cuda(q, k, v, out, full_row_ptr, part_row_ptr)
    if q.dtype != torch.float16 or k.dtype != torch.float16 or v.dtype != torch.float16 or out.dtype != torch.float16:
        raise _lib.StofError("block attention expects float16 q/k/v/out")
    B, H, S, D = q.shape
    if k.shape != q.shape or v.shape != q.shape or out.shape != q.shape:
        raise _lib.StofError("block attention: q, k, v and out must share one (B,H,S,D) shape")
    for t in (q, k, v, out):
        if t.stride(3) != 1:
            raise _lib.StofError("block attention: the head dimension must be contiguous")
    for t in (full_row_ptr, full_col_idx, part_row_ptr, part_col_idx):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise _lib.StofError("block attention: index tensors must be contiguous int32")
    if full_row_ptr.numel() != S // block_m + 1 or part_row_ptr.numel() != S // block_m + 1:
        raise _lib.StofError("block attention: row pointer arrays must have S / BLOCK_M + 1 entries")
    if part_block_mask is not None and (part_block_mask.dtype != torch.float16 or not part_block_mask.is_contiguous()):
        raise _lib.StofError("block attention: part_block_mask must be contiguous float16")
    scale = 1.0 / math.sqrt(D) if softmax_scale is None else float(softmax_scale)   # src/ops/src/block_attn_mask.cpp:32
    dev = q.device
    L = _lib.lib()
    plan = attention_plan(full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, S, int(block_m), int(block_n))
    schedule, sched_blocks = attention_schedule(plan, S, B, H, eager=plan.data_ptr() in _HOT_PLANS)
    with torch.cuda.device(dev):
        st = _lib.status_word(dev)
        if schedule is None:
            rc = L.stof_block_attn(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), B, H, S, D,
                                   _lib.strides3(q.stride()[:3]), _lib.strides3(k.stride()[:3]),
                                   _lib.strides3(v.stride()[:3]), _lib.strides3(out.stride()[:3]),
                                   _lib.ptr(part_row_ptr), _lib.ptr(part_block_mask), _lib.ptr(plan),
                                   int(block_m), int(block_n), int(num_warps), scale, _lib.ptr(st), _lib.current_stream_ptr(dev))
        else:
            rc = L.stof_block_attn_scheduled(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), B, H, S, D,
                                             _lib.strides3(q.stride()[:3]), _lib.strides3(k.stride()[:3]),
                                             _lib.strides3(v.stride()[:3]), _lib.strides3(out.stride()[:3]),
                                             _lib.ptr(part_row_ptr), _lib.ptr(part_block_mask), _lib.ptr(plan),
                                             int(block_m), int(block_n), int(num_warps), scale, _lib.ptr(schedule), int(sched_blocks),
                                             _lib.ptr(st), _lib.current_stream_ptr(dev))
    _lib.check(rc, "stof_block_attn")
    return out


def block_attn_mask(q, k, v, full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, part_block_mask,
                    load_row_ptr, load_col_idx, BLOCK_M, BLOCK_N, num_warps):
    """Semantics of the reference extension's `block_attn_mask.forward`
    (src/ops/src/block_attn_mask.cpp:17-49): overwrites `q` with the attention output."""
    if not q.is_contiguous():
        raise _lib.StofError("block_attn_mask: q must be contiguous (it is overwritten in place)")
    return block_attention(q, k.contiguous(), v.contiguous(), q, full_row_ptr, full_col_idx, part_row_ptr, part_col_idx,
                           part_block_mask.contiguous(), load_row_ptr, load_col_idx, BLOCK_M, BLOCK_N, num_warps)


def tapered_chunks(batch: int, chunk: int, taper: int):
    """Batch elements per chunk of the host pipeline: full chunks, the last one halved `taper` times (4 -> 2, 1, 1): what
    follows the last host-to-device copy - its kernel and the copy of its result back - is then a small chunk's worth."""
    sizes = [min(chunk, batch - b0) for b0 in range(0, batch, chunk)]
    for _ in range(taper):
        if not sizes or sizes[-1] < 2:
            break
        x = sizes.pop()
        sizes += [x - x // 2, x // 2]
    return sizes


class HostAttentionPipeline:
    """Block-masked attention for q, k, v that live in (pinned) HOST memory: the batch is cut into chunks that go
    through three CUDA streams - host-to-device copies of chunk c+1, the attention kernel on chunk c and the
    device-to-host copy of the result of chunk c-1 run at the same time, so that a call costs about the larger
    of the two PCIe directions instead of their sum plus the kernel.  Device staging (`slots` chunks of q, k, v;
    the output overwrites the q slot, as the reference operator does) is allocated once and reused by later calls
    of the same shape."""

    def __init__(self, device, chunk_batch: int = 2, slots: int = 3, taper: int = 2):
        self.device = torch.device(device)
        self.chunk = int(chunk_batch)
        self.slots = int(slots)
        self.taper = int(taper)
        self._shape = None
        self._stage = None
        self._s_in = torch.cuda.Stream(self.device)
        self._s_run = torch.cuda.Stream(self.device)
        self._s_out = torch.cuda.Stream(self.device)

    def chunk_sizes(self, batch: int):
        return tapered_chunks(batch, self.chunk, self.taper)

    def _staging(self, heads, seq_len, head_dim):
        shape = (self.chunk, heads, seq_len, head_dim)
        if self._shape != shape:
            self._stage = [tuple(torch.empty(shape, dtype=torch.float16, device=self.device) for _ in range(3)) for _ in range(self.slots)]
            self._shape = shape
        return self._stage

    def __call__(self, q_host, k_host, v_host, out_host, full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, part_block_mask,
                 load_row_ptr, load_col_idx, block_m: int, block_n: int, num_warps: int = 4):
        for t in (q_host, k_host, v_host, out_host):
            if t.device.type != "cpu" or t.dtype != torch.float16 or not t.is_contiguous():
                raise _lib.StofError("host attention: q, k, v and out must be contiguous float16 CPU tensors (pinned for overlap)")
        B, H, S, D = q_host.shape
        if k_host.shape != q_host.shape or v_host.shape != q_host.shape or out_host.shape != q_host.shape:
            raise _lib.StofError("host attention: q, k, v and out must share one (B,H,S,D) shape")
        stage = self._staging(H, S, D)
        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        for st in (self._s_in, self._s_run, self._s_out):
            st.wait_event(start)                       # everything enqueued before the call comes first
        slot_free = [None] * self.slots
        last = None
        sizes = self.chunk_sizes(B)
        starts = [sum(sizes[:i]) for i in range(len(sizes))]
        for c, (b0, nb) in enumerate(zip(starts, sizes)):
            qd, kd, vd = (t[:nb] for t in stage[c % self.slots])
            with torch.cuda.stream(self._s_in):
                if slot_free[c % self.slots] is not None:
                    self._s_in.wait_event(slot_free[c % self.slots])      # the slot's previous result has left the device
                qd.copy_(q_host[b0:b0 + nb], non_blocking=True)
                kd.copy_(k_host[b0:b0 + nb], non_blocking=True)
                vd.copy_(v_host[b0:b0 + nb], non_blocking=True)
                loaded = torch.cuda.Event()
                loaded.record(self._s_in)
            with torch.cuda.stream(self._s_run):
                self._s_run.wait_event(loaded)
                block_attention(qd, kd, vd, qd, full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, part_block_mask,
                                load_row_ptr, load_col_idx, block_m, block_n, num_warps)
                computed = torch.cuda.Event()
                computed.record(self._s_run)
            with torch.cuda.stream(self._s_out):
                self._s_out.wait_event(computed)
                out_host[b0:b0 + nb].copy_(qd, non_blocking=True)
                done = torch.cuda.Event()
                done.record(self._s_out)
            slot_free[c % self.slots] = done
            last = done
        if last is not None:
            cur.wait_event(last)                       # the caller's stream sees the whole result (copies leave in order)
        return out_host


_HOST_PIPELINES = {}


def block_attention_host(q_host, k_host, v_host, out_host, full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, part_block_mask,
                         load_row_ptr, load_col_idx, block_m: int, block_n: int, num_warps: int = 4, chunk_batch=None):
    """`block_attn_mask` for host-resident q, k, v: result in `out_host` (may be `q_host`), copies overlapped with
    the kernel by a per-device `HostAttentionPipeline`.  The block index tensors are device tensors, as for the
    device-side operator (src/ops/package_op.py:50-74).  `chunk_batch` defaults to a quarter of the batch: four chunks keep
    the copy engines busy in both directions while the per-chunk host work (copies, events, one launch) stays small."""
    if chunk_batch is None:
        chunk_batch = max(1, (q_host.shape[0] + 3) // 4)
    dev = full_row_ptr.device
    key = (str(dev), int(chunk_batch))
    pipe = _HOST_PIPELINES.get(key)
    if pipe is None:
        pipe = _HOST_PIPELINES[key] = HostAttentionPipeline(dev, chunk_batch)
    return pipe(q_host, k_host, v_host, out_host, full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, part_block_mask,
                load_row_ptr, load_col_idx, block_m, block_n, num_warps)
