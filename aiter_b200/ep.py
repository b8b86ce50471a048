"""Expert parallelism for the fused-MoE layer: one process per GPU, NCCL over NVLink/NVSwitch.

Rank r owns experts [r*E/G, (r+1)*E/G) and token rows [r*M/G, (r+1)*M/G).  One exchange on each
side of the local layer:

  1. 1x128-quantise the local rows, all-gather the e4m3 codes, their fp32 scales and the routing
     (ids + weights), so every rank holds all M rows in 1 byte per element;
  2. fused_moe stages on all rows with ``expert_mask`` = this rank's experts and global ids: the
     sort drops non-local routes, stage 2 leaves an fp32 partial sum [M, H];
  3. reduce-scatter(sum) of the fp32 partials, then the single final rounding to bf16 on the
     rank's own rows.

Reducing in fp32 keeps the result equal to the single-GPU one up to fp32 summation order.  The
reference reaches the same end with an all-to-all dispatch/combine
(op_tests/multigpu_tests/test_dispatch_combine.py:75-177, oracle run_ref :18-72).

With ``exchange="p2p"`` both exchanges go over NVLink peer memory (CUDA IPC mappings, plain peer stores) and
ship only rows that are needed: step 1 stores a token's quantised row into the buffers of the ranks that hold
one of its experts (the small routing table is still all-gathered, which doubles as the barrier), step 3 pushes
the partial rows a rank really produced into the owning rank's memory, runs a tiny all-reduce as the barrier,
and a combine kernel adds what arrived in a fixed rank order. With DeepSeek-V3's group-limited routing a token
has routes on at most half of 8 ranks, so half of the rows of the dense collectives do not travel.

The collectives go through ``torch.distributed`` so the same code runs on gloo/CPU ranks for the
host-logic tests; ``local_layer`` is injectable for that purpose.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from . import _lib, dtypes
from .enums import QuantType
from .fused_moe import _mark, fused_moe_stages, per_group_quant_hip, per_token_quant_hip


_MASKS: dict = {}


def expert_mask_for_rank(num_experts: int, rank: int, world: int, device=None, expert_rank=None) -> torch.Tensor:
    """[global_E] int32, 1 for the experts owned by ``rank``: the contiguous slice [rank*E/G, (rank+1)*E/G), or the
    entries of ``expert_rank`` ([global_E] int32, owning rank per expert) equal to ``rank``. The sort numbers the
    local experts in ascending global id, which is the order the rank's weight slices must have
    (``local_experts_of``)."""
    if expert_rank is not None:
        return (expert_rank.to(device) == rank).to(torch.int32)
    if num_experts % world != 0:
        raise ValueError(f"num_experts ({num_experts}) must be divisible by the EP world size ({world})")
    key = (num_experts, rank, world, str(device))
    mask = _MASKS.get(key)
    if mask is None:   # built once per layout: two launches less on every layer call
        per = num_experts // world
        mask = torch.zeros(num_experts, dtype=torch.int32, device=device)
        mask[rank * per:(rank + 1) * per] = 1
        _MASKS[key] = mask
    return mask


def balanced_expert_placement(route_counts, world: int, method: str = "swap", tolerance: float = 0.02) -> torch.Tensor:
    """Expert -> rank table [E] int32 with E/world experts per rank and the per-rank route totals levelled, from
    ``route_counts`` (routes per expert on a calibration batch). What a weight loader would run once, from routing
    statistics, to place the experts; contiguous slices leave the hottest rank 1.4x above the mean on the
    DeepSeek-V3 benchmark routing.

    ``method="lpt"``: experts in descending order of their counts each go to the rank with the smallest total that
    still has a free slot. Levels best, but scatters the experts of a routing group over all ranks, so a token with
    group-limited routing then has routes on more ranks and more rows travel in dispatch and combine.
    ``method="swap"``: starts from the contiguous slices (one routing group per rank when groups == ranks) and
    exchanges one expert of the most loaded rank with one of another rank, the pair that levels those two ranks best,
    until the most loaded rank is within ``tolerance`` of the mean or no exchange helps: the fewest experts leave
    their group."""
    counts = torch.as_tensor(route_counts).to(torch.int64).cpu()
    E = counts.numel()
    if E % world != 0:
        raise ValueError(f"num_experts ({E}) must be divisible by the EP world size ({world})")
    per = E // world
    if method == "lpt":
        load = [0] * world
        free = [per] * world
        table = torch.empty(E, dtype=torch.int32)
        for e in torch.argsort(counts, descending=True, stable=True).tolist():
            r = min((r for r in range(world) if free[r] > 0), key=lambda r: (load[r], r))
            table[e] = r
            load[r] += int(counts[e])
            free[r] -= 1
        return table
    if method != "swap":
        raise ValueError(f"method must be 'lpt' or 'swap', got {method!r}")
    c = counts.tolist()
    owner = [e // per for e in range(E)]
    load = [sum(c[r * per:(r + 1) * per]) for r in range(world)]
    mean = sum(load) / world
    for _ in range(4 * E):
        hi = max(range(world), key=lambda r: (load[r], -r))
        if load[hi] <= mean * (1.0 + tolerance):
            break
        best = None   # (resulting max of the two ranks, expert of hi, expert of the other rank)
        for lo in range(world):
            if lo == hi or load[lo] >= load[hi]:
                continue
            gap = load[hi] - load[lo]
            for a in (e for e in range(E) if owner[e] == hi):
                for b in (e for e in range(E) if owner[e] == lo):
                    d = c[a] - c[b]
                    if 0 < d < gap:
                        after = max(load[hi] - d, load[lo] + d)
                        if best is None or after < best[0]:
                            best = (after, a, b)
        if best is None:
            break
        _, a, b = best
        lo = owner[b]
        d = c[a] - c[b]
        owner[a], owner[b] = lo, hi
        load[hi] -= d
        load[lo] += d
    return torch.tensor(owner, dtype=torch.int32)


def local_experts_of(expert_rank, rank: int) -> torch.Tensor:
    """Global ids of the experts ``rank`` owns under ``expert_rank``, ascending: local expert i of that rank."""
    return torch.nonzero(torch.as_tensor(expert_rank).cpu() == rank).flatten()


def _gpu_local_layer(a1, a1_scale, w1, w2, topk_weight, topk_ids, expert_mask, w1_scale, w2_scale, timers=None,
                     chunks=1, on_chunk=None, sm_margin=0, quant_type=QuantType.per_1x128, ranges=1):
    """All rows, local experts -> fp32 partial [M, H] (or [chunks, M, H/chunks]); no final rounding."""
    return fused_moe_stages(a1, w1, w2, topk_weight, topk_ids, expert_mask, w1_scale, w2_scale,
                            a1_scale, None, None, timers=timers, stage2_chunks=chunks, on_chunk=on_chunk,
                            sm_margin=sm_margin, quant_type=quant_type, stage2_ranges=ranges)


def _gpu_quant(x, quant_type=QuantType.per_1x128):
    if QuantType(quant_type) == QuantType.per_Token:
        return per_token_quant_hip(x, quant_dtype=dtypes.fp8)
    return per_group_quant_hip(x, quant_dtype=dtypes.fp8)


def _gpu_finalize(acc, dtype):
    out = torch.empty(acc.shape, dtype=dtype, device=acc.device)
    _lib.call("b200_moe_finalize", out, acc, device=acc.device)
    return out


_STREAMS: dict = {}


def _side_streams(device):
    """(high-priority stream for the GEMM launches, stream for the pushes) of ``device``, created once."""
    key = device.index
    if key not in _STREAMS:
        _STREAMS[key] = (torch.cuda.Stream(device=device, priority=-1), torch.cuda.Stream(device=device))
    return _STREAMS[key]


class PeerExchange:
    """Buffers for the peer-memory exchange, one set per (process group, rows per rank, model_dim).

    Every rank allocates ONE arena holding recv [world, m_local, H] fp32 (partial rows pushed to it), a1
    [M, H] e4m3 and a1_scale [M, H/128] fp32 (token rows dispatched to it), exports the allocation through CUDA
    IPC, maps the arenas of all other ranks and keeps the addresses of the three buffers on every rank in device
    arrays for the kernels. Built once, on first use; building it is a collective call (all ranks of the group
    must reach it)."""

    _cache: dict = {}
    # (device index, 64-byte IPC handle) -> mapped base address. torch's allocator carves several tensors out of one
    # cudaMalloc segment; two arenas in one segment export the SAME handle (with different offsets), and a process may
    # open a handle only once, so mappings are shared between exchanges and closed together in clear().
    _opened: dict = {}

    def __init__(self, group, m_local, H, device):
        import ctypes
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        self.device = device
        M, kb = world * m_local, H // 128
        align = lambda n: (n + 255) // 256 * 256
        off_recv, off_a1 = 0, align(world * m_local * H * 4)
        off_a1s = off_a1 + align(M * H)
        total = off_a1s + align(M * kb * 4)
        self.arena = torch.empty((total,), dtype=torch.uint8, device=device)
        self.recv = self.arena[off_recv:off_recv + world * m_local * H * 4].view(torch.float32).view(world, m_local, H)
        self.a1 = self.arena[off_a1:off_a1 + M * H].view(torch.float8_e4m3fn).view(M, H)
        self.a1_scale = self.arena[off_a1s:off_a1s + M * kb * 4].view(torch.float32).view(M, kb)
        self.flag = torch.zeros(1, dtype=torch.int32, device=device)
        # Export, exchange, map. A failure on any rank (no IPC in this environment, no peer access) is agreed on
        # by all ranks before anybody raises, so that callers can fall back to the NCCL exchange together.
        handle = ctypes.create_string_buffer(64)
        offset = ctypes.c_int64(0)
        err = None
        try:
            _lib.call_plain("b200_ep_ipc_export", ctypes.byref(_lib.to_aiter(self.arena)), handle, ctypes.byref(offset))
        except RuntimeError as e:
            err = str(e)
        exported = [None] * world
        dist.all_gather_object(exported, (handle.raw, int(offset.value), err), group=group)
        # every peer's arena is mapped with THIS rank's device current: a mapping belongs to the device it was
        # opened under, and the kernels of this rank are what store through it
        self.mapped = []
        bases = []
        if all(e[2] is None for e in exported):
            try:
                for r in range(world):
                    if r == rank:
                        bases.append(self.arena.data_ptr())
                        continue
                    key = (int(device.index), bytes(exported[r][0]))
                    if key not in PeerExchange._opened:
                        base = ctypes.c_int64(0)
                        _lib.call_plain("b200_ep_ipc_open", ctypes.create_string_buffer(exported[r][0], 64),
                                        int(device.index), ctypes.byref(base))
                        PeerExchange._opened[key] = int(base.value)
                    bases.append(PeerExchange._opened[key] + exported[r][1])
            except RuntimeError as e:
                err = str(e)
        else:
            err = next(e[2] for e in exported if e[2] is not None)
        ok = torch.tensor([0 if err else 1], dtype=torch.int32, device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok.item()) == 0:
            self.close()
            raise RuntimeError(f"peer-memory exchange unavailable: {err or 'mapping failed on another rank'}")
        table = lambda off: torch.tensor([b + off for b in bases], dtype=torch.int64, device=device)
        self.ptrs_recv, self.ptrs_a1, self.ptrs_a1_scale = table(off_recv), table(off_a1), table(off_a1s)

    def close(self):
        """Mappings are shared between exchanges (see ``_opened``) and are closed by ``clear()``."""
        self.mapped = []

    @classmethod
    def get(cls, group, m_local, H, device):
        # keyed by the group's member ranks, not by the object's id (which a later group can reuse)
        key = (tuple(dist.get_process_group_ranks(group if group is not None else dist.group.WORLD)), m_local, H,
               device.index)
        if key not in cls._cache:
            cls._cache[key] = cls(group, m_local, H, device)
        return cls._cache[key]

    @classmethod
    def clear(cls):
        """Unmaps every peer arena and drops the cache. Call it before ``destroy_process_group`` (a collective point:
        no kernel of any rank may still be storing into a mapping that is being closed)."""
        for ex in cls._cache.values():
            ex.close()
        cls._cache.clear()
        for (dev_index, _handle), base in cls._opened.items():
            _lib.call_plain("b200_ep_ipc_close", base, dev_index)
        cls._opened.clear()


def _p2p_combine(ex, partial, ids, num_experts, group, dtype, timers, expert_rank=None, pushed=False):
    """partial [M, H] fp32 of this rank -> out [M/G, H]: push (unless the caller pushed the column ranges already),
    barrier, combine."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    M, H = partial.shape
    m_local = M // world
    epr = num_experts // world
    if not pushed:
        _lib.call("b200_ep_push_partials", partial, ids, ex.ptrs_recv, rank, world, epr, expert_rank, 0, 0, 0,
                  device=partial.device)
    _mark(timers, "ep_barrier")
    dist.all_reduce(ex.flag, group=group)   # passes only after every rank's push kernel has completed
    _mark(timers, "ep_combine")
    out = torch.empty((m_local, H), dtype=dtype, device=partial.device)
    _lib.call("b200_ep_combine", out, partial, ex.recv, ids, rank, world, epr, expert_rank, device=partial.device)
    return out


def ep_fused_moe(x_local, w1_local, w2_local, topk_weight_local, topk_ids_local, w1_scale_local,
                 w2_scale_local, num_experts, group=None, dtype=torch.bfloat16,
                 quant=_gpu_quant, local_layer=_gpu_local_layer, finalize=_gpu_finalize, timers=None,
                 overlap_chunks=None, sm_margin=16, exchange="nccl", quant_type=QuantType.per_1x128, expert_rank=None):
    """x_local [M/G, H] bf16, routing [M/G, topk] with GLOBAL expert ids -> out [M/G, H].

    Every rank must pass the same number of rows. With the NCCL exchange and ``overlap_chunks`` > 1 stage 2 runs in
    that many column ranges and the reduce-scatter of a finished range is issued beside the computation of the next;
    ``sm_margin`` SMs are kept free for NCCL during those launches. Off by default: on 8 B200s four ranges
    of 59 MB took as long in total as one 235 MB reduce-scatter after the unsplit stage 2 (1.47 vs 1.40 ms).
    With ``exchange="p2p"`` and ``overlap_chunks`` > 1 stage 2 fills the partial in that many column ranges and the push of
    a finished range runs beside the next range, on the ``sm_margin`` SMs that launch leaves idle (the local-layer
    timers are not recorded in this mode).
    ``exchange``: "nccl" = fp32 reduce-scatter of the partials; "p2p" = push of the produced rows into the
    owner's memory + combine (see the module docstring; the first call builds the IPC mappings).
    ``expert_rank``: optional [num_experts] int32 device tensor, the rank that owns each expert (a placement from
    ``balanced_expert_placement``); the rank's weights are then its experts in ascending global id. Default:
    contiguous slices.
    ``quant_type``: per_1x128 / per_128x128 (both exchanges) or per_Token (NCCL exchange: one scale per row travels
    with the codes)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    m_local, H = x_local.shape
    topk = topk_ids_local.shape[1]
    dev = x_local.device
    quant_type = QuantType(quant_type)
    if quant_type == QuantType.per_128x128:
        quant_type = QuantType.per_1x128
    if quant_type not in (QuantType.per_1x128, QuantType.per_Token):
        raise NotImplementedError(f"ep_fused_moe: quant_type={quant_type!r} is not supported (per_1x128, per_Token)")
    if quant_type == QuantType.per_Token and exchange == "p2p":
        raise NotImplementedError("ep_fused_moe: the peer-memory exchange carries 1x128 scales; use exchange='nccl' "
                                  "with QuantType.per_Token")
    layer_kw = {} if quant_type == QuantType.per_1x128 else {"quant_type": quant_type}
    ex = None
    if exchange not in ("nccl", "p2p"):
        raise ValueError(f"exchange must be 'nccl' or 'p2p', got {exchange!r}")
    # peer-memory exchange with the library's own quantiser: one kernel quantises a row and stores it on the ranks
    # that need it (the quantised row never exists here unless this rank is one of them)
    fused_dispatch = (world > 1 and exchange == "p2p" and quant is _gpu_quant
                      and x_local.dtype in (dtypes.bf16, dtypes.fp16))
    _mark(timers, "ep_quant")
    if not fused_dispatch:
        a1_l, a1s_l = quant(x_local) if quant_type == QuantType.per_1x128 else quant(x_local, quant_type)
        a1s_l = a1s_l.view(m_local, -1)
    _mark(timers, "ep_all_gather")
    if world == 1:
        a1, a1s, ids, wts = a1_l, a1s_l, topk_ids_local, topk_weight_local
    elif exchange == "p2p":
        # token rows go only to the ranks that hold one of their experts (peer stores); the routing table of all
        # tokens is small and is all-gathered - a collective issued after the dispatch kernel, so passing it also
        # means every rank's rows have landed
        ex = PeerExchange.get(group, m_local, H, dev)
        ids_l = topk_ids_local.contiguous()
        if fused_dispatch:
            _lib.call("b200_ep_quant_dispatch", x_local.contiguous(), ids_l, ex.ptrs_a1, ex.ptrs_a1_scale, rank, world,
                      num_experts // world, expert_rank, device=dev)
        else:
            _lib.call("b200_ep_dispatch", a1_l, a1s_l.view(m_local, -1), ids_l, ex.ptrs_a1, ex.ptrs_a1_scale, rank, world,
                      num_experts // world, expert_rank, device=dev)
        side_l = torch.cat([ids_l.view(torch.int32), topk_weight_local.contiguous().view(torch.int32)], dim=1)
        side = torch.empty((world * m_local, side_l.shape[1]), dtype=torch.int32, device=dev)
        dist.all_gather_into_tensor(side, side_l, group=group)
        a1, a1s = ex.a1, ex.a1_scale
        ids = side[:, :topk].contiguous()
        wts = side[:, topk:].contiguous().view(torch.float32)
    else:
        # two collectives: the codes, and one int32 side buffer per row with scales, ids and weights
        kb = a1s_l.shape[1]
        side_l = torch.cat([a1s_l.view(torch.int32), topk_ids_local.view(torch.int32),
                            topk_weight_local.contiguous().view(torch.int32)], dim=1)
        a1 = torch.empty((world * m_local, H), dtype=torch.uint8, device=dev)
        side = torch.empty((world * m_local, side_l.shape[1]), dtype=torch.int32, device=dev)
        dist.all_gather_into_tensor(a1, a1_l.view(torch.uint8), group=group)
        dist.all_gather_into_tensor(side, side_l, group=group)
        a1 = a1.view(torch.float8_e4m3fn)
        a1s = side[:, :kb].contiguous().view(torch.float32)
        ids = side[:, kb:kb + topk].contiguous()
        wts = side[:, kb + topk:].contiguous().view(torch.float32)
    mask = expert_mask_for_rank(num_experts, rank, world, device=dev, expert_rank=expert_rank)
    if overlap_chunks is None:
        overlap_chunks = 1   # measured on 8 x B200: the ranged reduce-scatters gain nothing over one call
    if overlap_chunks > 1 and ex is not None:
        # Peer-memory exchange: stage 2 fills the [M, H] partial in column ranges and the push of a finished range
        # runs beside the next range. The GEMM launches go to a high-priority stream, so that when a range's push and
        # the next range's GEMM become ready together the GEMM's CTAs are placed first and the push takes the SMs
        # that launch leaves idle (a GEMM CTA needs a whole SM; behind resident push CTAs it would wait for them).
        main = torch.cuda.current_stream(dev)
        gemm_stream, push_stream = _side_streams(dev)
        epr = num_experts // world

        def on_range(c, block):
            acc, c0, c1 = block
            push_stream.wait_stream(gemm_stream)
            with torch.cuda.stream(push_stream):
                _lib.call("b200_ep_push_partials", acc, ids, ex.ptrs_recv, rank, world, epr, expert_rank, c0, c1,
                          sm_margin if c + 1 < overlap_chunks else 0, device=dev)

        gemm_stream.wait_stream(main)
        with torch.cuda.stream(gemm_stream):
            partial = local_layer(a1, a1s, w1_local, w2_local, wts, ids, mask, w1_scale_local, w2_scale_local,
                                  ranges=overlap_chunks, on_chunk=on_range, sm_margin=sm_margin, **layer_kw)
        main.wait_stream(gemm_stream)
        main.wait_stream(push_stream)
        _mark(timers, "ep_push")
        out = _p2p_combine(ex, partial, ids, num_experts, group, dtype, timers, expert_rank, pushed=True)
        _mark(timers, "end")
        return out
    if overlap_chunks > 1:
        # column ranges: the reduce-scatter of range c runs (on NCCL's stream) beside stage 2 of range c+1
        hc = H // overlap_chunks
        mine = torch.empty((overlap_chunks, m_local, hc), dtype=torch.float32, device=dev)
        works = []

        def on_chunk(c, block):
            works.append(dist.reduce_scatter_tensor(mine[c], block, op=dist.ReduceOp.SUM, group=group,
                                                    async_op=True))

        partial = local_layer(a1, a1s, w1_local, w2_local, wts, ids, mask, w1_scale_local, w2_scale_local,
                              timers=timers, chunks=overlap_chunks, on_chunk=on_chunk, sm_margin=sm_margin, **layer_kw)
        if timers is not None:
            timers.pop()
        _mark(timers, "ep_reduce_scatter")
        for w in works:
            w.wait()
        _mark(timers, "ep_finalize")
        out = finalize(mine.view(overlap_chunks * m_local, hc), dtype)
        out = out.view(overlap_chunks, m_local, hc).permute(1, 0, 2).reshape(m_local, H)
        _mark(timers, "end")
        del partial
        return out
    if timers is not None:
        partial = local_layer(a1, a1s, w1_local, w2_local, wts, ids, mask, w1_scale_local, w2_scale_local,
                              timers=timers, **layer_kw)
        timers.pop()   # the local layer's own "end" mark: the next mark takes its place
    else:
        partial = local_layer(a1, a1s, w1_local, w2_local, wts, ids, mask, w1_scale_local, w2_scale_local, **layer_kw)
    if ex is not None:
        _mark(timers, "ep_push")
        out = _p2p_combine(ex, partial, ids, num_experts, group, dtype, timers, expert_rank)
        _mark(timers, "end")
        return out
    _mark(timers, "ep_reduce_scatter")
    if world == 1:
        mine = partial
    else:
        mine = torch.empty((m_local, H), dtype=torch.float32, device=dev)
        dist.reduce_scatter_tensor(mine, partial, op=dist.ReduceOp.SUM, group=group)
    _mark(timers, "ep_finalize")
    out = finalize(mine, dtype)
    _mark(timers, "end")
    return out
