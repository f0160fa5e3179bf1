"""Expert-parallel layer: the experts of a MoE layer split contiguously over the ranks of a process group.

Each rank keeps the planes of its own experts only; its device table marks the others level 0, which the kernels
already treat as "not resident here, contributes nothing" (the reference's hook: sm120/nqmoe.cu:393,727,1026-1030).
Two exchange patterns, both over torch.distributed (NCCL on GPUs, gloo in the CPU tests):

  decode(x, sel, rw)    tokens replicated on every rank (1..32 tokens): local layer call, then an all-reduce of the
                        [B, H] partial outputs - what the reference's evaluation harness does with all-gather +
                        reduce-scatter (sm120/eval/eval_reg.py:137-142,181); latency-bound, tiny messages.
  prefill(x, sel, rw)   tokens sharded (each rank owns T_r tokens): dispatch = all-to-all of each token row to every
                        rank that owns one of its picked experts (once per destination rank, not once per pick), with
                        its picks masked to that rank; local prefill on the received rows; combine = the owner adds
                        the partial rows in rank order (deterministic).  On NVLink-connected GPUs the partial rows stay
                        where they were computed, in a symmetric-memory buffer, and the owner's combine kernel
                        (nq_ep_combine) reads them from the peers directly; otherwise (gloo, no peer access, more rows
                        than the buffer holds) they come back by an all-to-all and an indexed add.

The local layer is any object with .E, .H, __call__(x, sel, rw) and .prefill(x, sel, rw) - nestquant_b200.moe.MoELayer on a
GPU; the CPU tests plug in a stand-in to check the exchange logic without a device.
"""
import torch
import torch.distributed as dist


def owned_experts(E, world, rank):
    per = (E + world - 1) // world
    return range(rank * per, min(E, (rank + 1) * per))


def _has_alltoall(group):
    return dist.get_backend(group) != "gloo"        # gloo has neither all_to_all nor all_to_all_single


def _all_to_all(out_splits, inp, in_splits, group):
    """variable-size all-to-all along dim 0 (point-to-point sends where the backend has no all-to-all)"""
    out = inp.new_empty((sum(out_splits),) + tuple(inp.shape[1:]))
    if _has_alltoall(group):
        dist.all_to_all_single(out, inp.contiguous(), out_splits, in_splits, group=group)
        return out
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    ins, outs = [t.contiguous() for t in inp.split(in_splits)], list(out.split(out_splits))
    outs[rank].copy_(ins[rank])
    reqs = []
    for d in range(world):
        if d != rank:
            if out_splits[d]:
                reqs.append(dist.irecv(outs[d], src=dist.get_global_rank(group, d) if group is not None else d, group=group))
            if in_splits[d]:
                reqs.append(dist.isend(ins[d], dst=dist.get_global_rank(group, d) if group is not None else d, group=group))
    for r in reqs:
        r.wait()
    return out


def _exchange_counts(counts, group):
    """counts[d] = rows this rank sends to rank d  ->  the whole matrix m[src][dst] as nested lists (host)"""
    world = dist.get_world_size(group)
    allc = [torch.empty_like(counts) for _ in range(world)]
    dist.all_gather(allc, counts, group=group)
    return torch.stack(allc).cpu().tolist()


class _PeerRows:
    """symmetric-memory buffer [rows, H] fp32 per rank for the partial rows of the prefill, with every rank's address"""

    def __init__(s, rows, H, dev, group):
        import torch.distributed._symmetric_memory as symm
        s.buf = symm.empty(rows, H, dtype=torch.float32, device=dev)
        s.hdl = symm.rendezvous(s.buf, group if group is not None else dist.group.WORLD)
        s.rows = rows
        s.ptrs = [int(p) for p in s.hdl.buffer_ptrs]

    def barrier(s):
        s.hdl.barrier()


class EPLayer:
    def __init__(s, local_layer, rank=None, world=None, group=None, peer_rows=0):
        """peer_rows > 0: keep up to that many partial rows per rank in symmetric memory and combine over peer loads
        (NCCL groups on peer-connected GPUs only; silently off where symmetric memory cannot be set up)."""
        s.L, s.group = local_layer, group
        s.rank = dist.get_rank(group) if rank is None else rank
        s.world = dist.get_world_size(group) if world is None else world
        s.E, s.H = local_layer.E, local_layer.H
        s.per = (s.E + s.world - 1) // s.world
        s.last_stats = {}
        s.peer = None
        if peer_rows > 0 and s.world > 1 and s.world <= 8 and _has_alltoall(group):
            ok = torch.ones(1, dtype=torch.int32, device=local_layer.table.device)
            try:
                s.peer = _PeerRows(peer_rows, s.H, local_layer.table.device, group)
            except Exception as e:                      # no peer access / no symmetric memory on this system
                s.peer_error = repr(e)
                ok.zero_()
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)       # all ranks take the same path
            if int(ok) == 0:
                s.peer = None

    # ---- 1..32 replicated tokens
    def decode(s, x, sel, rw, out=None):
        y = s.L(x, sel, rw) if out is None else s.L(x, sel, rw, out=out)
        if s.world > 1:
            dist.all_reduce(y, group=s.group)
        return y

    # ---- sharded tokens
    def prefill(s, x, sel, rw):
        """x fp16 [T_r, H], sel int64 [T_r, topk], rw fp16 [T_r, topk] (this rank's tokens) -> fp32 [T_r, H]"""
        if s.world == 1:
            return s.L.prefill(x, sel, rw)
        T, k = sel.shape
        dev = x.device
        owner = torch.div(sel, s.per, rounding_mode="floor")                       # [T, k] destination rank of each pick
        idx, send_x, send_sel, send_rw = [], [], [], []
        for d in range(s.world):
            mine = owner == d
            rows = torch.nonzero(mine.any(1)).reshape(-1)
            idx.append(rows)
            send_x.append(x[rows])
            send_sel.append(sel[rows])
            send_rw.append(torch.where(mine[rows], rw[rows], torch.zeros_like(rw[rows])))   # picks of other ranks: weight 0
        in_splits = [int(r.numel()) for r in idx]
        m = _exchange_counts(torch.tensor(in_splits, dtype=torch.int64, device=dev), s.group)            # host sync: split sizes
        out_splits = [int(m[src][s.rank]) for src in range(s.world)]
        xr = _all_to_all(out_splits, torch.cat(send_x), in_splits, s.group)
        selr = _all_to_all(out_splits, torch.cat(send_sel), in_splits, s.group)
        rwr = _all_to_all(out_splits, torch.cat(send_rw), in_splits, s.group)
        s.last_stats = dict(sent_rows=sum(in_splits), recv_rows=sum(out_splits), dispatch_bytes=sum(in_splits) * s.H * 2,
                            combine_bytes=sum(out_splits) * s.H * 4)
        nrecv = sum(out_splits)
        if s.peer is not None and max(sum(int(m[src][d]) for src in range(s.world)) for d in range(s.world)) <= s.peer.rows:
            # partial rows stay in this rank's symmetric buffer; every owner reads what it needs from its peers
            from .capi import check, lib
            import ctypes as C
            if nrecv:
                s.L.prefill(xr, selr, rwr, out=s.peer.buf[:nrecv])
            rows = torch.full((s.world, T), -1, dtype=torch.int32, device=dev)
            for d in range(s.world):
                if in_splits[d]:                                                   # my rows sit after those of the ranks before me
                    first = sum(int(m[src][d]) for src in range(s.rank))
                    rows[d, idx[d]] = torch.arange(first, first + in_splits[d], dtype=torch.int32, device=dev)
            out = torch.empty(T, s.H, dtype=torch.float32, device=dev)
            s.peer.barrier()                                                       # every rank's partial rows are complete
            ptrs = (C.c_void_p * s.world)(*s.peer.ptrs)
            check(lib().nq_ep_combine(out.data_ptr(), ptrs, rows.data_ptr(), T, s.H, s.world, torch.cuda.current_stream(dev).cuda_stream),
                  "ep_combine")
            s.peer.barrier()                                                       # buffers may be overwritten from here on
            s.last_stats["combine"] = "peer loads"
            return out
        part = s.L.prefill(xr, selr, rwr) if xr.shape[0] else torch.zeros(0, s.H, dtype=torch.float32, device=dev)
        back = _all_to_all(in_splits, part, out_splits, s.group)                   # partial rows return to their owners
        s.last_stats["combine"] = "all-to-all"
        out = torch.zeros(T, s.H, dtype=torch.float32, device=dev)
        o = 0
        for d in range(s.world):                                                   # fixed rank order: repeatable sums
            n = in_splits[d]
            if n:
                out.index_add_(0, idx[d], back[o:o + n])
            o += n
        return out
