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
    """symmetric-memory buffers per rank, with every rank's address: partial rows [rows, H] fp32 of the prefill and the
    rank's own input rows [rows_x, H] fp16"""

    def __init__(s, rows, H, dev, group, world):
        import torch.distributed._symmetric_memory as symm
        g = group if group is not None else dist.group.WORLD
        s.buf = symm.empty(rows, H, dtype=torch.float32, device=dev)
        s.hdl = symm.rendezvous(s.buf, g)
        s.rows = rows
        s.ptrs = [int(p) for p in s.hdl.buffer_ptrs]
        s.rows_x = (rows + world - 1) // world
        s.xbuf = symm.empty(s.rows_x, H, dtype=torch.float16, device=dev)
        s.xhdl = symm.rendezvous(s.xbuf, g)
        s.xptrs = [int(p) for p in s.xhdl.buffer_ptrs]
        s.xstage = None
        # decode: two alternating [32, H] fp32 buffers for the partial outputs
        s.dec, s.dec_hdl, s.dec_ptrs, s.dec_turn = [], [], [], 0
        for _ in range(2):
            b = symm.empty(32, H, dtype=torch.float32, device=dev)
            h = symm.rendezvous(b, g)
            s.dec.append(b); s.dec_hdl.append(h); s.dec_ptrs.append([int(p) for p in h.buffer_ptrs])
        s.dec_rows = {}

    def barrier(s):
        s.hdl.barrier()


class EPLayer:
    def __init__(s, local_layer, rank=None, world=None, group=None, peer_rows=0, peer_decode=False):
        """peer_rows > 0: keep up to that many partial rows per rank in symmetric memory and combine over peer loads
        (NCCL groups on peer-connected GPUs only; silently off where symmetric memory cannot be set up)."""
        s.L, s.group = local_layer, group
        s.rank = dist.get_rank(group) if rank is None else rank
        s.world = dist.get_world_size(group) if world is None else world
        s.E, s.H = local_layer.E, local_layer.H
        s.per = (s.E + s.world - 1) // s.world
        s.last_stats = {}
        s.peer = None
        s.peer_decode = peer_decode
        if peer_rows > 0 and s.world > 1 and s.world <= 8 and _has_alltoall(group):
            ok = torch.ones(1, dtype=torch.int32, device=local_layer.table.device)
            try:
                s.peer = _PeerRows(peer_rows, s.H, local_layer.table.device, group, s.world)
            except Exception as e:                      # no peer access / no symmetric memory on this system
                s.peer_error = repr(e)
                ok.zero_()
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)       # all ranks take the same path
            if int(ok) == 0:
                s.peer = None

    # ---- 1..32 replicated tokens
    def decode(s, x, sel, rw, out=None):
        """1..32 replicated tokens -> the summed [B, H] output on every rank.  With peer buffers: each rank leaves its partial
        output in a symmetric buffer and, after one barrier, sums all ranks' partials itself by peer loads in rank order
        (one small kernel, every rank gets bitwise the same result); two buffers alternate so that the barrier of the
        next call also protects the reads of this one.  Otherwise an all-reduce of the collective library - the default
        (peer_decode = False): measured on 2 B200s a 1-token call takes 143 us with NCCL's all-reduce and 154 us with the
        symmetric-memory barrier + combine kernel."""
        if s.peer is None or not s.peer_decode or s.world == 1 or x.shape[0] > s.peer.dec[0].shape[0]:
            y = s.L(x, sel, rw) if out is None else s.L(x, sel, rw, out=out)
            if s.world > 1:
                dist.all_reduce(y, group=s.group)
            return y
        import ctypes as C
        from .capi import check, lib
        B, dev = x.shape[0], x.device
        i = s.peer.dec_turn
        s.peer.dec_turn ^= 1
        s.L(x, sel, rw, out=s.peer.dec[i][:B])
        y = torch.empty(B, s.H, dtype=torch.float32, device=dev) if out is None else out
        s.peer.dec_hdl[i].barrier()                                                # every rank's partial output is complete
        pp = (C.c_void_p * s.world)(*s.peer.dec_ptrs[i])
        if B not in s.peer.dec_rows:                                               # row t of every rank
            s.peer.dec_rows[B] = torch.arange(B, dtype=torch.int32, device=dev).repeat(s.world, 1).contiguous()
        check(lib().nq_ep_combine(y.data_ptr(), pp, s.peer.dec_rows[B].data_ptr(), B, s.H, s.world,
                                  torch.cuda.current_stream(dev).cuda_stream), "ep_combine")
        return y

    # ---- sharded tokens
    def prefill(s, x, sel, rw):
        """x fp16 [T_r, H], sel int64 [T_r, topk], rw fp16 [T_r, topk] (this rank's tokens) -> fp32 [T_r, H]"""
        if s.world == 1:
            return s.L.prefill(x, sel, rw)
        T, k = sel.shape
        dev = x.device
        # every rank asks the same question in the same order, so all of them take the same path
        if s.peer is not None and s._same_count(T) and T * s.world <= s.peer.rows and T <= s.peer.rows_x:
            return s._prefill_peer(x, sel, rw)
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

    def _same_count(s, T):
        """every rank brings the same number of tokens (the peer path addresses tokens as rank * T + t)"""
        c = torch.tensor([T, -T], dtype=torch.int64, device=s.L.table.device)
        dist.all_reduce(c, op=dist.ReduceOp.MAX, group=s.group)
        return int(c[0]) == T and int(c[1]) == -T

    def _prefill_peer(s, x, sel, rw):
        """Exchange over peer memory: only the picks (sel, rw: a few hundred KB) travel by a collective.  Each rank pulls the
        input rows of the tokens that picked its experts from their owners (nq_ep_gather), runs its local prefill on the
        global token list with the other ranks' picks zeroed, leaves the partial rows in its symmetric buffer, and every
        owner sums its tokens' partial rows from the peers in rank order (nq_ep_combine).  No sizes go through the host."""
        import ctypes as C
        from .capi import check, lib
        T, k = sel.shape
        dev, W, P = x.device, s.world, s.peer
        st = torch.cuda.current_stream(dev).cuda_stream
        P.xbuf[:T].copy_(x)
        sel_all = torch.empty(W * T, k, dtype=sel.dtype, device=dev)
        rw_all = torch.empty(W * T, k, dtype=rw.dtype, device=dev)
        dist.all_gather_into_tensor(sel_all, sel.contiguous(), group=s.group)
        dist.all_gather_into_tensor(rw_all, rw.contiguous(), group=s.group)
        owner = torch.div(sel_all, s.per, rounding_mode="floor")
        rw_mine = torch.where(owner == s.rank, rw_all, torch.zeros_like(rw_all))
        if P.xstage is None or P.xstage.shape[0] < W * T:
            P.xstage = torch.zeros(W * T, s.H, dtype=torch.float16, device=dev)
        P.barrier()                                                                # every rank's input rows are in place
        xp = (C.c_void_p * W)(*P.xptrs)
        check(lib().nq_ep_gather(P.xstage.data_ptr(), xp, sel_all.data_ptr(), rw_all.data_ptr(), T, k, s.H, W, s.rank, s.per, st), "ep_gather")
        s.L.prefill(P.xstage[:W * T], sel_all, rw_mine, out=P.buf[:W * T])
        mine = owner[s.rank * T:(s.rank + 1) * T]                                  # ranks that hold a pick of my tokens
        live = rw != 0
        rows = torch.full((W, T), -1, dtype=torch.int32, device=dev)
        tok = torch.arange(s.rank * T, (s.rank + 1) * T, dtype=torch.int32, device=dev)
        for d in range(W):
            rows[d] = torch.where(((mine == d) & live).any(1), tok, rows[d])
        out = torch.empty(T, s.H, dtype=torch.float32, device=dev)
        P.barrier()                                                                # every rank's partial rows are complete
        pp = (C.c_void_p * W)(*P.ptrs)
        check(lib().nq_ep_combine(out.data_ptr(), pp, rows.data_ptr(), T, s.H, W, st), "ep_combine")
        P.barrier()                                                                # buffers may be overwritten from here on
        s.last_stats = dict(dispatch="peer loads", combine="peer loads", dispatch_bytes=None, combine_bytes=None)
        return out
