"""Expert-parallel layer: the experts of a MoE layer split contiguously over the ranks of a process group.

Each rank keeps the planes of its own experts only; its device table marks the others level 0, which the kernels
already treat as "not resident here, contributes nothing" (the reference's hook: sm120/nqmoe.cu:393,727,1026-1030).
Two exchange patterns, both over torch.distributed (NCCL on GPUs, gloo in the CPU tests):

  decode(x, sel, rw)    tokens replicated on every rank (1..32 tokens): local layer call, then an all-reduce of the
                        [B, H] partial outputs - what the reference's evaluation harness does with all-gather +
                        reduce-scatter (sm120/eval/eval_reg.py:137-142,181); latency-bound, tiny messages.
  prefill(x, sel, rw)   tokens sharded (each rank owns T_r tokens).  On NVLink-connected GPUs the exchange runs over peer
                        memory: every rank's input rows sit in a symmetric-memory buffer, only the picks travel by a
                        collective (an all-gather of a few hundred KB), each rank's prefill reads the rows of its pairs
                        straight from their owners in its first pass, leaves its partial output rows in a symmetric
                        buffer, and each owner sums its tokens' partial rows from the peers in rank order
                        (nq_ep_combine).  The barriers in between are nq_ep_barrier (bounded waits).  Otherwise (gloo, no
                        peer access, more rows than the buffers hold): all-to-all of each token row to every rank that
                        owns one of its picks, local prefill, all-to-all back, indexed add in rank order.

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


PICKS_MAX = 16        # picks per token that the symmetric pick buffers are sized for


class PeerBuffers:
    """Symmetric-memory buffers of one rank, with every rank's address of each, and a barrier of our own over them.

    part   fp32 [rows, H]      partial output rows of the prefill (row = global token)
    xbuf   fp16 [rows_x, H]    this rank's input rows, read by the peers' first prefill pass
    sel, rw  int64 / fp16 [rows_x * 16]   this rank's picks, read by the peers before they sort (nq_ep_picks)
    dec    2 x fp32 [32, H]    partial outputs of the decode path (alternating), for the barrier + sum-kernel variant
    recv   fp32 [2, world, 32, H], rcnt int32 [2, 32 * 64]   receive slots and arrival counters of the in-kernel all-reduce
    flags  int32 [8]           barrier flags: flag [r] = last call number rank r announced to this rank

    torch's symmetric-memory module only allocates and exchanges the addresses; the barrier is nq_ep_barrier, whose wait is
    bounded (timeout_s) and raises `status` instead of hanging the GPU when a peer never arrives."""

    def __init__(s, rows, H, dev, group, rank, world, timeout_s=2.0):
        import torch.distributed._symmetric_memory as symm
        g = group if group is not None else dist.group.WORLD
        s.rank, s.world, s.H, s.rows = rank, world, H, rows
        s.timeout_ns = int(timeout_s * 1e9)

        def shared(*shape, dtype):
            t = symm.empty(*shape, dtype=dtype, device=dev)
            return t, [int(p) for p in symm.rendezvous(t, g).buffer_ptrs]

        s.part, s.part_ptrs = shared(rows, H, dtype=torch.float32)
        s.rows_x = (rows + world - 1) // world
        s.xbuf, s.x_ptrs = shared(s.rows_x, H, dtype=torch.float16)
        s.sel, s.sel_ptrs = shared(s.rows_x * PICKS_MAX, dtype=torch.int64)      # this rank's picks, read by the peers
        s.rw, s.rw_ptrs = shared(s.rows_x * PICKS_MAX, dtype=torch.float16)
        s.dec, s.dec_ptrs, s.dec_turn, s.dec_rows = [], [], 0, {}
        for _ in range(2):
            b, p = shared(32, H, dtype=torch.float32)
            s.dec.append(b); s.dec_ptrs.append(p)
        from .capi import lib
        # in-kernel all-reduce of the decode path: receive slots and arrival counters of every rank, this rank's call counter
        s.recv, s.recv_ptrs = shared(int(lib().nq_moe_ep_recv_floats(world, H)), dtype=torch.float32)
        s.rcnt, s.rcnt_ptrs = shared(int(lib().nq_moe_ep_counter_ints()), dtype=torch.int32)
        s.rcnt.zero_()
        s.dec_epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        s.flags, s.flag_ptrs = shared(8, dtype=torch.int32)
        s.flags.zero_()
        s.epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        s.status = torch.zeros(1, dtype=torch.int32, device=dev)
        # (the caller's next collective on this stream orders the zeroing before any peer's first announcement)

    def barrier(s):
        """all ranks' earlier work on the current stream is complete and visible once this has run on every rank"""
        import ctypes as C
        from .capi import check, lib
        arr = (C.c_void_p * s.world)(*s.flag_ptrs)
        check(lib().nq_ep_barrier(arr, s.rank, s.world, s.epoch.data_ptr(), s.status.data_ptr(), s.timeout_ns,
                                  torch.cuda.current_stream(s.flags.device).cuda_stream), "ep_barrier")

    def timed_out(s):
        """True if a barrier wait has run out since the buffers were made (synchronises with the device)"""
        return bool(int(s.status.item()))


class EPLayer:
    def __init__(s, local_layer, rank=None, world=None, group=None, peer_rows=0, peer_decode=False, timeout_s=2.0, fused_decode=True):
        """peer_rows > 0: exchange over peer memory for up to that many tokens of the whole group per prefill call (NCCL groups
        on peer-connected GPUs only; silently off where symmetric memory cannot be set up).  With peer buffers, decode() sums
        the ranks' partial outputs inside the layer kernel (fused_decode), or by a barrier kernel + sum kernel (peer_decode),
        or, without either, by the collective library's all-reduce."""
        s.L, s.group = local_layer, group
        s.rank = dist.get_rank(group) if rank is None else rank
        s.world = dist.get_world_size(group) if world is None else world
        s.E, s.H = local_layer.E, local_layer.H
        s.per = (s.E + s.world - 1) // s.world
        s.last_stats = {}
        s.peer = None
        s.peer_decode, s.fused_decode = peer_decode, fused_decode
        s.events = None              # set to [] to have prefill() record (label, cuda event) marks between its phases
        s._same = set()
        if peer_rows > 0 and s.world > 1 and s.world <= 8 and _has_alltoall(group):
            ok = torch.ones(1, dtype=torch.int32, device=local_layer.table.device)
            try:
                s.peer = PeerBuffers(peer_rows, s.H, local_layer.table.device, group, s.rank, s.world, timeout_s)
            except Exception as e:                      # no peer access / no symmetric memory on this system
                s.peer_error = repr(e)
                ok.zero_()
            # all ranks take the same path; the collective also orders every rank's zeroed flags before anybody's first barrier
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            if int(ok) == 0:
                s.peer = None

    def ep_args(s):
        """the `ep` argument of MoELayer.__call__ / .capture for this rank, or None without peer buffers"""
        P = s.peer
        return None if P is None or s.world == 1 else (s.world, s.rank, P.recv_ptrs, P.rcnt_ptrs, P.dec_epoch)

    def _mark(s, label):
        if s.events is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            s.events.append((label, ev))

    # ---- 1..32 replicated tokens
    def decode(s, x, sel, rw, out=None):
        """1..32 replicated tokens -> the summed [B, H] output on every rank.  With peer buffers and peer_decode: each rank
        leaves its partial output in a symmetric buffer and, after one barrier, sums all ranks' partials itself by peer
        loads in rank order (one small kernel, every rank gets bitwise the same result); two buffers alternate so that the
        barrier of the next call also protects the reads of this one.  Otherwise an all-reduce of the collective library -
        for 24 KB per token NCCL's all-reduce was measured faster than barrier + combine kernel.  The default with peer
        buffers is neither: the all-reduce inside the layer kernel (fused_decode)."""
        if s.peer is not None and s.fused_decode and s.world > 1:
            # one kernel: every rank's partial output slices land in every rank's receive buffer as they are finished, and each
            # rank adds them up in rank order at the end of the same launch
            P = s.peer
            return s.L(x, sel, rw, **({} if out is None else {"out": out}), ep=(s.world, s.rank, P.recv_ptrs, P.rcnt_ptrs, P.dec_epoch))
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
        s.peer.barrier()                                                           # every rank's partial output is complete
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
        if s.peer is not None and T * s.world <= s.peer.rows and T <= s.peer.rows_x and s._same_count(T):
            return s._prefill_peer(x, sel, rw)
        return s._prefill_alltoall(x, sel, rw)

    def _prefill_alltoall(s, x, sel, rw):
        """the exchange by collectives (the CPU tests' gloo groups, or GPUs without peer access): all-to-all of each token row
        to every rank that owns one of its picks, local prefill, all-to-all back, indexed add in rank order"""
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
        s.last_stats = dict(dispatch="all-to-all", combine="all-to-all", sent_rows=sum(in_splits), recv_rows=sum(out_splits),
                            dispatch_bytes=sum(in_splits) * s.H * 2, combine_bytes=sum(out_splits) * s.H * 4)
        part = s.L.prefill(xr, selr, rwr) if xr.shape[0] else torch.zeros(0, s.H, dtype=torch.float32, device=dev)
        back = _all_to_all(in_splits, part, out_splits, s.group)                   # partial rows return to their owners
        out = torch.zeros(T, s.H, dtype=torch.float32, device=dev)
        o = 0
        for d in range(s.world):                                                   # fixed rank order: repeatable sums
            n = in_splits[d]
            if n:
                out.index_add_(0, idx[d], back[o:o + n])
            o += n
        return out

    def _same_count(s, T):
        """every rank brings the same number of tokens (the peer path addresses tokens as rank * T + t); asked once per T"""
        if T in s._same:
            return True
        c = torch.tensor([T, -T], dtype=torch.int64, device=s.L.table.device)
        dist.all_reduce(c, op=dist.ReduceOp.MAX, group=s.group)
        ok = int(c[0]) == T and int(c[1]) == -T
        if ok:
            s._same.add(T)
        return ok

    def _prefill_peer(s, x, sel, rw):
        """Exchange over peer memory: only the picks (sel, rw: a few hundred KB) travel by a collective.  Each rank runs its
        local prefill on the global token list with the other ranks' picks zeroed (they sort behind its own pairs and cost
        nothing); the first pass of that prefill reads each pair's input row from its owner's buffer (the dispatch), the
        partial rows stay in this rank's symmetric buffer, and every owner sums its tokens' partial rows from the peers in
        rank order (nq_ep_combine, the combine).  No sizes go through the host."""
        import ctypes as C
        from .capi import check, lib
        T, k = sel.shape
        dev, W, P = x.device, s.world, s.peer
        st = torch.cuda.current_stream(dev).cuda_stream
        s._mark("start")
        P.xbuf[:T].copy_(x)
        sel_all = torch.empty(W * T, k, dtype=torch.int64, device=dev)
        rw_mine = torch.empty(W * T, k, dtype=torch.float16, device=dev)
        if k <= PICKS_MAX:
            # the picks stay where they are: after the barrier every rank reads them from the owners' buffers
            P.sel[:T * k].copy_(sel.reshape(-1))
            P.rw[:T * k].copy_(rw.reshape(-1))
            P.barrier()                                                            # every rank's rows and picks are in place
            check(lib().nq_ep_picks((C.c_void_p * W)(*P.sel_ptrs), (C.c_void_p * W)(*P.rw_ptrs), T, k, W, s.rank, s.per,
                                    sel_all.data_ptr(), rw_mine.data_ptr(), st), "ep_picks")
        else:
            # one collective for both: the expert id in the low 32 bits (two's complement), the fp16 weight in bits 32..47
            packed = (sel & 0xFFFFFFFF) | (rw.contiguous().view(torch.int16).to(torch.int64) & 0xFFFF) << 32
            packed_all = torch.empty(W * T, k, dtype=torch.int64, device=dev)
            dist.all_gather_into_tensor(packed_all, packed.contiguous(), group=s.group)
            sel_all = (packed_all << 32) >> 32                                     # sign-extends padded (negative) ids
            rw_all = (packed_all >> 32).to(torch.int16).view(torch.float16)
            rw_mine = torch.where(torch.div(sel_all, s.per, rounding_mode="floor") == s.rank, rw_all, torch.zeros_like(rw_all))
            P.barrier()                                                            # every rank's input rows are in place
        s._mark("picks gathered, inputs in place")
        s.L.prefill(x, sel_all, rw_mine, out=P.part[:W * T], x_peers=(P.x_ptrs, T))
        s._mark("local prefill (dispatch by peer loads in its first pass)")
        mine = torch.div(sel, s.per, rounding_mode="floor")                        # ranks that hold a pick of my tokens
        live = rw != 0
        tok = torch.arange(s.rank * T, (s.rank + 1) * T, dtype=torch.int32, device=dev)
        held = (torch.where(live, mine, -1).unsqueeze(0) == torch.arange(W, device=dev).view(W, 1, 1)).any(2)   # [W, T]
        rows = torch.where(held, tok.unsqueeze(0), -1).to(torch.int32).contiguous()
        out = torch.empty(T, s.H, dtype=torch.float32, device=dev)
        P.barrier()                                                                # every rank's partial rows are complete
        pp = (C.c_void_p * W)(*P.part_ptrs)
        check(lib().nq_ep_combine(out.data_ptr(), pp, rows.data_ptr(), T, s.H, W, st), "ep_combine")
        P.barrier()                                                                # buffers may be overwritten from here on
        s._mark("combine by peer loads")
        s.last_stats = dict(dispatch="peer loads", combine="peer loads", dispatch_bytes=None, combine_bytes=None)
        return out
