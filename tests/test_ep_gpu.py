"""Expert-parallel layer on 2 GPUs (skipped on a single-GPU box): the prefill whose exchange runs over peer memory (input
rows read from their owners by the first prefill pass, partial rows summed by nq_ep_combine from the peers'
symmetric-memory buffers, nq_ep_barrier in between) must equal, bit for bit, the all-to-all + indexed-add path, and both
must match a single-GPU layer holding every expert; decode = replicated tokens + all-reduce, with the experts split by id
or cut along their intermediate dimension (tensor parallel).  The exchange kernels and the
bounded barrier are also tested on one GPU with emulated ranks."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    try:
        from nestquant_b200 import moe
        from nestquant_b200.ep import EPLayer, owned_experts
        from tests.util import layer_errors
        H, I, NE, topk, T = 1024, 512, 8, 3, 192
        exs = [moe.Expert(H, I, seed=700 + i, rk_gu=0, rk_dn=7, var=True, sv=0.02, dev=dev) for i in range(NE)]
        levels = [4, 2, 4, 4, 2, 4, 4, 2]
        mine = set(owned_experts(NE, world, rank))
        full = moe.MoELayer(NE, H, I, Bmax=4, topk=topk, dev=dev)
        part = moe.MoELayer(NE, H, I, Bmax=4, topk=topk, dev=dev, share=1.0 / world)
        for e in range(NE):
            full.set(e, exs[e], levels[e])
            part.set(e, exs[e], levels[e] if e in mine else 0)
        g = torch.Generator().manual_seed(9)                      # same inputs on every rank; each rank owns a slice of the tokens
        x = torch.randn(world * T, H, generator=g).bfloat16().half()
        sel = torch.stack([torch.randperm(NE, generator=g)[:topk] for _ in range(world * T)])
        rw = torch.softmax(torch.randn(world * T, topk, generator=g), 1).half()
        sl = slice(rank * T, (rank + 1) * T)
        xr, selr, rwr = x[sl].to(dev), sel[sl].to(dev), rw[sl].to(dev)
        ref = full.prefill(xr, selr, rwr)
        ep_a2a = EPLayer(part, rank, world)
        ep_peer = EPLayer(part, rank, world, peer_rows=world * T, peer_decode=True)
        y_a2a = ep_a2a.prefill(xr, selr, rwr)
        y_peer = ep_peer.prefill(xr, selr, rwr)
        y_peer2 = ep_peer.prefill(xr, selr, rwr)
        torch.cuda.synchronize()
        res = dict(peer_on=ep_peer.peer is not None, combine=ep_peer.last_stats.get("combine"), dispatch=ep_peer.last_stats.get("dispatch"),
                   timed_out=ep_peer.peer is not None and ep_peer.peer.timed_out(),
                   same=bool(torch.equal(y_a2a, y_peer)) and bool(torch.equal(y_peer, y_peer2)),
                   err=layer_errors(y_peer.cpu().numpy(), ref.cpu().numpy())[1])
        xd, seld, rwd = x[:3].to(dev), sel[:3].to(dev), rw[:3].to(dev)
        yd = ep_a2a.decode(xd, seld, rwd).clone()
        want = full(xd, seld, rwd).cpu().numpy()
        res["decode_err"] = layer_errors(yd.cpu().numpy(), want)[1]
        # the all-reduce inside the layer kernel (default with peer buffers): several calls in a row alternate the buffer halves;
        # a token whose picks all belong to the other rank makes this rank send a zero slice
        yp = [ep_peer.decode(xd, seld, rwd).clone() for _ in range(5)]
        torch.cuda.synchronize()
        res["decode_peer_err"] = max(layer_errors(y.cpu().numpy(), want)[1] for y in yp)
        res["decode_peer_same"] = all(bool(torch.equal(yp[0], y)) for y in yp[1:])
        sel_one = torch.tensor([[0, 1, 2], [5, 6, 7], [3, 4, 0]]).to(dev)         # token 0: rank 0 only, token 1: rank 1 only (2 ranks)
        y1 = ep_peer.decode(xd, sel_one, rwd).clone()
        res["decode_one_sided_err"] = layer_errors(y1.cpu().numpy(), full(xd, sel_one, rwd).cpu().numpy())[1]
        allr = [torch.empty_like(y1) for _ in range(world)]
        dist.all_gather(allr, y1)
        res["decode_same_on_all_ranks"] = all(bool(torch.equal(allr[0], t)) for t in allr[1:])
        res["decode_status"] = part.status()
        # the variant with a barrier kernel and a sum kernel
        ep_bar = EPLayer(part, rank, world, peer_rows=64, peer_decode=True, fused_decode=False)
        yb = [ep_bar.decode(xd, seld, rwd).clone() for _ in range(3)]
        torch.cuda.synchronize()
        res["decode_barrier_err"] = max(layer_errors(y.cpu().numpy(), want)[1] for y in yb)
        # tensor-parallel decode: rank r holds shard r of every expert (I / world columns: an expert of its own), the partial
        # outputs are summed inside the layer kernel; reference = the shards' layers one after the other on this GPU, in rank
        # order (bitwise), and the CPU oracle's sum over the shards
        import numpy as np
        from oracle import nq_oracle as O
        from tests.util import expert_to_oracle
        Is = I // world
        shards = []
        for r in range(world):
            Lr = moe.MoELayer(NE, H, Is, Bmax=4, topk=topk, dev=dev)
            sx = [moe.Expert(H, Is, seed=900 + 50 * r + i, rk_gu=0, rk_dn=7, var=True, sv=0.02, dev=dev) for i in range(NE)]
            for e in range(NE):
                Lr.set(e, sx[e], levels[e])
            shards.append((Lr, sx))
        ref_tp = torch.zeros(3, H, dtype=torch.float32, device=dev)
        for Lr, _ in shards:
            ref_tp += Lr(xd, seld, rwd)[:3]
        tp = EPLayer(shards[rank][0], rank, world, peer_rows=world, fused_decode=True)
        yt = [tp.decode(xd, seld, rwd).clone() for _ in range(3)]
        torch.cuda.synchronize()
        res["tp_bitwise"] = all(bool(torch.equal(y, ref_tp)) for y in yt)
        want_tp = sum(O.moe_ref([expert_to_oracle(e) for e in sx], levels, xd.cpu().numpy(), seld.cpu().numpy(), rwd.cpu().numpy()) for _, sx in shards)
        res["tp_err"] = layer_errors(yt[0].cpu().numpy(), want_tp.astype(np.float32))[1]
        res["tp_status"] = shards[rank][0].status() + int(tp.peer is None or tp.peer.timed_out())
        # the same with production shards: rank r loads shard r of the nestquant-v1 fixture layer (tp 8 layout), the two ranks'
        # partial outputs are summed in the kernel; reference = the oracle on both shards
        from nestquant_b200 import nqload
        root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "nqload")
        lv3 = {0: 4, 3: 2}
        RL = nqload.RankLayer(root, 3, rank, tp=8, dev=dev)
        Ln = moe.MoELayer(4, RL.H, RL.I, Bmax=4, topk=2, dev=dev)
        for e, ex in RL.ex.items():
            ex.signs = ex.sc[lv3[e]]
            Ln.set(e, ex, lv3[e])
        xn = torch.randn(3, RL.H, generator=g).half().to(dev)
        seln = torch.tensor([[0, 3], [3, 0], [0, 2]]).to(dev)                   # expert 2 is not in the layer
        rwn = torch.tensor([[0.6, 0.4], [0.5, 0.5], [1.0, 0.7]]).half().to(dev)
        tpn = EPLayer(Ln, rank, world, peer_rows=world, fused_decode=True)
        yn = tpn.decode(xn, seln, rwn).clone()
        torch.cuda.synchronize()
        want_n = 0
        for r in range(world):
            shard = nqload.RankLayer(root, 3, r, tp=8, dev="cpu")
            exs_o, lv_o = [None] * 4, [0] * 4
            for e, ex in shard.ex.items():
                ex.signs = ex.sc[lv3[e]]
                exs_o[e], lv_o[e] = expert_to_oracle(ex), lv3[e]
            want_n = want_n + O.moe_ref(exs_o, lv_o, xn.cpu().numpy(), seln.cpu().numpy(), rwn.cpu().numpy())
        res["shards_err"] = layer_errors(yn.cpu().numpy(), want_n.astype(np.float32))[1]
        res["shards_status"] = Ln.status() + int(tpn.peer is None or tpn.peer.timed_out())
        q.put((rank, res))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_prefill_combine_over_peer_memory():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 300
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0, p.exitcode
    out = dict(q.get(timeout=10) for _ in range(2))
    for rank, r in out.items():
        assert r["peer_on"] and r["combine"] == "peer loads" and r["dispatch"] == "peer loads", (rank, r)
        assert r["same"] and r["err"] <= 1e-4 and r["decode_err"] <= 1e-4 and not r["timed_out"], (rank, r)
        assert r["decode_peer_err"] <= 1e-4 and r["decode_peer_same"] and r["decode_barrier_err"] <= 1e-4, (rank, r)
        assert r["decode_one_sided_err"] <= 1e-4 and r["decode_same_on_all_ranks"] and r["decode_status"] == 0, (rank, r)
        assert r["tp_bitwise"] and r["tp_err"] <= 1e-4 and r["tp_status"] == 0, (rank, r)
        assert r["shards_err"] <= 1e-4 and r["shards_status"] == 0, (rank, r)


def test_exchange_kernels_on_one_gpu():
    """nq_ep_gather / nq_ep_picks / nq_ep_combine with the buffers of three emulated ranks on one device (the kernels only see addresses):
    the gathered rows and the rank-ordered sums must equal plain indexing."""
    import ctypes as C
    from nestquant_b200.capi import check, lib
    W, T, k, H, per, rank = 3, 50, 4, 256, 4, 1
    g = torch.Generator().manual_seed(21)
    xs = [torch.randn(T, H, generator=g).half().cuda() for _ in range(W)]
    sel = torch.randint(0, W * per, (W * T, k), generator=g).cuda()
    rw = torch.rand(W * T, k, generator=g).half().cuda()
    rw[5] = 0                                              # a token without any weight is not fetched
    stage = torch.full((W * T, H), 7.0, dtype=torch.float16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    ptrs = (C.c_void_p * W)(*[x.data_ptr() for x in xs])
    check(lib().nq_ep_gather(stage.data_ptr(), ptrs, sel.data_ptr(), rw.data_ptr(), T, k, H, W, rank, per, st), "ep_gather")
    need = (((sel // per) == rank) & (rw != 0)).any(1)
    want = torch.where(need[:, None], torch.cat(xs), torch.full_like(stage, 7.0))
    torch.cuda.synchronize()
    assert torch.equal(stage, want) and 0 < int(need.sum()) < W * T and not bool(need[5])
    # nq_ep_picks: every rank's picks read from the ranks' buffers, the weights of other ranks' experts zeroed
    sels = [torch.randint(-2, W * per + 2, (T, k), generator=g).cuda() for _ in range(W)]       # some ids out of range
    rws = [torch.rand(T, k, generator=g).half().cuda() for _ in range(W)]
    sel_all = torch.empty(W * T, k, dtype=torch.int64, device="cuda")
    rw_mine = torch.empty(W * T, k, dtype=torch.float16, device="cuda")
    ps, pr = (C.c_void_p * W)(*[t.data_ptr() for t in sels]), (C.c_void_p * W)(*[t.data_ptr() for t in rws])
    check(lib().nq_ep_picks(ps, pr, T, k, W, rank, per, sel_all.data_ptr(), rw_mine.data_ptr(), st), "ep_picks")
    cat_sel, cat_rw = torch.cat(sels), torch.cat(rws)
    torch.cuda.synchronize()
    assert torch.equal(sel_all, cat_sel)
    assert torch.equal(rw_mine, torch.where(torch.div(cat_sel, per, rounding_mode="floor") == rank, cat_rw, torch.zeros_like(cat_rw)))
    parts = [torch.randn(W * T, H, generator=g).cuda() for _ in range(W)]
    rows = torch.randint(-1, W * T, (W, T), generator=g, dtype=torch.int32).cuda()
    out = torch.empty(T, H, device="cuda")
    pp = (C.c_void_p * W)(*[p.data_ptr() for p in parts])
    check(lib().nq_ep_combine(out.data_ptr(), pp, rows.data_ptr(), T, H, W, st), "ep_combine")
    ref = torch.zeros(T, H, device="cuda")
    for r in range(W):                                     # rank order
        ok = rows[r] >= 0
        ref = ref + torch.where(ok[:, None], parts[r][rows[r].clamp(min=0).long()], torch.zeros_like(ref))
    torch.cuda.synchronize()
    assert torch.equal(out, ref)


def test_barrier_wait_is_bounded_and_prefill_first_pass_reads_peer_rows():
    """nq_ep_barrier on one GPU, as rank 0 of 2: with the peer's flag already at the call number the barrier passes and the
    call number advances; with a flag that nothing sets the wait runs out after its (short) limit, the status word is raised
    and the kernel returns - the device stays usable.  Then nq_pf_pre_ep with the buffers of three emulated ranks on this
    device (the kernel only sees addresses) against nq_pf_pre on the concatenated rows."""
    import ctypes as C
    import time
    from nestquant_b200 import ext, moe
    from nestquant_b200.capi import check, lib
    st = torch.cuda.current_stream().cuda_stream
    mine = torch.zeros(8, dtype=torch.int32, device="cuda")          # my flags: [r] = what rank r announced to me
    theirs = torch.zeros(8, dtype=torch.int32, device="cuda")        # the emulated peer's flags
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    flags = (C.c_void_p * 2)(mine.data_ptr(), theirs.data_ptr())
    mine[1] = 1                                                      # the peer has announced call 1 already
    check(lib().nq_ep_barrier(flags, 0, 2, epoch.data_ptr(), status.data_ptr(), 50_000_000, st), "ep_barrier")
    torch.cuda.synchronize()
    assert int(status) == 0 and int(epoch) == 1 and int(theirs[0]) == 1 and int(mine[0]) == 1
    t = time.perf_counter()
    check(lib().nq_ep_barrier(flags, 0, 2, epoch.data_ptr(), status.data_ptr(), 50_000_000, st), "ep_barrier")   # call 2: nobody answers
    torch.cuda.synchronize()
    dt = time.perf_counter() - t
    assert int(status) == 1 and int(epoch) == 2 and int(theirs[0]) == 2, "the wait must give up and say so"
    assert 0.03 < dt < 1.0, dt                                       # 50 ms limit
    assert float(torch.ones(4, device="cuda").sum()) == 4.0          # the context is alive

    W, Tl, H, I, NE, topk = 3, 20, 512, 256, 6, 2
    exs = [moe.Expert(H, I, seed=40 + i, sv=0.02) for i in range(NE)]
    L = moe.MoELayer(NE, H, I, Bmax=1, topk=topk)
    for e in range(NE):
        L.set(e, exs[e], 2 if e != 4 else 0)
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(Tl, H, generator=g).half().cuda() for _ in range(W)]
    R = W * Tl * topk
    pt = torch.randint(0, W * Tl, (R,), generator=g).int().cuda()
    pe = torch.randint(-1, NE + 1, (R,), generator=g).int().cuda()     # includes ids outside [0, E) and a level-0 expert
    outs = []
    for peers in (False, True):
        xg = torch.full((R, H), 3.0, dtype=torch.float16, device="cuda")
        xu = torch.full((R, H), 3.0, dtype=torch.float16, device="cuda")
        zg = torch.zeros(R, 4, device="cuda")
        if peers:
            ext.pf_pre_ep([x.data_ptr() for x in xs], Tl, H, pt, pe, L.table, xg, xu, zg, I, kperm=True)
        else:
            ext.pf_pre(torch.cat(xs), pt, pe, L.table, xg, xu, zg, I, kperm=True)
        outs.append((xg, xu))
    torch.cuda.synchronize()
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    skipped = (pe < 0) | (pe >= NE) | (pe == 4)
    assert bool((outs[1][0][skipped] == 3.0).all()) and bool((outs[1][0][~skipped] != 3.0).any())
