"""Promotion copy (pinned host record -> slot -> staged row -> sequence number on a side stream) and the record layout.
Mirrors the reference's sm120/levelswitch_mbox.py: a captured graph [mailbox.apply, layer] replays while a side stream
promotes and demotes experts; every replay must match the reference output of the level set it actually applied, freed
slots are overwritten with junk, and a switch takes effect at most one replay late."""
import random

import numpy as np
import pytest
import torch

from oracle import nq_oracle as O
from tests.util import expert_to_oracle, layer_errors

pytestmark = pytest.mark.gpu


def test_record_layout_matches_reference_sizes():
    """GLM expert record = 10,088,448 B; config-0 expert = 434,176 B (streaming/p4rec.py with the reference's plane sizes)"""
    from nestquant_b200 import moe, p4rec
    ex = moe.Expert(6144, 2048, seed=1, rk_gu=0, rk_dn=7, dev="cpu")
    lay = p4rec.layout(ex, 6144, 2048)
    assert lay["rec_bytes"] == 10088448
    assert all(o % 256 == 0 for o, _ in lay["seg"].values())
    assert p4rec.layout(moe.Expert(1024, 512, seed=1, rk_gu=0, rk_dn=7, dev="cpu"), 1024, 512)["rec_bytes"] == 434176
    rec = p4rec.pack(ex, lay, pin=False)
    o, n = lay["seg"]["dn.p4"]
    assert torch.equal(rec[o:o + n], ex.dn.p4.view(torch.uint8))


def test_promotions_race_a_captured_graph():
    from nestquant_b200 import moe, p4rec
    H, I, NE, topk, B, NSLOT = 1024, 512, 8, 4, 3, 3
    exs = [moe.Expert(H, I, seed=40 + i, rk_gu=0, rk_dn=7, var=True, sv=0.02) for i in range(NE)]
    exs_o = [expert_to_oracle(e) for e in exs]
    lay = p4rec.layout(exs[0], H, I)
    records = [p4rec.pack(e, lay) for e in exs]
    # the resident copy keeps only the base: move the residual planes away so a stale pointer would be caught
    for e in exs:
        for p in (e.gu, e.dn):
            p.p4 = torch.zeros(1, dtype=torch.int32, device="cuda"); p.d4 = torch.zeros(1, dtype=torch.int32, device="cuda")
    L = moe.MoELayer(NE, H, I, Bmax=B, topk=topk)
    MB = moe.Mailbox(L)
    pool = p4rec.SlotPool(NSLOT, lay["rec_bytes"])
    junk = torch.randint(0, 255, (lay["rec_bytes"],), dtype=torch.uint8).pin_memory()
    for e in range(NE):
        L.set(e, exs[e], 2)
    rng = random.Random(2)
    sel = torch.tensor([rng.sample(range(NE), topk) for _ in range(B)])
    rw = torch.softmax(torch.randn(B, topk), 1).half()
    x = torch.randn(B, H).bfloat16().half()
    xd, seld, rwd = x.cuda(), sel.cuda(), rw.cuda()
    s, side = torch.cuda.Stream(), torch.cuda.Stream()
    with torch.cuda.stream(s):
        for _ in range(3):
            MB.apply(); L(xd, seld, rwd)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        MB.apply(); L(xd, seld, rwd)
    torch.cuda.synchronize()
    level = [2] * NE
    pending = {}
    cache = {}
    lags = []
    for step in range(40):
        for _ in range(rng.randint(0, 2)):                  # scheduler: new operations on the side stream, no host sync
            idle = [e for e in range(NE) if e not in pending]
            ups = [e for e in idle if level[e] == 2 and e not in pool.slot_of]
            downs = [e for e in idle if level[e] == 4]
            if pool.free and ups and (not downs or rng.random() < 0.5):
                e = rng.choice(ups)
                pool.promote(MB, e, exs[e], lay, records[e], moe.entry, side); pending[e] = (4, step)
            elif downs:
                e = rng.choice(downs)
                pool.demote(MB, e, exs[e], moe.entry, side); pending[e] = (2, step)
        g.replay()                                          # races the side stream
        torch.cuda.current_stream().synchronize()
        out = L.out[:B].clone()
        for e in list(pending):                             # which operations did this replay's mailbox apply?
            if MB.done(e):
                lv, st0 = pending.pop(e)
                level[e] = lv; lags.append(step - st0)
                if lv == 2:                                 # released: scribble the slot, then recycle it
                    i = pool.slot_of[e]
                    with torch.cuda.stream(side):
                        pool.buf[i].copy_(junk, non_blocking=True)
                    pool.release(e)
        key = tuple(level)
        if key not in cache:
            cache[key] = O.moe_ref(exs_o, list(level), x.numpy(), sel.numpy(), rw.numpy())
        ma, rl = layer_errors(out.cpu().numpy(), cache[key])
        assert rl <= 5e-4, (step, level, rl)
    side.synchronize()
    assert lags and max(lags) <= 2 and len(cache) > 3       # switches landed, several distinct level sets were checked


def test_engine_promotes_from_a_record_file(tmp_path):
    """The host engine end to end on the GPU: records in a file -> pinned host cache -> slots -> staged rows -> sequence
    numbers, applied by the mailbox of a captured layer call; outputs follow the oracle at the levels that are live."""
    from nestquant_b200 import moe, p4rec
    from nestquant_b200.engine import Engine, write_records
    H, I, NE, topk, B = 1024, 512, 6, 3, 2
    exs = [moe.Expert(H, I, seed=90 + i, rk_gu=0, rk_dn=7, var=True, sv=0.02) for i in range(NE)]
    exs_o = [expert_to_oracle(e) for e in exs]
    lay = p4rec.layout(exs[0], H, I)
    path = str(tmp_path / "rank0.bin")
    write_records(path, [p4rec.pack(e, lay, pin=False) for e in exs])
    for e in exs:                                           # resident copy keeps only the base
        for p in (e.gu, e.dn):
            p.p4 = torch.zeros(1, dtype=torch.int32, device="cuda"); p.d4 = torch.zeros(1, dtype=torch.int32, device="cuda")
    L = moe.MoELayer(NE, H, I, Bmax=B, topk=topk)
    MB = moe.Mailbox(L)
    for e in range(NE):
        L.set(e, exs[e], 2)
    pool = p4rec.SlotPool(4, lay["rec_bytes"])
    eng = Engine(path, lay["rec_bytes"], 3, 2, torch.cuda.current_device())
    g = torch.Generator().manual_seed(3)
    sel = torch.stack([torch.randperm(NE, generator=g)[:topk] for _ in range(B)])
    rw = torch.softmax(torch.randn(B, topk, generator=g), 1).half()
    x = torch.randn(B, H, generator=g).bfloat16().half()
    G = L.capture(B, with_mailbox=MB)
    G.x.copy_(x); G.sel.copy_(sel); G.rw.copy_(rw)

    def settle(tags):
        got, t0 = [], __import__("time").time()
        while len(got) < len(tags) and __import__("time").time() - t0 < 20:
            got += eng.poll()
        assert sorted(t for t, *_ in got) == sorted(tags), (got, eng.stats())
        G.replay(); torch.cuda.synchronize()                # this replay's mailbox applies the rows
        return got

    def check(levels):
        ref = O.moe_ref(exs_o, levels, x.numpy(), sel.numpy(), rw.numpy())
        ma, rl = layer_errors(G.out.cpu().numpy(), ref)
        assert rl <= 5e-4, (levels, rl)

    G.replay(); torch.cuda.synchronize(); check([2] * NE)
    ups = [1, 4, 2]
    for i, e in enumerate(ups):                             # three promotions through two reader threads
        MB.hseq[e] += 1
        pool.slot_of[e] = pool.free.pop()
        eng.upgrade(e, e, pool.slot_ptr(pool.slot_of[e]), MB.stage[e].data_ptr(), p4rec.row(exs[e], lay, pool.slot_ptr(pool.slot_of[e]), moe.entry),
                    MB.seq[e:e + 1].data_ptr(), MB.hseq[e])
    res = settle(ups)
    assert all(tr >= 0 and te >= tr for _, _, tr, te in res) and all(MB.done(e) for e in ups)
    check([4 if e in ups else 2 for e in range(NE)])
    MB.hseq[4] += 1                                         # demotion: row only
    eng.post(104, MB.stage[4].data_ptr(), moe.entry(exs[4], 2), MB.seq[4:5].data_ptr(), MB.hseq[4])
    settle([104])
    check([4 if e in (1, 2) else 2 for e in range(NE)])
    pool.buf[pool.slot_of[4]].fill_(0xAB); pool.release(4)  # the freed slot may be scribbled over
    MB.hseq[4] += 1                                         # and promoted again: the record is still in the host cache
    pool.slot_of[4] = pool.free.pop()
    eng.upgrade(204, 4, pool.slot_ptr(pool.slot_of[4]), MB.stage[4].data_ptr(), p4rec.row(exs[4], lay, pool.slot_ptr(pool.slot_of[4]), moe.entry),
                MB.seq[4:5].data_ptr(), MB.hseq[4])
    (_, hit, _, _), = settle([204])
    assert hit
    check([4 if e in ups else 2 for e in range(NE)])
    st = eng.stats()
    assert st["upgrades"] == 4 and st["host_hits"] == 1 and st["posts"] == 1 and st["device_errors"] == 0
    eng.close()
