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
