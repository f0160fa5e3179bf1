"""Decode-path layer (nq_moe_forward through MoELayer) against the reference-generated golden layer and the CPU oracle.
Mirrors the reference's sm120/check.py (mixed levels 0/2/4 + mask mode, B = 1..4, routing patterns, repeatability,
workspace clean on exit) and sm120/levelswitch_mbox.py (mailbox level switch)."""
import random

import numpy as np
import pytest
import torch

from oracle import nq_oracle as O
from tests.golden_io import layer_from
from tests.util import MAX_ABS_TOL, REL_L2_TOL, expert_to_device, expert_to_oracle, layer_errors, layer_report

pytestmark = pytest.mark.gpu


def _routing(B, E, topk, gen, mode="rand", live=None):
    live = list(range(E)) if live is None else live
    rows = []
    for b in range(B):
        if mode == "same" and rows:
            rows.append(rows[0])
        else:
            rows.append(gen.sample(live, topk))
    sel = torch.tensor(rows, dtype=torch.long)
    g = torch.Generator().manual_seed(gen.randrange(1 << 30))
    w = torch.rand(sel.shape, generator=g) + 0.1
    return sel, (w / w.sum(1, keepdim=True)).half()


def _check(L, exs_o, levels, x, sel, rw, tag):
    ref = O.moe_ref(exs_o, levels, x.cpu().numpy(), sel.numpy(), rw.numpy())
    y = L(x.cuda(), sel.cuda(), rw.cuda()).clone()
    y2 = L(x.cuda(), sel.cuda(), rw.cuda()).clone()
    torch.cuda.synchronize()
    assert torch.equal(y, y2), f"{tag}: not bitwise repeatable"
    ma, rl = layer_errors(y.cpu().numpy(), ref)
    rep = layer_report(y.cpu().numpy(), ref)      # raw max-abs beside the normalised one, in every failure message
    assert ma <= MAX_ABS_TOL and rl <= REL_L2_TOL, (tag, rep)
    assert rl <= 5e-4, (tag, rep)             # what the fp16-operand / fp32-accumulate path actually achieves
    for t in (L.cnt_gu, L.cnt_d, L.wq):
        assert int(t.abs().sum()) == 0, f"{tag}: counters not clean on exit"
    return ma, rl


def test_golden_layer():
    from nestquant_b200 import moe
    g = layer_from("layer.npz")
    L = moe.MoELayer(g["E"], g["H"], g["I"], nm_gu=1, nm_dn=1, Bmax=8, topk=g["topk"])
    keep = []
    for e, eo in enumerate(g["experts"]):
        if eo is None:
            continue
        ex = expert_to_device(eo); keep.append(ex)
        L.set(e, ex, g["levels"][e])
    x = torch.from_numpy(g["x"].copy()).cuda()
    y = L(x, torch.from_numpy(g["sel"]).cuda(), torch.from_numpy(g["rw"].copy()).cuda())
    torch.cuda.synchronize()
    ma, rl = layer_errors(y.cpu().numpy(), g["out"])
    assert ma <= MAX_ABS_TOL and rl <= REL_L2_TOL and rl <= 5e-4, (ma, rl)
    assert not y[4].any()                    # token routed only to a level-0 expert


def test_golden_layer_with_low_rank_and_wide_rotation():
    """decode path on the reference-generated layer with the low-rank plane (ranks 2/1 and 1/3) and a 512-wide
    down-input rotation; mirrors sm120/check_lr.py: with the plane removed the result must be plainly wrong"""
    from nestquant_b200 import moe
    g = layer_from("layer_lr.npz")
    L = moe.MoELayer(g["E"], g["H"], g["I"], Bmax=4, topk=g["topk"], ksplit=(2, 2))
    keep = [expert_to_device(eo) for eo in g["experts"]]
    for e, ex in enumerate(keep):
        L.set(e, ex, g["levels"][e])
    x, sel, rw = torch.from_numpy(g["x"].copy()).cuda(), torch.from_numpy(g["sel"]).cuda(), torch.from_numpy(g["rw"].copy()).cuda()
    for ks in ([1], [2]):
        y = L(x, sel, rw, cfg_gu=ks, cfg_dn=ks).clone()
        torch.cuda.synchronize()
        ma, rl = layer_errors(y.cpu().numpy(), g["out"])
        assert ma <= MAX_ABS_TOL and rl <= REL_L2_TOL and rl <= 5e-4, (ks, ma, rl)
    assert int(L.cnt_gu.abs().sum()) == 0
    for ex in keep:
        ex.lr = ex.lr4 = None
    for e, ex in enumerate(keep):
        L.set(e, ex, g["levels"][e])
    y0 = L(x, sel, rw)
    torch.cuda.synchronize()
    assert layer_errors(y0.cpu().numpy(), g["out"])[1] > 20 * max(rl, 1e-6)


@pytest.mark.parametrize("H,I", [(1024, 512), (768, 384)])
def test_mixed_levels_vs_oracle(H, I):
    """12 experts, levels 2/4/0, three masked (50 % of chunks refined), production window codes and signs"""
    from nestquant_b200 import moe
    NE, topk = 12, 4
    nmg, nmd = H // 128 // 2, I // 128 // 2
    masked = {1, 4, 8}
    levels = [2, 4, 4, 2, 4, 4, 2, 4, 4, 4, 2, 0]
    exs = [moe.Expert(H, I, seed=100 + i, nm_gu=nmg if i in masked else None, nm_dn=nmd if i in masked else None,
                      rk_gu=(0, 6, 3)[i % 3], rk_dn=(7, 8, 0)[i % 3], var=i % 4 != 3, sv=0.02) for i in range(NE)]
    exs_o = [expert_to_oracle(e) for e in exs]
    L = moe.MoELayer(NE, H, I, nmg, nmd, Bmax=32, topk=topk)
    for e in range(NE):
        L.set(e, exs[e], levels[e])
    rng = random.Random(0)
    gen = torch.Generator().manual_seed(1)
    for B in (1, 2, 3, 4, 8, 17, 32):
        for mode in ("rand", "same"):
            sel, rw = _routing(B, NE, topk, rng, mode)
            if B == 3:
                rw[1, 2] = 0                  # a zero-weight pick is skipped
            x = torch.randn(B, H, generator=gen).bfloat16().half()
            _check(L, exs_o, levels, x, sel, rw, (H, I, B, mode))


def test_pattern_rate_base_layer_decode_and_prefill():
    """Experts with the 1.75-bit base (base code 1) and the residual codes of that build (3 for gate|up, 9 for down) beside
    ordinary ones, levels 2 and 4, one in mask mode: decode path and fused prefill against the oracle."""
    from nestquant_b200 import moe
    H, I, NE, topk = 768, 512, 6, 3
    nmg, nmd = H // 128 // 2, I // 128 // 2
    exs = [moe.Expert(H, I, seed=600 + i, nm_gu=nmg if i == 3 else None, nm_dn=nmd if i == 3 else None, rk_gu=3 if i < 4 else 0,
                      rk_dn=9 if i < 4 else 7, var=True, sv=0.02, bk_gu=1 if i < 4 else 0, bk_dn=1 if i < 4 else 0) for i in range(NE)]
    exs_o = [expert_to_oracle(e) for e in exs]
    levels = [4, 2, 4, 4, 4, 2]
    L = moe.MoELayer(NE, H, I, nmg, nmd, Bmax=8, topk=topk)
    for e in range(NE):
        L.set(e, exs[e], levels[e])
    rng = random.Random(5)
    gen = torch.Generator().manual_seed(6)
    for B in (1, 4, 8):
        sel, rw = _routing(B, NE, topk, rng)
        x = torch.randn(B, H, generator=gen).bfloat16().half()
        _check(L, exs_o, levels, x, sel, rw, ("bk1", B))
    T = 150
    sel, rw = _routing(T, NE, topk, rng)
    x = torch.randn(T, H, generator=gen).bfloat16().half()
    ref = O.moe_ref(exs_o, levels, x.numpy(), sel.numpy(), rw.numpy())
    y = L.prefill(x.cuda(), sel.cuda(), rw.cuda())
    from tests.prefill_lib import prefill_library
    y_lib = prefill_library(L, x.cuda(), sel.cuda(), rw.cuda())
    torch.cuda.synchronize()
    for got in (y, y_lib):
        ma, rl = layer_errors(got.cpu().numpy(), ref)
        assert ma <= MAX_ABS_TOL and rl <= 5e-4, (ma, rl)
    bad = moe.Expert(H, I, seed=1, rk_gu=0, rk_dn=7, bk_gu=1, bk_dn=1)
    with pytest.raises(AssertionError):
        L.set(0, bad, 4)                      # base code 1 is built with residual codes 3 and 9 only
    L.set(0, bad, 2)                          # at level 2 the residual code does not matter


def test_glm_shape_one_and_four_tokens():
    from nestquant_b200 import moe
    H, I, NE, topk = 6144, 2048, 10, 8
    levels = [4, 2, 4, 4, 2, 4, 2, 4, 4, 2]
    exs = [moe.Expert(H, I, seed=200 + i, rk_gu=0, rk_dn=7, var=True, sv=0.02) for i in range(NE)]
    exs_o = [expert_to_oracle(e) for e in exs]
    L = moe.MoELayer(NE, H, I, Bmax=4, topk=topk)
    for e in range(NE):
        L.set(e, exs[e], levels[e])
    rng = random.Random(5)
    gen = torch.Generator().manual_seed(2)
    for B in (1, 4):
        sel, rw = _routing(B, NE, topk, rng)
        x = torch.randn(B, H, generator=gen).bfloat16().half()
        _check(L, exs_o, levels, x, sel, rw, ("glm", B))
        for e in exs_o:
            e._cache.clear()


def test_nothing_resident_gives_zeros_and_hits_are_counted():
    from nestquant_b200 import moe
    H, I, NE, topk = 256, 128, 4, 2
    exs = [moe.Expert(H, I, seed=i, sv=0.02) for i in range(NE)]
    L = moe.MoELayer(NE, H, I, Bmax=4, topk=topk)
    for e in range(NE):
        L.set(e, exs[e], 0 if e < 2 else 2)
    hits = torch.zeros(NE, dtype=torch.int32, device="cuda")
    L.hits_ptr = hits.data_ptr()
    L.out.fill_(7.0)
    x = torch.randn(2, H).half().cuda()
    sel = torch.tensor([[0, 1], [1, 0]]).cuda()
    rw = torch.tensor([[0.5, 0.5], [0.25, 0.0]]).half().cuda()
    y = L(x, sel, rw)
    torch.cuda.synchronize()
    assert not y.any()
    assert hits.tolist() == [1, 2, 0, 0]       # every pick with a non-zero weight, whatever its level
    sel2 = torch.tensor([[0, 2], [3, 1]]).cuda()
    y = L(x, sel2, rw)
    torch.cuda.synchronize()
    assert y[0].any() and y[1].any() and hits.tolist() == [2, 2, 1, 1]


def test_bad_arguments_raise():
    from nestquant_b200 import moe
    from nestquant_b200.capi import NestQuantError
    L = moe.MoELayer(4, 256, 128, Bmax=2, topk=2)
    x = torch.zeros(2, 256, dtype=torch.float16, device="cuda")
    sel = torch.zeros(2, 2, dtype=torch.long, device="cuda")
    rw = torch.zeros(2, 2, dtype=torch.float16, device="cuda")
    with pytest.raises(NestQuantError):
        L(x, sel, rw, cfg_gu=[5])              # 2 chunks cannot be cut into 5 slices
    with pytest.raises(NestQuantError):
        L.M.moe_forward(x, sel, rw, L.table, L.out, L.acc_gu[:8], L.h, L.acc_d, L.cnt_gu, L.cnt_d, L.wq, 128, 0, 0, [1], [1],
                        4, 0, 3, 0, L.zd, L.cnt_h)
    with pytest.raises(NestQuantError):
        L.M.moe_forward(x, sel, rw, L.table, L.out, L.acc_gu, L.h, L.acc_d, L.cnt_gu, L.cnt_d, L.wq, 128, 0, 0, [1], [1],
                        2, 0, 3, 0, L.zd, L.cnt_h)   # ring width 2 is not built
    with pytest.raises(AssertionError):
        L(x.float(), sel, rw)


def test_mailbox_switches_levels_inside_a_graph():
    """Graph = [mailbox.apply, layer].  Rows staged on a side stream take effect at the next replay, never earlier."""
    from nestquant_b200 import moe
    H, I, NE, topk, B = 512, 256, 6, 3, 2
    exs = [moe.Expert(H, I, seed=300 + i, rk_dn=7, var=True, sv=0.02) for i in range(NE)]
    exs_o = [expert_to_oracle(e) for e in exs]
    L = moe.MoELayer(NE, H, I, Bmax=B, topk=topk)
    MB = moe.Mailbox(L)
    levels = [2] * NE
    for e in range(NE):
        L.set(e, exs[e], 2)
    rng = random.Random(9)
    sel, rw = _routing(B, NE, topk, rng)
    x = torch.randn(B, H).bfloat16().half()
    xd, seld, rwd = x.cuda(), sel.cuda(), rw.cuda()
    s = torch.cuda.Stream(); side = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for _ in range(3):
            MB.apply(); L(xd, seld, rwd)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        MB.apply(); L(xd, seld, rwd)
    torch.cuda.synchronize()
    for step in range(6):
        e = int(sel[0, step % topk])
        new = 4 if levels[e] == 2 else 2
        MB.post(e, moe.entry(exs[e], new), side)
        side.synchronize()
        g.replay(); torch.cuda.synchronize()
        assert MB.done(e)
        levels[e] = new
        ref = O.moe_ref(exs_o, levels, x.numpy(), sel.numpy(), rw.numpy())
        ma, rl = layer_errors(L.out[:B].cpu().numpy(), ref)
        assert rl <= 5e-4, (step, rl)
        stale = list(levels); stale[e] = 6 - new
        _, rl_stale = layer_errors(L.out[:B].cpu().numpy(), O.moe_ref(exs_o, stale, x.numpy(), sel.numpy(), rw.numpy()))
        assert rl_stale > 20 * rl              # the other level would be plainly wrong


def test_config0_layer_as_stated():
    """The CPU-runnable configuration of the workload list exactly as stated: 64 routed experts, top-4 softmax routing from
    seeded bf16 N(0,1) logits, hidden 1024, intermediate 512, level map 25 % 2-bit / 25 % 3-bit (level 4 with half of the
    chunks refined) / 50 % 4-bit, |N(0, 0.02)| output scales, 16 tokens of bf16 N(0,1) activations: decode path (16 tokens in
    one call) and prefill against the oracle, with the raw max-abs error reported beside the normalised one."""
    from nestquant_b200 import moe, synth
    cfg = synth.C0
    E, topk, H, I = cfg["E"], cfg["topk"], cfg["H"], cfg["I"]
    g = torch.Generator().manual_seed(77)
    perm = torch.randperm(E, generator=g).tolist()
    kind = {e: (2 if i < E // 4 else 3 if i < E // 2 else 4) for i, e in enumerate(perm)}
    nmg, nmd = H // 128 // 2, I // 128 // 2
    exs = [moe.Expert(H, I, seed=7000 + e, nm_gu=nmg if kind[e] == 3 else None, nm_dn=nmd if kind[e] == 3 else None,
                      rk_gu=0, rk_dn=7, var=True, sv=0.02) for e in range(E)]
    levels = [2 if kind[e] == 2 else 4 for e in range(E)]
    L = moe.MoELayer(E, H, I, nmg, nmd, Bmax=16, topk=topk)
    for e in range(E):
        L.set(e, exs[e], levels[e])
    sel, rw = synth.routing(16, E, topk, 78)
    x = synth.tokens(16, H, 79)
    exs_o = [expert_to_oracle(e) for e in exs]
    ref = O.moe_ref(exs_o, levels, x.numpy(), sel.numpy(), rw.numpy())
    y = L(x.cuda(), sel.cuda(), rw.cuda()).clone()
    yp = L.prefill(x.cuda(), sel.cuda(), rw.cuda())
    torch.cuda.synchronize()
    for name, got in (("decode path", y), ("prefill", yp)):
        rep = layer_report(got.cpu().numpy(), ref)
        assert rep["max_abs_unit_rms"] <= MAX_ABS_TOL and rep["rel_l2"] <= REL_L2_TOL and rep["rel_l2"] <= 5e-4, (name, rep)
    assert L.status() == 0 and L.prefill_status() == 0


def test_prefill_ignores_picks_without_a_valid_expert_id():
    """-1 padding and ids >= E in sel: the prefill path skips them like the decode path does (same outputs as with those
    picks given weight 0), and the kernels read no table row for them."""
    from nestquant_b200 import moe
    H, I, NE, topk, T = 512, 256, 5, 3, 24
    exs = [moe.Expert(H, I, seed=910 + i, rk_dn=7, var=True, sv=0.02) for i in range(NE)]
    levels = [4, 2, 0, 4, 2]
    L = moe.MoELayer(NE, H, I, Bmax=T, topk=topk)
    for e in range(NE):
        L.set(e, exs[e], levels[e])
    rng = random.Random(12)
    sel, rw = _routing(T, NE, topk, rng)
    x = torch.randn(T, H, generator=torch.Generator().manual_seed(13)).bfloat16().half()
    bad = sel.clone()
    bad[0, 1], bad[3, 0], bad[7, 2], bad[9, :] = -1, NE, NE + 40, -1
    clean_rw = torch.where((bad < 0) | (bad >= NE), torch.zeros_like(rw), rw)
    ref = O.moe_ref([expert_to_oracle(e) for e in exs], levels, x.numpy(), sel.numpy(), clean_rw.numpy())
    yp = L.prefill(x.cuda(), bad.cuda(), rw.cuda())
    yd = L(x.cuda(), bad.cuda(), rw.cuda()).clone()
    torch.cuda.synchronize()
    for got in (yp, yd):
        ma, rl = layer_errors(got.cpu().numpy(), ref)
        assert ma <= MAX_ABS_TOL and rl <= 5e-4, (ma, rl)
    assert not yp[9].any() and not yd[9].any()
    assert L.prefill_status() == 0
