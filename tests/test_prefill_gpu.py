"""Prefill path (MoELayer.prefill and the pf_* helpers through the C ABI) against the reference-generated golden layers
and the CPU oracle.  Mirrors the reference's sm120/smoke_prefill.py: prefill == decode-path slices == dense reference,
hits exported, plus the low-rank plane and the 512-wide rotation (sm120/check_lr.py)."""
import random

import numpy as np
import pytest
import torch

from oracle import nq_oracle as O
from tests.golden_io import layer_from
from tests.prefill_lib import prefill_library
from tests.util import MAX_ABS_TOL, REL_L2_TOL, expert_to_device, expert_to_oracle, layer_errors

pytestmark = pytest.mark.gpu


def _layer_from_golden(name, **kw):
    from nestquant_b200 import moe
    g = layer_from(name)
    L = moe.MoELayer(g["E"], g["H"], g["I"], Bmax=8, topk=g["topk"], **kw)
    keep = []
    for e, eo in enumerate(g["experts"]):
        if eo is not None:
            ex = expert_to_device(eo); keep.append(ex)
            L.set(e, ex, g["levels"][e])
    x = torch.from_numpy(g["x"].copy()).cuda()
    return g, L, keep, x, torch.from_numpy(g["sel"]).cuda(), torch.from_numpy(g["rw"].copy()).cuda()


@pytest.mark.parametrize("deterministic,fused", [(True, True), (True, False), (False, False)])
def test_golden_layer_prefill(deterministic, fused):
    g, L, keep, x, sel, rw = _layer_from_golden("layer.npz", nm_gu=1, nm_dn=1)
    y = L.prefill(x, sel, rw) if fused else prefill_library(L, x, sel, rw, deterministic=deterministic)
    torch.cuda.synchronize()
    ma, rl = layer_errors(y.cpu().numpy(), g["out"])
    assert ma <= MAX_ABS_TOL and rl <= REL_L2_TOL and rl <= 5e-4, (ma, rl)
    assert not y[4].any()
    if deterministic:
        assert torch.equal(y, L.prefill(x, sel, rw) if fused else prefill_library(L, x, sel, rw))
    assert L.prefill_status() == 0


def test_golden_layer_with_low_rank_and_wide_rotation():
    g, L, keep, x, sel, rw = _layer_from_golden("layer_lr.npz")
    for fused in (True, False):
        # tiny chunks: exercises the chunk loops (fused: chunks of 5 pairs cut experts' pair ranges in two)
        y = L.prefill(x, sel, rw, R=5) if fused else prefill_library(L, x, sel, rw, R=4, G=1)
        torch.cuda.synchronize()
        ma, rl = layer_errors(y.cpu().numpy(), g["out"])
        assert ma <= MAX_ABS_TOL and rl <= REL_L2_TOL and rl <= 5e-4, (fused, ma, rl)
    # without the low-rank plane the result must be plainly different (the plane is really applied)
    for ex in keep:
        ex.lr = ex.lr4 = None
    for e, ex in enumerate(keep):
        L.set(e, ex, g["levels"][e])
    y0 = L.prefill(x, sel, rw)
    torch.cuda.synchronize()
    _, rl0 = layer_errors(y0.cpu().numpy(), g["out"])
    assert rl0 > 20 * max(rl, 1e-6)


def test_prefill_matches_decode_path_and_oracle():
    from nestquant_b200 import moe
    H, I, NE, topk, T = 1024, 512, 16, 4, 96
    nmg, nmd = H // 128 // 2, I // 128 // 2
    levels = [2, 4, 4, 0, 4, 2, 4, 4, 2, 4, 4, 2, 4, 0, 2, 4]
    masked = {2, 9}
    exs = [moe.Expert(H, I, seed=700 + i, nm_gu=nmg if i in masked else None, nm_dn=nmd if i in masked else None,
                      rk_gu=(0, 6)[i % 2], rk_dn=7, var=True, sv=0.02) for i in range(NE)]
    L = moe.MoELayer(NE, H, I, nmg, nmd, Bmax=32, topk=topk)
    for e in range(NE):
        L.set(e, exs[e], levels[e])
    hits = torch.zeros(NE, dtype=torch.int32, device="cuda")
    L.hits_ptr = hits.data_ptr()
    g = torch.Generator().manual_seed(4)
    x = torch.randn(T, H, generator=g).bfloat16().half()
    logits = torch.randn(T, NE, generator=g) + torch.linspace(2, -2, NE)      # skewed: some experts get many tokens
    tv, sel = logits.topk(topk, dim=1)
    rw = torch.softmax(tv, 1).half()
    rw[7, 1] = 0
    xd, seld, rwd = x.cuda(), sel.cuda(), rw.cuda()
    y_lib = prefill_library(L, xd, seld, rwd, R=64, G=3)
    hits.zero_()
    y = L.prefill(xd, seld, rwd)
    torch.cuda.synchronize()
    assert layer_errors(y.cpu().numpy(), y_lib.cpu().numpy())[1] <= 1e-4       # fused GEMM == library GEMM on decoded weights
    want_hits = torch.bincount(sel[rw != 0].reshape(-1), minlength=NE).tolist()
    assert hits.tolist() == want_hits
    ref = O.moe_ref([expert_to_oracle(e) for e in exs], levels, x.numpy(), sel.numpy(), rw.numpy())
    ma, rl = layer_errors(y.cpu().numpy(), ref)
    assert ma <= MAX_ABS_TOL and rl <= REL_L2_TOL and rl <= 5e-4, (ma, rl)
    L.hits_ptr = 0
    ys = torch.cat([L(xd[i:i + 32], seld[i:i + 32], rwd[i:i + 32]).clone() for i in range(0, T, 32)])
    ma2, rl2 = layer_errors(y.cpu().numpy(), ys.cpu().numpy())
    assert rl2 <= 5e-4, rl2                       # same math, different fp32 accumulation order


def test_prefill_glm_shape_fused_matches_library_gemm():
    """Full-size expert shape (H 6144, I 2048, top-8), 32 experts, 1024 tokens: ~256 tokens per expert as in the
    8192-token prefill of the 256-expert layer.  The fused GEMM must agree with the library GEMM on the decoded
    weights, be deterministic, and scale linearly in the routing weights."""
    from nestquant_b200 import synth
    cfg = dict(synth.GLM); cfg["E"] = 32
    levels = [4] * 24 + [2] * 6 + [0] * 2
    L, _ = synth.build_layer(cfg, levels, seed=11, Bmax=1, masked={3, 17})
    T = 1024
    sel, rw = synth.routing(T, cfg["E"], cfg["topk"], 12)
    x = synth.tokens(T, cfg["H"], 13).cuda()
    sel, rw = sel.cuda(), rw.cuda()
    y_lib = prefill_library(L, x, sel, rw)
    y = L.prefill(x, sel, rw)
    y2 = L.prefill(x, sel, rw)
    yh = L.prefill(x, sel, (rw.float() * 0.5).half())
    torch.cuda.synchronize()
    assert torch.equal(y, y2)
    ma, rl = layer_errors(y.cpu().numpy(), y_lib.cpu().numpy())
    assert rl <= 1e-4 and ma <= MAX_ABS_TOL, (ma, rl)
    assert layer_errors((2 * yh).cpu().numpy(), y.cpu().numpy())[1] <= 1e-3      # halving fp16 weights is exact up to subnormals


def test_prefill_glm_shape_against_the_oracle():
    """Full-size expert shape (H 6144, I 2048, top-8): 1024 tokens through the fused prefill, 24 of them (every expert level
    and the masked experts among their picks) checked against the CPU oracle, which decodes the whole experts."""
    from nestquant_b200 import synth
    from tests.util import layer_report
    cfg = dict(synth.GLM); cfg["E"] = 12
    levels = [4] * 7 + [2] * 4 + [0]
    L, experts = synth.build_layer(cfg, levels, seed=21, Bmax=1, masked={2, 5})
    T, S = 1024, 24
    sel, rw = synth.routing(T, cfg["E"], cfg["topk"], 22)
    x = synth.tokens(T, cfg["H"], 23)
    y = L.prefill(x.cuda(), sel.cuda(), rw.cuda())
    torch.cuda.synchronize()
    assert L.prefill_status() == 0
    exs_o = [expert_to_oracle(experts[e]) if e in experts else None for e in range(cfg["E"])]
    ref = O.moe_ref(exs_o, levels, x[:S].numpy(), sel[:S].numpy(), rw[:S].numpy())
    rep = layer_report(y[:S].cpu().numpy(), ref)
    assert rep["max_abs_unit_rms"] <= MAX_ABS_TOL and rep["rel_l2"] <= REL_L2_TOL and rep["rel_l2"] <= 5e-4, rep


def test_prefill_many_tokens_per_expert():
    """Experts with more tokens than one pass holds (384) and than one MMA is wide (256): several passes per expert,
    token tiles cut in two column halves; against the library-GEMM path and the oracle."""
    from nestquant_b200 import moe
    H, I, NE, topk, T = 256, 384, 3, 2, 900
    exs = [moe.Expert(H, I, seed=820 + i, rk_gu=(0, 6, 0)[i], rk_dn=7, var=True, sv=0.02) for i in range(NE)]
    L = moe.MoELayer(NE, H, I, Bmax=1, topk=topk)
    levels = [4, 2, 4]
    for e in range(NE):
        L.set(e, exs[e], levels[e])
    g = torch.Generator().manual_seed(5)
    x = torch.randn(T, H, generator=g).bfloat16().half()
    logits = torch.randn(T, NE, generator=g) + torch.tensor([1.5, 0.0, -0.5])
    tv, sel = logits.topk(topk, dim=1)
    rw = torch.softmax(tv, 1).half()
    counts = torch.bincount(sel.reshape(-1), minlength=NE).tolist()
    assert max(counts) > 768 and any(256 < c <= 384 for c in counts), counts      # 3 passes for one expert, a split tile for another
    xd, seld, rwd = x.cuda(), sel.cuda(), rw.cuda()
    y_lib = prefill_library(L, xd, seld, rwd)
    y = L.prefill(xd, seld, rwd)
    torch.cuda.synchronize()
    assert layer_errors(y.cpu().numpy(), y_lib.cpu().numpy())[1] <= 1e-4
    ref = O.moe_ref([expert_to_oracle(e) for e in exs], levels, x.numpy(), sel.numpy(), rw.numpy())
    ma, rl = layer_errors(y.cpu().numpy(), ref)
    assert ma <= MAX_ABS_TOL and rl <= 5e-4, (ma, rl)


def test_pf_helpers_reject_bad_sizes():
    from nestquant_b200 import ext
    from nestquant_b200.capi import NestQuantError
    t = torch.zeros(4, 20, dtype=torch.int64, device="cuda")
    x = torch.zeros(2, 256, dtype=torch.float16, device="cuda")
    idx = torch.zeros(3, dtype=torch.int32, device="cuda")
    with pytest.raises(NestQuantError):
        ext.pf_pre(x, idx, idx, t, x, x, torch.zeros(3, 4, device="cuda"), 128)       # xg too small for 3 pairs
    with pytest.raises(NestQuantError):
        ext.pf_pre(x.float(), idx, idx, t, x, x, torch.zeros(3, 4, device="cuda"), 128)


def test_pair_sort_is_a_stable_counting_sort():
    """nq_pf_sort against torch's stable argsort of the same keys: live picks by expert in pick order, then everything that
    contributes nothing (padding ids, experts that are not resident, zero weights); hit counts as the reference counts them"""
    from nestquant_b200 import ext, moe
    H, I, NE, topk, T = 256, 128, 37, 5, 1111           # 5555 picks: 22 slices, the last one ragged
    exs = [moe.Expert(H, I, seed=i, sv=0.02) for i in range(3)]
    L = moe.MoELayer(NE, H, I, Bmax=1, topk=topk)
    for e in range(NE):
        L.set(e, exs[e % 3], 0 if e % 7 == 3 else 2)
    g = torch.Generator().manual_seed(3)
    sel = torch.randint(-2, NE + 2, (T, topk), generator=g)
    rw = torch.rand(T, topk, generator=g).half()
    rw[torch.rand(T, topk, generator=g) < 0.1] = 0
    P = T * topk
    mk = lambda n: torch.empty(n, dtype=torch.int32, device="cuda")
    pe, pt, pos, start = mk(P), mk(P), mk(P), mk(NE + 2)
    hits = torch.zeros(NE, dtype=torch.int32, device="cuda")
    ext.pf_sort(sel.cuda(), rw.cuda(), L.table, pe, pt, pos, start, hits, mk(ext.pf_sort_scratch_ints(P, NE)))
    torch.cuda.synchronize()
    flat, rwf = sel.reshape(-1), rw.reshape(-1)
    valid = (flat >= 0) & (flat < NE) & (rwf != 0)
    level = L.table[:, 0].cpu()
    live = valid & (level[flat.clamp(0, NE - 1)] > 0)
    key = torch.where(live, flat, NE)
    order = torch.argsort(key, stable=True)
    assert torch.equal(pe.cpu().long(), key[order]) and torch.equal(pt.cpu().long(), order // topk)
    inv = torch.empty(P, dtype=torch.long)
    inv[order] = torch.arange(P)
    assert torch.equal(pos.cpu().long(), inv)
    want_start = torch.zeros(NE + 2, dtype=torch.long)
    want_start[1:] = torch.cumsum(torch.bincount(key, minlength=NE + 1), 0)
    assert torch.equal(start.cpu().long(), want_start)
    assert torch.equal(hits.cpu().long(), torch.bincount(flat[valid], minlength=NE))
