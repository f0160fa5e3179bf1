"""Every window code through the hot kernels themselves.

(a) Layer outputs of the decode path and of the fused prefill for each of the ten residual codes (both projections, dense
    and mask mode) against the oracle: the reference's sm120/verify_ext.py part (b) covers every compiled code this way.
(b) The decoder inside the decode-path kernel and inside the fused prefill GEMM, bit for bit: fed one-hot inputs, the
    kernels' own fp32 sums hold columns of the decoded weight matrices exactly (a product of two fp16 numbers is exact in
    fp32 and every other term is zero), so they can be compared bitwise with the oracle's dense decode - the role of the
    reference's NQ_WDUMP hook (sm120/nqmoe.cu:246-248,852-853)."""
import random

import numpy as np
import pytest
import torch

from oracle import nq_oracle as O
from tests.util import MAX_ABS_TOL, REL_L2_TOL, expert_to_oracle, layer_errors, same_fp16_bits

pytestmark = pytest.mark.gpu


def _routing(B, E, topk, rng):
    sel = torch.tensor([rng.sample(range(E), topk) for _ in range(B)], dtype=torch.long)
    g = torch.Generator().manual_seed(rng.randrange(1 << 30))
    w = torch.rand(sel.shape, generator=g) + 0.1
    return sel, (w / w.sum(1, keepdim=True)).half()


@pytest.mark.parametrize("rk", range(10))
def test_layer_outputs_for_every_residual_code(rk):
    """dense and masked level-4 experts whose gate|up AND down planes use residual code rk, beside a level-2 expert"""
    from nestquant_b200 import moe
    H, I, NE, topk = 768, 384, 4, 2
    nmg, nmd = 3, 1
    exs = [moe.Expert(H, I, seed=4000 + 10 * rk + i, nm_gu=nmg if i == 1 else None, nm_dn=nmd if i == 1 else None,
                      rk_gu=rk, rk_dn=rk, var=i != 2, sv=0.02) for i in range(NE)]
    levels = [4, 4, 4, 2]
    exs_o = [expert_to_oracle(e) for e in exs]
    L = moe.MoELayer(NE, H, I, nmg, nmd, Bmax=12, topk=topk)
    for e in range(NE):
        L.set(e, exs[e], levels[e])
    rng = random.Random(rk)
    gen = torch.Generator().manual_seed(100 + rk)
    for B in (1, 5, 12):
        sel, rw = _routing(B, NE, topk, rng)
        x = torch.randn(B, H, generator=gen).bfloat16().half()
        ref = O.moe_ref(exs_o, levels, x.numpy(), sel.numpy(), rw.numpy())
        y = L(x.cuda(), sel.cuda(), rw.cuda())
        torch.cuda.synchronize()
        ma, rl = layer_errors(y.cpu().numpy(), ref)
        assert ma <= MAX_ABS_TOL and rl <= REL_L2_TOL and rl <= 5e-4, ("decode path", rk, B, ma, rl)
    assert L.status() == 0
    T = 70
    sel, rw = _routing(T, NE, topk, rng)
    x = torch.randn(T, H, generator=gen).bfloat16().half()
    ref = O.moe_ref(exs_o, levels, x.numpy(), sel.numpy(), rw.numpy())
    y = L.prefill(x.cuda(), sel.cuda(), rw.cuda())
    torch.cuda.synchronize()
    ma, rl = layer_errors(y.cpu().numpy(), ref)
    assert ma <= MAX_ABS_TOL and rl <= REL_L2_TOL and rl <= 5e-4, ("prefill", rk, ma, rl)


def _hadamard128():
    i = np.arange(128)
    return np.where(np.vectorize(lambda v: bin(v).count("1") & 1)(i[:, None] & i[None, :]), -1.0, 1.0).astype(np.float32)


# (residual code gate|up, residual code down, base code, level, masked)
CASES = [(rk, rk, 0, 4, False) for rk in range(10)] + [(0, 7, 0, 2, False), (6, 7, 0, 4, True), (3, 9, 1, 4, False),
                                                         (3, 9, 1, 2, False), (9, 3, 1, 4, True)]


@pytest.mark.parametrize("rk_gu,rk_dn,bk,level,masked", CASES)
@pytest.mark.parametrize("B", [8, 32])
def test_decode_path_kernel_decodes_bit_exactly(rk_gu, rk_dn, bk, level, masked, B):
    """columns of W_gate|up and W_down read back from the split-k partial sums of the decode-path kernel (8 tokens: one
    column tile per run; 32 tokens: four)"""
    from nestquant_b200 import ext, moe
    H, I = 384, 256
    nmg, nmd = (2, 1) if masked else (None, None)
    ex = moe.Expert(H, I, seed=5000 + 31 * rk_gu + rk_dn + 7 * bk + level, nm_gu=nmg, nm_dn=nmd, rk_gu=rk_gu, rk_dn=rk_dn, var=True,
                    sv=0.02, bk_gu=bk, bk_dn=bk)
    eo = expert_to_oracle(ex)
    Wgu, Wdn = O.decode_proj(eo.gu, level), O.decode_proj(eo.dn, level)          # fp16 [2I, H], [H, I]
    L = moe.MoELayer(2, H, I, nmg or 0, nmd or 0, Bmax=B, topk=1)
    L.set(1, ex, level)
    ks = ext.default_ksplit(B, H, I)
    sel = torch.ones(B, 1, dtype=torch.long, device="cuda")
    rw = torch.ones(B, 1, dtype=torch.float16, device="cuda")
    Hm = _hadamard128()
    signs = ex.signs.float().cpu().numpy()
    su = {0: signs[:H], 1: signs[2 * H + 3 * I:]}
    scale = float(np.float16(np.float32(128.0) * np.float32(0.08838834764831845)))   # fp16(WHT128 of a matching +-1 row)
    for up in (0, 1):                                     # gate rows need x built from su_g, up rows from su_u
        for k0 in range(0, H, B):
            x = np.zeros((B, H), np.float32)
            for b in range(B):
                k = k0 + b
                blk = k // 128
                x[b, blk * 128:(blk + 1) * 128] = su[up][blk * 128:(blk + 1) * 128] * Hm[k % 128]
            L(torch.from_numpy(x).half().cuda(), sel, rw, which=1)
            torch.cuda.synchronize()
            part = L.acc_gu[:ks[0] * B * 2 * I].view(ks[0], B, 2 * I).double().sum(0).cpu().numpy()      # [B, 2I]
            got = (part[:, up * I:(up + 1) * I] / scale).astype(np.float32)
            assert np.array_equal(got.astype(np.float16).astype(np.float32), got), "not an fp16 value: the input was not one-hot"
            want = Wgu[up * I:(up + 1) * I, k0:k0 + B].T
            assert same_fp16_bits(got.astype(np.float16), np.ascontiguousarray(want)) == 0, (up, k0)
    pos = ext.operand_order(I)
    for k0 in range(0, I, B):
        h = torch.zeros(B, I, dtype=torch.float16)
        for b in range(B):
            h[b, pos[k0 + b]] = 1.0
        L.h[:B * I].copy_(h.reshape(-1).cuda())
        L(torch.zeros(B, H, dtype=torch.float16, device="cuda"), sel, rw, which=2)
        torch.cuda.synchronize()
        got = L.acc_d[:ks[1] * B * H].view(ks[1], B, H).double().sum(0).cpu().numpy().astype(np.float32)
        want = Wdn[:, k0:k0 + B].T
        assert same_fp16_bits(got.astype(np.float16), np.ascontiguousarray(want)) == 0, ("down", k0)
        assert np.array_equal(got.astype(np.float16).astype(np.float32), got)
    assert L.status() == 0
    for t in (L.cnt_gu, L.cnt_d, L.wq):
        assert int(t.abs().sum()) == 0


@pytest.mark.parametrize("rk_gu,rk_dn,bk,level,masked", CASES)
def test_fused_prefill_gemm_decodes_bit_exactly(rk_gu, rk_dn, bk, level, masked):
    """one-hot activation rows (one pair per k, all routed to one expert): the GEMM outputs are the weight columns"""
    from nestquant_b200 import ext, moe
    H, I = 512, 384                                    # 512 pairs for gate|up: two passes (384 + 128)
    nmg, nmd = (2, 1) if masked else (None, None)
    ex = moe.Expert(H, I, seed=6000 + 31 * rk_gu + rk_dn + 7 * bk + level, nm_gu=nmg, nm_dn=nmd, rk_gu=rk_gu, rk_dn=rk_dn, var=True,
                    sv=0.02, bk_gu=bk, bk_dn=bk)
    eo = expert_to_oracle(ex)
    Wgu, Wdn = O.decode_proj(eo.gu, level), O.decode_proj(eo.dn, level)
    E = 3
    L = moe.MoELayer(E, H, I, nmg or 0, nmd or 0, Bmax=1, topk=1)
    L.set(1, ex, level)
    dev = "cuda"
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for down in (False, True):
        K, N = (I, H) if down else (H, I)
        P = K
        cnt = torch.tensor([0, P, 0], dtype=torch.int32, device=dev)
        plan = torch.empty(ext.pf_plan_ints(E, P), dtype=torch.int32, device=dev)
        ext.pf_plan(cnt, L.table, plan, P)
        act = torch.zeros(P, K, dtype=torch.float16)
        act[torch.arange(P), ext.kperm_order(K)] = 1.0
        act = act.to(dev)
        out0 = torch.full((P, N), float("nan"), dtype=torch.float32, device=dev)
        out1 = torch.full((P, N), float("nan"), dtype=torch.float32, device=dev)
        ext.pf_gemm(L.table, plan, act, None if down else act, out0, None if down else out1, H, I, L.nm_gu, L.nm_dn, down, status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        if down:
            assert same_fp16_bits(out0.cpu().numpy().astype(np.float16), np.ascontiguousarray(Wdn.T)) == 0
            assert torch.equal(out0.half().float(), out0)
        else:
            assert same_fp16_bits(out0.cpu().numpy().astype(np.float16), np.ascontiguousarray(Wgu[:I].T)) == 0
            assert same_fp16_bits(out1.cpu().numpy().astype(np.float16), np.ascontiguousarray(Wgu[I:].T)) == 0
            assert torch.equal(out0.half().float(), out0) and torch.equal(out1.half().float(), out1)
