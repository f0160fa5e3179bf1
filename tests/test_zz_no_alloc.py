"""The allocation-free layer call (nq_moe_forward_static, workspaces in an array built into the library) against the
ordinary entry point with caller-owned workspaces.  Collected last on purpose: a failure here cannot hide other tests
from a run that stops at the first failure.  It needs nothing from the other tests and passes in a fresh process."""
import random

import pytest
import torch

from tests.util import MAX_ABS_TOL, REL_L2_TOL, layer_errors

pytestmark = pytest.mark.gpu


def test_static_workspace_call_matches_regular_call_twice_in_a_row():
    from nestquant_b200 import ext, moe
    from nestquant_b200.capi import NestQuantError, lib
    H, I, NE, topk = 1024, 512, 8, 4
    levels = [4, 2, 4, 4, 2, 0, 4, 2]
    exs = [moe.Expert(H, I, seed=900 + i, rk_gu=(0, 6)[i % 2], rk_dn=7, var=True, sv=0.02) for i in range(NE)]
    L = moe.MoELayer(NE, H, I, Bmax=3, topk=topk, ksplit=(4, 2))
    for e in range(NE):
        L.set(e, exs[e], levels[e])
    rng = random.Random(3)
    gen = torch.Generator().manual_seed(8)
    free_before = None
    # Every call finds the array as the previous one left it, and the shape changes from call to call, so the workspaces are
    # carved differently each time: counters of one call land on bytes that held partial sums of the call before.
    for call, (B, ks) in enumerate([(3, (2, 1)), (1, (4, 2)), (3, (2, 1)), (2, (1, 1))]):
        sel = torch.tensor([rng.sample(range(NE), topk) for _ in range(B)]).cuda()
        rw = torch.softmax(torch.randn(B, topk, generator=gen), 1).half().cuda()
        x = torch.randn(B, H, generator=gen).bfloat16().half().cuda()
        want = L(x, sel, rw, cfg_gu=[ks[0]], cfg_dn=[ks[1]]).clone()
        out = torch.full((B, H), float("nan"), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        if call == 1:
            free_before = torch.cuda.mem_get_info()[0]      # the first call is behind us: lazy loading is done
        ext.moe_forward_static(x, sel, rw, L.table, out, I, 0, 0, ks[0], ks[1])
        torch.cuda.synchronize()
        if call >= 1:
            assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the amount of free device memory"
        ma, rl = layer_errors(out.cpu().numpy(), want.cpu().numpy())
        assert ma <= MAX_ABS_TOL and rl <= REL_L2_TOL, (call, ma, rl)
        assert torch.equal(out, want), f"call {call}: same kernel, same summation order - expected identical bits"
    # a shape whose workspaces exceed the built-in array is refused with a clear message, before anything is launched
    assert lib().nq_moe_static_scratch_bytes() == 4 << 20
    big = torch.zeros(32, 6144, dtype=torch.float16, device="cuda")
    with pytest.raises(NestQuantError, match="built-in array"):
        ext.moe_forward_static(big, torch.zeros(32, 8, dtype=torch.long, device="cuda"),
                               torch.zeros(32, 8, dtype=torch.float16, device="cuda"),
                               torch.zeros(256, 20, dtype=torch.int64, device="cuda"),
                               torch.zeros(32, 6144, dtype=torch.float32, device="cuda"), 2048, 0, 0, 1, 1)


def test_static_workspace_call_at_the_full_expert_shape():
    """one token at the GLM expert shape (H 6144, I 2048) with the default k-split of a 1-token call, against the oracle;
    the same shape with four tokens fits at k-split (2, 1) and is refused at (4, 2)"""
    from nestquant_b200 import ext, moe
    from nestquant_b200.capi import NestQuantError
    from oracle import nq_oracle as O
    from tests.util import expert_to_oracle
    H, I, NE, topk = 6144, 2048, 3, 2
    exs = [moe.Expert(H, I, seed=950 + i, rk_gu=0, rk_dn=7, var=True, sv=0.02) for i in range(NE)]
    levels = [4, 2, 4]
    L = moe.MoELayer(NE, H, I, Bmax=4, topk=topk)
    for e in range(NE):
        L.set(e, exs[e], levels[e])
    gen = torch.Generator().manual_seed(9)
    x = torch.randn(1, H, generator=gen).bfloat16().half()
    sel = torch.tensor([[2, 1]])
    rw = torch.tensor([[0.625, 0.375]]).half()
    ks = ext.default_ksplit(1, H, I)
    out = torch.empty(1, H, dtype=torch.float32, device="cuda")
    ext.moe_forward_static(x.cuda(), sel.cuda(), rw.cuda(), L.table, out, I, 0, 0, ks[0], ks[1])
    torch.cuda.synchronize()
    ref = O.moe_ref([expert_to_oracle(e) for e in exs], levels, x.numpy(), sel.numpy(), rw.numpy())
    ma, rl = layer_errors(out.cpu().numpy(), ref)
    assert ma <= MAX_ABS_TOL and rl <= REL_L2_TOL and rl <= 5e-4, (ma, rl)
    x4 = torch.randn(4, H, generator=gen).bfloat16().half().cuda()
    sel4 = torch.tensor([[0, 1], [1, 2], [2, 0], [0, 2]]).cuda()
    rw4 = torch.full((4, topk), 0.5).half().cuda()
    out4 = torch.empty(4, H, dtype=torch.float32, device="cuda")
    big = moe.MoELayer(NE, H, I, Bmax=4, topk=8)           # top-8: the call shape of the full layer
    sel8 = torch.zeros(4, 8, dtype=torch.long, device="cuda")
    rw8 = torch.zeros(4, 8, dtype=torch.float16, device="cuda")
    ext.moe_forward_static(x4, sel8, rw8, big.table, out4, I, 0, 0, 2, 1)          # 4 tokens x top-8 at (2, 1): fits
    with pytest.raises(NestQuantError, match="built-in array"):
        ext.moe_forward_static(x4, sel8, rw8, big.table, out4, I, 0, 0, 4, 2)      # at (4, 2) it needs 4.6 MB
    torch.cuda.synchronize()
