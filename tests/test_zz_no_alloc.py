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
    H, I, NE, topk, B = 1024, 512, 8, 4, 3
    levels = [4, 2, 4, 4, 2, 0, 4, 2]
    exs = [moe.Expert(H, I, seed=900 + i, rk_gu=(0, 6)[i % 2], rk_dn=7, var=True, sv=0.02) for i in range(NE)]
    L = moe.MoELayer(NE, H, I, Bmax=B, topk=topk)
    for e in range(NE):
        L.set(e, exs[e], levels[e])
    ks = ext.default_ksplit(B, H, I)
    rng = random.Random(3)
    gen = torch.Generator().manual_seed(8)
    out = torch.full((B, H), float("nan"), dtype=torch.float32, device="cuda")
    for call in range(2):                      # the second call finds the array as the first one left it
        sel = torch.tensor([rng.sample(range(NE), topk) for _ in range(B)]).cuda()
        rw = torch.softmax(torch.randn(B, topk, generator=gen), 1).half().cuda()
        x = torch.randn(B, H, generator=gen).bfloat16().half().cuda()
        want = L(x, sel, rw).clone()
        out.fill_(float("nan"))
        ext.moe_forward_static(x, sel, rw, L.table, out, I, 0, 0, ks[0], ks[1])
        torch.cuda.synchronize()
        ma, rl = layer_errors(out.cpu().numpy(), want.cpu().numpy())
        assert ma <= MAX_ABS_TOL and rl <= REL_L2_TOL, (call, ma, rl)
        assert torch.equal(out, want), f"call {call}: same kernels, same summation order - expected identical bits"
    # a shape whose workspaces exceed the built-in array is refused with a clear message, before anything is launched
    assert lib().nq_moe_static_scratch_bytes() == 4 << 20
    big = torch.zeros(32, 6144, dtype=torch.float16, device="cuda")
    with pytest.raises(NestQuantError, match="built-in array"):
        ext.moe_forward_static(big, torch.zeros(32, 8, dtype=torch.long, device="cuda"),
                               torch.zeros(32, 8, dtype=torch.float16, device="cuda"),
                               torch.zeros(256, 20, dtype=torch.int64, device="cuda"),
                               torch.zeros(32, 6144, dtype=torch.float32, device="cuda"), 2048, 0, 0, 1, 1)
