"""Decode salience export (nq_salience) against the oracle: fp16 and bf16 inputs, strided rows, duplicate experts in one
call, zero-weight picks skipped, running sums over calls, host mirror."""
import numpy as np
import pytest
import torch

from oracle import nq_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_salience_running_sums(dtype):
    from nestquant_b200 import ext
    E, topk, H, rsf = 40, 8, 1536, 2.5
    g = torch.Generator().manual_seed(17)
    acc = torch.zeros(E, dtype=torch.float64, device="cuda")
    host = torch.zeros(E, dtype=torch.float64).pin_memory()
    want = np.zeros(E)
    for B in (1, 4, 8, 32):
        buf = torch.randn(B, H + 64, generator=g).to(dtype).cuda()
        x = buf[:, :H]                                     # rows strided by H + 64
        sel = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(B)])
        if B > 1:
            sel[1] = sel[0]                                # the same experts twice in one call
        rw = torch.softmax(torch.randn(B, topk, generator=g), 1).half()
        rw[0, 3] = 0                                       # skipped
        ext.sal(x, rw.cuda(), sel.cuda(), rsf, acc, host.data_ptr())
        want += O.salience_ref(x.float().cpu().numpy(), rw.numpy(), sel.numpy(), rsf, E)
    torch.cuda.synchronize()
    got = acc.cpu().numpy()
    assert np.allclose(got, want, rtol=2e-6, atol=0) and np.array_equal(host.numpy()[want != 0], got[want != 0])
    assert (got[want == 0] == 0).all()


def test_salience_rejects_bad_arguments():
    from nestquant_b200 import ext
    from nestquant_b200.capi import NestQuantError
    acc = torch.zeros(8, dtype=torch.float64, device="cuda")
    x = torch.zeros(33, 128, dtype=torch.float16, device="cuda")
    sel = torch.zeros(33, 2, dtype=torch.int64, device="cuda")
    with pytest.raises(NestQuantError):
        ext.sal(x, sel.half(), sel, 1.0, acc)              # more than 32 tokens
    with pytest.raises(NestQuantError):
        ext.sal(x[:2].float(), sel[:2].half(), sel[:2], 1.0, acc)
