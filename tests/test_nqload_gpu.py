"""Production shards through the loader onto the GPU: the kernels' dense decode of the loaded planes against the dense
matrices of the encoder-side decoder (bit for bit), and the loaded experts through the decode path and the prefill path
against the CPU oracle.  Mirrors what the reference's sm120/smoke_layer.py does with nqload.RankLayer."""
import hashlib
import os

import numpy as np
import pytest
import torch

from oracle import nq_oracle as O
from tests.util import MAX_ABS_TOL, REL_L2_TOL, expert_to_oracle, layer_errors, layer_report

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.join(HERE, "golden", "nqload")
G = np.load(os.path.join(HERE, "golden", "nqload.npz"))


def _bits(t):
    b = t.detach().cpu().contiguous().view(torch.int16).numpy().copy()
    b[b == -32768] = 0
    return b


@pytest.mark.parametrize("E", [0, 3])
def test_kernel_decode_equals_encoder_side_decoder(E):
    from nestquant_b200 import nqload
    RL = nqload.RankLayer(ROOT, 3, 0, tp=8, dev="cuda")
    ex, scales, (Qg, Qu, Qd) = nqload.kernel_expert(RL.art(E), "cuda", want_Q=True)
    assert torch.equal(scales(4), ex.sc[4]) and not hasattr(ex, "signs")
    tag = f"L3.tp8.r0.E{E}"
    for lv in (2, 4):
        gu, dn = _bits(torch.cat([Qg[lv], Qu[lv]])), _bits(Qd[lv])
        assert gu.shape == (2 * RL.I, RL.H) and dn.shape == (RL.H, RL.I)
        np.testing.assert_array_equal(gu[:32], G[f"{tag}.Q{lv}.gu.head"])
        np.testing.assert_array_equal(dn[:32], G[f"{tag}.Q{lv}.dn.head"])
        assert hashlib.sha256(gu.tobytes()).hexdigest() == str(G[f"{tag}.Q{lv}.gu.sha"])
        assert hashlib.sha256(dn.tobytes()).hexdigest() == str(G[f"{tag}.Q{lv}.dn.sha"])


@pytest.mark.parametrize("L,tp,levels", [(3, 8, {0: 2, 3: 4}), (3, 8, {0: 4, 3: 2}), (3, 4, {0: 4, 3: 4}), (4, 8, {1: 4}), (4, 8, {1: 2})])
def test_loaded_layer_decode_and_prefill_against_oracle(L, tp, levels):
    from nestquant_b200 import moe, nqload
    RL = nqload.RankLayer(ROOT, L, 0, tp=tp, dev="cuda")          # tp 4: a group of two shards (I 512)
    E, topk = 4, 2
    M = moe.MoELayer(E, RL.H, RL.I, Bmax=4, topk=topk)
    exs_o, lv = [None] * E, [0] * E
    for e, x in RL.ex.items():
        x.signs = x.sc[levels[e]]
        M.set(e, x, levels[e])
        exs_o[e], lv[e] = expert_to_oracle(x), levels[e]
    g = torch.Generator().manual_seed(77 + L)
    live = sorted(RL.ex)
    for B in (1, 4, 24):
        x = torch.randn(B, RL.H, generator=g).half()
        sel = torch.stack([torch.tensor((live * topk)[b % len(live):][:topk]) for b in range(B)])
        if len(live) == 1:
            sel[:, 1] = 2                         # the second pick goes to an expert that is not resident
        rw = (torch.rand(B, topk, generator=g) + 0.2).half()
        ref = O.moe_ref(exs_o, lv, x.numpy(), sel.numpy(), rw.numpy())
        if B <= 4:
            y = M(x.cuda(), sel.cuda(), rw.cuda()).clone()
        else:
            y = M.prefill(x.cuda(), sel.cuda(), rw.cuda())
            assert M.prefill_status() == 0
        torch.cuda.synchronize()
        ma, rl = layer_errors(y.cpu().numpy(), ref)
        assert ma <= MAX_ABS_TOL and rl <= REL_L2_TOL, (L, levels, B, layer_report(y.cpu().numpy(), ref))
    assert M.status() == 0
