"""The production-shard loader (nestquant_b200.nqload) against what the reference's own loader made of the same files
(tests/golden/make_golden_nqload.py), and the CPU oracle's decode of the loaded planes against the dense matrices of the
encoder-side decoder (an implementation independent of the kernel-side reference decode the oracle restates)."""
import hashlib
import os

import numpy as np
import pytest
import torch

from nestquant_b200 import nqload
from oracle import nq_oracle as O
from tests.util import proj_to_oracle

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.join(HERE, "golden", "nqload")
G = np.load(os.path.join(HERE, "golden", "nqload.npz"))
sha = lambda t: hashlib.sha256(t.contiguous().cpu().numpy().tobytes()).hexdigest()


def check_expert(tag, ex):
    for pj, p in (("gu", ex.gu), ("dn", ex.dn)):
        assert [p.N, p.K, p.rk, p.bk] == G[f"{tag}.{pj}.codes"].tolist()
        for k in ("base", "p4", "d4", "var"):
            t = getattr(p, k)
            assert [t.numel(), t.element_size()] == G[f"{tag}.{pj}.{k}.numel"].tolist(), (tag, pj, k)
            if f"{tag}.{pj}.{k}" in G:          # the full plane is stored for the smallest cases: says where a mismatch is
                np.testing.assert_array_equal(t.numpy(), G[f"{tag}.{pj}.{k}"], err_msg=f"{tag}.{pj}.{k}")
            assert sha(t) == str(G[f"{tag}.{pj}.{k}.sha"]), (tag, pj, k)
        assert p.flags is None and p.z == nqload.proj_sizes(p.N, p.K, None, p.rk, p.bk)
    for lv in (2, 4):
        assert sha(ex.sc[lv]) == str(G[f"{tag}.sc{lv}.sha"]), (tag, lv)
    assert [ex.rg, ex.rd, ex.H, ex.I] == G[f"{tag}.ranks"].tolist()
    if ex.rg + ex.rd:
        assert sha(ex.lr) == str(G[f"{tag}.lr.sha"]) and sha(ex.lr4) == str(G[f"{tag}.lr4.sha"])
    else:
        assert ex.lr is None and ex.lr4 is None
    assert nqload.p4_bytes(ex) == int(G[f"{tag}.p4_bytes"][0])
    assert not hasattr(ex.gu, "p4w") and not hasattr(ex.gu, "bw")


@pytest.mark.parametrize("L,tp,rank", [(3, 8, 0), (3, 8, 1), (3, 4, 0), (4, 8, 0)])
def test_rank_layer_matches_reference_loader(L, tp, rank):
    RL = nqload.RankLayer(ROOT, L, rank, tp=tp, dev="cpu")
    assert [RL.slot_bytes(), RL.H, RL.I, RL.had_dn] == G[f"L{L}.tp{tp}.r{rank}.slot_bytes"].tolist()
    assert RL.experts == {3: [0, 3], 4: [1]}[L] and RL.ss == list(range(rank * 8 // tp, (rank + 1) * 8 // tp))
    for E in RL.experts:
        check_expert(f"L{L}.tp{tp}.r{rank}.E{E}", RL.ex[E])
        assert RL.ex[E].had_dn == 128


def test_expert_filter_and_safetensors_container():
    RL = nqload.RankLayer(ROOT, 3, 0, tp=8, experts={3}, dev="cpu")
    assert RL.experts == [3] and list(RL.ex) == [3]
    # the same shard in the safetensors container under root/layers/L4
    st_root = os.path.join(HERE, "golden", "nqload_st")
    assert nqload.layer_dir(st_root, 4).endswith("layers/L4") and nqload.layer_dir(ROOT, 4).endswith("nqload/L4")
    a, b = nqload.load_part(nqload.layer_dir(ROOT, 4), 0), nqload.load_part(nqload.layer_dir(st_root, 4), 0)
    assert list(a) == list(b) and [type(k) for k in a] == [type(k) for k in b]
    for E in a:
        for pn in a[E]:
            assert list(a[E][pn]) == list(b[E][pn])
            for k, v in a[E][pn].items():
                w = b[E][pn][k]
                if torch.is_tensor(v):
                    assert v.dtype == w.dtype and v.shape == w.shape and torch.equal(v, w), (E, pn, k)
                else:
                    assert v == w
    check_expert("L4.tp8.r0.E1", nqload.RankLayer(st_root, 4, 0, tp=8, dev="cpu").ex[1])


def test_refusals():
    with pytest.raises(AssertionError):
        nqload.RankLayer(ROOT, 3, 0, tp=3, dev="cpu")
    with pytest.raises(AssertionError):
        nqload.RankLayer(ROOT, 3, 8, tp=8, dev="cpu")
    RL = nqload.RankLayer(ROOT, 3, 0, tp=8, dev="cpu")
    art = RL.art(0)
    art["gate"]["meta"]["res_rule"] = dict(kind="pos", K=2, K_hi=3, frac=0.5)
    with pytest.raises(ValueError):
        nqload.repack(art["gate"], "cpu")
    art = RL.art(3)
    art["up"]["base"]["lr"]["V"] = art["up"]["base"]["lr"]["V"] + 1
    with pytest.raises(AssertionError):
        nqload.kernel_expert(art, "cpu")
    with pytest.raises(RuntimeError):           # the dense matrices come from the GPU decode kernel
        nqload.kernel_expert(RL.art(0), "cpu", want_Q=True)


@pytest.mark.parametrize("E", [0, 3])
def test_oracle_decode_of_loaded_planes_equals_encoder_side_decoder(E):
    ex = nqload.RankLayer(ROOT, 3, 0, tp=8, dev="cpu").ex[E]
    tag = f"L3.tp8.r0.E{E}"
    for lv in (2, 4):
        for pj, p in (("gu", ex.gu), ("dn", ex.dn)):
            W = O.decode_proj(proj_to_oracle(p), lv).copy()
            W[W == 0x8000] = 0                                          # -0 counts as +0
            np.testing.assert_array_equal(W[:32].view(np.int16), G[f"{tag}.Q{lv}.{pj}.head"])
            assert hashlib.sha256(W.tobytes()).hexdigest() == str(G[f"{tag}.Q{lv}.{pj}.sha"]), (tag, lv, pj)
