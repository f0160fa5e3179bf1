"""CPU-side checks: the shared library loads and exports every symbol the header declares; host-side format helpers."""
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from nestquant_b200 import build, capi
    build.build()
    lib = capi.lib()
    hdr = open(os.path.join(ROOT, "include", "nestquant_b200.h")).read()
    declared = set(re.findall(r"\b(nq_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "no declarations found"
    assert declared == set(capi.SIGNATURES), (declared ^ set(capi.SIGNATURES))
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.nq_build_arch() == 100


def test_format_queries_need_no_gpu():
    from nestquant_b200 import ext, moe
    assert ext.rk_codes() == [1023, 1023] and ext.bk_codes() == [3, 3]
    lib = __import__("nestquant_b200.capi", fromlist=["lib"]).lib()
    for c in range(10):
        assert lib.nq_plane_bytes(12288 * 32, c) == moe.proj_sizes(4096, 6144, None, c)["p4"]
    assert lib.nq_plane_bytes(32, 10) == 0
    w = ext.moe_workspace(4, 8, 6144, 2048, 2, 1)
    assert w["acc_gu_floats"] == 2 * 32 * 4096 and w["acc_d_floats"] == 32 * 6144 and w["wq_ints"] == 4 and w["cnt_gu_ints"] == 2 * 32 * 16 + 32
    from nestquant_b200.capi import NestQuantError
    with pytest.raises(NestQuantError):
        ext.moe_workspace(33, 8, 6144, 2048, 1, 1)
    with pytest.raises(NestQuantError):
        ext.moe_workspace(4, 8, 6144, 2048, 5, 1)


def test_plane_sizes_match_the_reference_byte_counts():
    """GLM expert, gate|up code 0 / down code 7: 9,455,616 B at level 2 and 19,458,052 B at level 4"""
    from nestquant_b200 import moe
    H, I = 6144, 2048
    gu, dn = moe.proj_sizes(2 * I, H, None, 0), moe.proj_sizes(H, I, None, 7)
    l2 = gu["base"] + dn["base"] + gu["S"] * gu["C"] + dn["S"] * dn["C"]
    l4 = l2 + gu["p4"] + gu["d4"] + dn["p4"] + dn["d4"]
    assert (l2, l4) == (9455616, 19458052)
    m = moe.proj_sizes(2 * I, H, H // 128 // 2, 0), moe.proj_sizes(H, I, I // 128 // 2, 7)
    assert l2 + sum(z["p4"] + z["d4"] + z["flags"] for z in m) == 14461956


def test_pack_unpack_round_trip_and_golden():
    from nestquant_b200 import moe
    from tests.golden_io import load
    z = load("pack.npz")
    for c in range(10):
        b = moe.rbits(c)
        for n in (32, 160):
            w = torch.from_numpy(z[f"c{c}.n{n}.words"].astype(np.int64))
            packed = moe.pack_words(w, b)
            assert np.array_equal(packed.view(torch.uint8).numpy(), z[f"c{c}.n{n}.packed"]), (c, n)
            assert torch.equal(moe.unpack_words(packed, n, b), w)


def test_generators_are_seeded_and_well_formed():
    from nestquant_b200 import moe
    a = moe.Expert(256, 128, seed=5, nm_gu=1, nm_dn=1, dev="cpu", rk_gu=6, rk_dn=7, var=True, sv=0.02)
    b = moe.Expert(256, 128, seed=5, nm_gu=1, nm_dn=1, dev="cpu", rk_gu=6, rk_dn=7, var=True, sv=0.02)
    for p, q in ((a.gu, b.gu), (a.dn, b.dn)):
        assert torch.equal(p.base, q.base) and torch.equal(p.p4, q.p4) and torch.equal(p.d4, q.d4) and torch.equal(p.flags, q.flags)
        Mb, N = p.d4 & 255, (p.d4 >> 8) & 255
        assert int(Mb.min()) >= 1 and int((Mb + N).max()) <= 257
        assert p.p4.numel() * 4 == p.z["p4"]
        S = p.N // 16
        fl = p.fl.view(-1, 8, p.K // 128) if S % 8 == 0 else None
        if fl is not None:
            assert bool((fl == fl[:, :1]).all())            # flags uniform over each group of 8 strips
        assert int(p.fl.sum(1).min()) == int(p.fl.sum(1).max()) == p.z["nm"]
    s = a.signs.float()
    H, I = 256, 128
    assert set(s[:H].abs().tolist()) == {1.0} and float(s[H:H + 2 * I].max()) < 0.2
    e = moe.entry(a, 4)
    assert e[0] == 4 and e[10] == 6 and e[11] == 7 and e[1] == a.gu.base.data_ptr() and e[18] == 0 and e[19] == 0


def test_default_ksplit_divides_the_chunks_for_every_shape():
    """the k-split rule of the decode call: both numbers divide the chunk counts (a workspace can be sized for them) for the
    GLM shape, its tensor-parallel shards, small test shapes and expert-parallel shares; the tuned points stay put"""
    from nestquant_b200 import ext
    for H in (128, 1024, 4096, 6144, 8192):
        for I in (128, 256, 512, 1024, 1536, 2048, 8192):
            for B in (1, 2, 3, 4, 8, 16, 32):
                for share in (1.0, 0.5, 0.25, 0.125):
                    for topk in (1, 4, 8):
                        g, d = ext.default_ksplit(B, H, I, share, topk)
                        assert 1 <= g <= 24 and 1 <= d <= 24 and (H // 128) % g == 0 and (I // 128) % d == 0, (B, H, I, share, topk, g, d)
    assert ext.default_ksplit(1, 6144, 2048) == (4, 2) and ext.default_ksplit(2, 6144, 2048) == (2, 1)
    assert ext.default_ksplit(32, 6144, 2048) == (1, 1) and ext.default_ksplit(1, 6144, 256) == (12, 1)
    assert ext.default_ksplit(1, 6144, 2048, 0.125) == (8, 4)
