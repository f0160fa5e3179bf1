"""Bit-exactness of the CUDA trellis decoder (through the C ABI) against the golden fixtures and the CPU oracle.
Mirrors the reference's sm120/verify_ext.py part (b): every residual window code, dense and mask mode, ring signs,
levels 2 and 4, and every valid block word."""
import numpy as np
import pytest
import torch

from oracle import nq_oracle as O
from tests.golden_io import load, proj_from
from tests.util import f16_bits, proj_to_oracle, same_fp16_bits

pytestmark = pytest.mark.gpu


def _dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a).copy())
    return t.cuda() if dtype is None else t.view(dtype).cuda()


def _decode_gu(planes, level, nm):
    """decode an [N, K] projection by presenting it as the gate|up part of an expert with H = K, 2I = N"""
    from nestquant_b200 import ext
    keep = [_dev(planes.base), _dev(planes.p4), _dev(planes.d4),
            None if planes.flags is None else _dev(planes.flags), None if planes.var is None else _dev(planes.var)]
    row = torch.zeros(1, 20, dtype=torch.int64)
    row[0, 0] = level
    for i, t in enumerate(keep[:4]):
        row[0, 1 + i] = 0 if t is None else t.data_ptr()
    row[0, 10] = planes.rk
    row[0, 19] = planes.bk
    row[0, 12] = 0 if keep[4] is None else keep[4].data_ptr()
    table = row.cuda()
    W = torch.full((planes.N, planes.K), float("nan"), dtype=torch.float16, device="cuda")
    ext.pf_decode(table, torch.zeros(1, dtype=torch.int32, device="cuda"), W, None, planes.K, planes.N // 2, nm, 0)
    torch.cuda.synchronize()
    return f16_bits(W)


def test_golden_projections_bit_exact():
    z = load("decode.npz")
    n = 0
    for i in range(int(z["ncases"][0])):
        p = proj_from(z, f"case{i}.")
        for level in (2, 4):
            got = _decode_gu(p, level, p.nm)
            assert same_fp16_bits(got, z[f"case{i}.W{level}"]) == 0, (i, level)
            n += 1
    assert n >= 32


@pytest.mark.parametrize("rk", range(10))
def test_random_projection_vs_oracle(rk):
    from nestquant_b200 import moe
    gen = torch.Generator().manual_seed(40 + rk)
    for nm in (None, 3):
        p = moe.Proj(256, 1024, gen, nm=nm, rk=rk, mbn=("exh", rk * 3000), var=rk % 2 == 0)
        po = proj_to_oracle(p)
        for level in (2, 4):
            got = _decode_gu(po, level, nm or 0)
            assert same_fp16_bits(got, O.decode_proj(po, level)) == 0, (rk, nm, level)


@pytest.mark.parametrize("rk", (3, 9))
def test_pattern_rate_base_vs_oracle(rk):
    """base window code 1 (1.75 bits per weight, 112-bit records in the sub-array layout) with the residual codes it ships
    with (sm120/NQ_RES_V2.md), dense and mask mode"""
    from nestquant_b200 import moe
    gen = torch.Generator().manual_seed(70 + rk)
    for nm in (None, 2):
        p = moe.Proj(256, 1024, gen, nm=nm, rk=rk, mbn=("exh", rk * 2500), var=True, bk=1)
        po = proj_to_oracle(p)
        for level in (2, 4):
            got = _decode_gu(po, level, nm or 0)
            assert same_fp16_bits(got, O.decode_proj(po, level)) == 0, (rk, nm, level)


def test_full_experts_every_block_word():
    """GLM-shaped experts (H 6144, I 2048), production codes gate|up 0 / down 7; the two experts together hold every
    valid (Mb, N) block word."""
    from nestquant_b200 import ext, moe
    H, I = 6144, 2048
    units = (2 * I // 16) * (H // 128) + (H // 16) * (I // 128)
    exs = [moe.Expert(H, I, seed=5 + i, rk_gu=0, rk_dn=7, mbn=("exh", i * units), var=True) for i in range(2)]
    words = set()
    for ex in exs:
        for p in (ex.gu, ex.dn):
            words |= set((p.Mb.cpu() * 256 + p.Nn.cpu()).tolist())
    assert len(words) == len(moe.all_MbN()) == 33149
    L = moe.MoELayer(2, H, I)
    for i, ex in enumerate(exs):
        L.set(i, ex, 4)
    Wgu = torch.empty(2 * I, H, dtype=torch.float16, device="cuda")
    Wdn = torch.empty(H, I, dtype=torch.float16, device="cuda")
    for i, ex in enumerate(exs):
        ids = torch.full((1,), i, dtype=torch.int32, device="cuda")
        for level in (4, 2) if i == 0 else (4,):
            Wgu.fill_(float("nan")); Wdn.fill_(float("nan"))
            ext.pf_decode(L.table, ids, Wgu, Wdn, H, I, 0, 0, level)
            torch.cuda.synchronize()
            assert same_fp16_bits(f16_bits(Wdn), O.decode_proj(proj_to_oracle(ex.dn), level)) == 0
            assert same_fp16_bits(f16_bits(Wgu), O.decode_proj(proj_to_oracle(ex.gu), level)) == 0


def test_level0_decodes_to_zero_and_bad_args_raise():
    from nestquant_b200 import ext
    from nestquant_b200.capi import NestQuantError
    table = torch.zeros(2, 20, dtype=torch.int64, device="cuda")
    W = torch.full((256, 128), 1.0, dtype=torch.float16, device="cuda")
    ext.pf_decode(table, torch.tensor([1], dtype=torch.int32, device="cuda"), W, None, 128, 128, 0, 0)
    torch.cuda.synchronize()
    assert not W.any()
    with pytest.raises(NestQuantError):
        ext.pf_decode(table, torch.tensor([1], dtype=torch.int32, device="cuda"), W, None, 100, 128, 0, 0)
    with pytest.raises(NestQuantError):
        ext.pf_decode(table, torch.tensor([1], dtype=torch.int32, device="cuda"), W[:1], None, 128, 128, 0, 0)
