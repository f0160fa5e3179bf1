"""Test helpers: package objects (torch tensors) -> the oracle's plain numpy containers, and comparison helpers."""
import numpy as np
import torch

from oracle.nq_oracle import ExpertPlanes, ProjPlanes


def np_u8(t):
    return None if t is None else t.detach().cpu().contiguous().view(torch.uint8).numpy().copy()


def proj_to_oracle(p) -> ProjPlanes:
    return ProjPlanes(N=p.N, K=p.K, base=np_u8(p.base), p4=np_u8(p.p4), d4=np_u8(p.d4).view(np.uint32),
                      flags=None if p.flags is None else np_u8(p.flags).view(np.uint64),
                      var=None if p.var is None else np_u8(p.var), nm=p.z["nm"] or 0, rk=p.rk, bk=p.bk)


def expert_to_oracle(ex) -> ExpertPlanes:
    o = ExpertPlanes(H=ex.H, I=ex.I, gu=proj_to_oracle(ex.gu), dn=proj_to_oracle(ex.dn),
                     scales=np_u8(ex.signs).view(np.uint16), had_dn=int(getattr(ex, "had_dn", 128) or 128))
    if getattr(ex, "lr", None) is not None:
        o.lr, o.lr4, o.rg, o.rd = np_u8(ex.lr).view(np.uint16), np_u8(ex.lr4).view(np.uint16), ex.rg, ex.rd
    return o


def same_fp16_bits(a: np.ndarray, b: np.ndarray):
    """bitwise equality of fp16 patterns, +0 and -0 counted equal; returns the number of mismatches"""
    a, b = a.view(np.uint16), b.view(np.uint16)
    bad = (a != b) & (((a | b) & 0x7FFF) != 0)
    return int(bad.sum())


def f16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)
