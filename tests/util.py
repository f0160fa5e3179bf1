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


class _Obj:
    pass


def expert_to_device(o: ExpertPlanes, dev="cuda"):
    """oracle containers -> an object shaped like nestquant_b200.moe.Expert (device tensors), for moe.entry / MoELayer.set"""
    def proj(p):
        q = _Obj()
        q.N, q.K, q.rk, q.bk = p.N, p.K, p.rk, p.bk
        q.z = dict(nm=p.nm if p.flags is not None else None)
        t = lambda a: None if a is None else torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).copy()).to(dev)
        q.base, q.p4, q.d4, q.var = t(p.base), t(p.p4), t(p.d4), t(p.var)
        q.flags = None if p.flags is None else torch.from_numpy(p.flags.view(np.int64).copy()).to(dev)
        return q
    ex = _Obj()
    ex.H, ex.I, ex.gu, ex.dn = o.H, o.I, proj(o.gu), proj(o.dn)
    ex.signs = torch.from_numpy(o.scales.view(np.float16).copy()).to(dev)
    ex.had_dn = o.had_dn
    ex.lr = ex.lr4 = None
    ex.rg = ex.rd = 0
    if o.lr is not None:
        ex.lr = torch.from_numpy(o.lr.view(np.float16).copy()).to(dev)
        ex.lr4 = torch.from_numpy(o.lr4.view(np.float16).copy()).to(dev)
        ex.rg, ex.rd = o.rg, o.rd
    return ex


def layer_errors(got: np.ndarray, ref: np.ndarray):
    """(max abs error in units of the output scale, relative L2 error).

    The synthetic layers (N(0,1) activations, |N(0,0.02)| output scales) produce outputs with an RMS of 10-20 and
    isolated values of several hundred at the GLM shape, so the absolute bound is applied to outputs normalised to
    unit RMS: max|got - ref| / max(1, rms(ref))."""
    ref64 = ref.astype(np.float64)
    d = got.astype(np.float64) - ref64
    scale = max(1.0, float(np.sqrt((ref64 ** 2).mean())))
    return float(np.abs(d).max()) / scale, float(np.linalg.norm(d) / max(np.linalg.norm(ref64), 1e-30))


def layer_report(got: np.ndarray, ref: np.ndarray) -> dict:
    """every reading of the layer-output error at once: raw max |got - ref|, the same on unit-RMS outputs, relative L2,
    and the RMS of the reference (so that the raw figure can be judged)"""
    ref64 = ref.astype(np.float64)
    d = got.astype(np.float64) - ref64
    rms = float(np.sqrt((ref64 ** 2).mean()))
    raw = float(np.abs(d).max()) if d.size else 0.0
    return dict(max_abs_raw=raw, max_abs_unit_rms=raw / max(1.0, rms), rel_l2=float(np.linalg.norm(d) / max(np.linalg.norm(ref64), 1e-30)),
                ref_rms=rms)


# layer-output tolerance of the path (fp16 operands, fp32 accumulate-order tolerance): max-abs 1e-2 (on unit-RMS
# outputs) and relative L2 2e-3
MAX_ABS_TOL, REL_L2_TOL = 1e-2, 2e-3
