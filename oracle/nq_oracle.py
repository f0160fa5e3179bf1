"""ctypes front end of the CPU oracle (oracle/nq_oracle.c) plus a tiny numpy second opinion.

TEST INFRASTRUCTURE ONLY: used by tests/, by the smoke check and by the CPU-baseline legs of the
benchmark.  The shipped package never imports this module.

The C functions restate the reference's CPU path (sm120/moe.py:109-210, sm120/ref15_spec.py); each
one cites the lines it follows.  `decode_unit_numpy` is an independent vectorised restatement of the
unit decode (sm120/ref15_spec.py:43-90) used to cross-check the C code on small inputs.
"""
import ctypes as C
import os
import subprocess
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

# window patterns per code: step p of a ring is KA + ((MASK >> (p % 16)) & 1) bits wide (sm120/moe.py:10-11)
PATTERNS = {0: (2, 0x0000), 1: (1, 0xEEEE), 2: (2, 0xAAAA), 3: (2, 0x8888), 4: (3, 0x0000), 5: (1, 0xAAAA),
            6: (1, 0xFFFE), 7: (2, 0x9248), 8: (1, 0xFEFE), 9: (2, 0xD5AA)}
HASH_MUL = 0x83DCD12D


def build(force=False):
    """Compile oracle/libnq_oracle.so with the Makefile beside this file."""
    so = os.path.join(HERE, "libnq_oracle.so")
    src = os.path.join(HERE, "nq_oracle.c")
    if force or not os.path.exists(so) or (os.path.exists(src) and os.path.getmtime(src) > os.path.getmtime(so)):
        subprocess.run(["make", "-C", HERE], check=True, capture_output=True)
    return so


def lib():
    global _LIB
    if _LIB is None:
        L = C.CDLL(build())
        u8p, u16p, u32p, u64p, f32p = (C.c_void_p,) * 5
        L.nqo_rbits.argtypes = [C.c_int]; L.nqo_rbits.restype = C.c_int
        L.nqo_plane_bytes.argtypes = [C.c_size_t, C.c_int]; L.nqo_plane_bytes.restype = C.c_size_t
        L.nqo_f2h.argtypes = [C.c_float]; L.nqo_f2h.restype = C.c_uint16
        L.nqo_h2f.argtypes = [C.c_uint16]; L.nqo_h2f.restype = C.c_float
        L.nqo_hash_sum.argtypes = [C.c_uint32]; L.nqo_hash_sum.restype = C.c_int
        L.nqo_q2.argtypes = [C.c_int, C.c_int]; L.nqo_q2.restype = C.c_uint16
        L.nqo_q4.argtypes = [C.c_int] * 5; L.nqo_q4.restype = C.c_uint16
        L.nqo_fold_consts.argtypes = [C.c_int, C.c_int, C.POINTER(C.c_uint16), C.POINTER(C.c_uint16)]
        L.nqo_fold_consts.restype = None
        L.nqo_record_words.argtypes = [u8p, C.c_size_t, C.c_size_t, C.c_int, u32p]; L.nqo_record_words.restype = None
        L.nqo_decode_proj.argtypes = [u8p, u8p, u32p, u64p, u8p] + [C.c_int] * 6 + [u16p]
        L.nqo_decode_proj.restype = C.c_int
        L.nqo_wht.argtypes = [f32p, C.c_int, C.c_int]; L.nqo_wht.restype = None
        L.nqo_expert_forward.argtypes = [u16p, u16p, u16p, C.c_int, C.c_int, C.c_int, u16p, u16p, C.c_int, C.c_int,
                                         C.c_int, f32p, C.c_int, f32p]
        L.nqo_expert_forward.restype = C.c_int
        L.nqo_threads.restype = C.c_int
        _LIB = L
    return _LIB


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def rbits(code):
    return lib().nqo_rbits(code)


def plane_bytes(nrec, code):
    return lib().nqo_plane_bytes(nrec, rbits(code))


def fold_consts(Mb, N):
    a, c = C.c_uint16(), C.c_uint16()
    lib().nqo_fold_consts(int(Mb), int(N), C.byref(a), C.byref(c))
    return a.value, c.value


def record_words(plane_u8, rec, nrec, bits):
    out = np.zeros((bits + 31) // 32, np.uint32)
    lib().nqo_record_words(_ptr(np.ascontiguousarray(plane_u8)), rec, nrec, bits, _ptr(out))
    return out


@dataclass
class ProjPlanes:
    """Packed planes of one projection as host byte arrays (the format the device table rows point at)."""
    N: int
    K: int
    base: np.ndarray                       # uint8, bytes of the base plane
    p4: Optional[np.ndarray] = None        # uint8, bytes of the residual plane (+ 4 B pad when it has a tail)
    d4: Optional[np.ndarray] = None        # uint32 block words Mb | N << 8
    flags: Optional[np.ndarray] = None     # uint64 per strip (mask mode) or None
    var: Optional[np.ndarray] = None       # uint8 per unit or None
    nm: int = 0                            # flagged chunks per strip in mask mode
    rk: int = 0                            # residual window code
    bk: int = 0                            # base window code


@dataclass
class ExpertPlanes:
    H: int
    I: int
    gu: ProjPlanes
    dn: ProjPlanes
    scales: np.ndarray                     # uint16 fp16 bits [H su_g | I sv_g | I sv_u | I su_d | H sv_o | H su_u]
    had_dn: int = 128
    lr: Optional[np.ndarray] = None        # uint16 fp16 bits
    lr4: Optional[np.ndarray] = None
    rg: int = 0
    rd: int = 0
    _cache: dict = field(default_factory=dict)


def _u8(a):
    return None if a is None else np.ascontiguousarray(a).view(np.uint8).reshape(-1)


def decode_proj(p: ProjPlanes, level: int) -> np.ndarray:
    """Dense decode of one projection -> uint16 fp16 bit patterns [N, K] (sm120/moe.py:156-166)."""
    W = np.empty((p.N, p.K), np.uint16)
    d4 = None if p.d4 is None else np.ascontiguousarray(p.d4, dtype=np.uint32)
    fl = None if p.flags is None else np.ascontiguousarray(p.flags).view(np.uint64)
    base, p4, var = _u8(p.base), _u8(p.p4), _u8(p.var)
    if level == 4 and (p4 is None or d4 is None):
        raise ValueError("level 4 needs the residual plane and block words")
    rc = lib().nqo_decode_proj(_ptr(base), _ptr(p4), _ptr(d4), _ptr(fl), _ptr(var), p.N, p.K, int(p.nm), int(p.rk),
                               int(p.bk), int(level), _ptr(W))
    if rc:
        raise ValueError(f"nqo_decode_proj failed with {rc}")
    return W


def expert_forward(ex: ExpertPlanes, level: int, x32: np.ndarray) -> np.ndarray:
    """x32: fp32 [T, H] holding fp16 values -> fp32 [T, H] (sm120/moe.py:196-210)."""
    key = level
    if key not in ex._cache:
        ex._cache[key] = (decode_proj(ex.gu, level), decode_proj(ex.dn, level))
    Wgu, Wdn = ex._cache[key]
    x32 = np.ascontiguousarray(x32, dtype=np.float32)
    y = np.empty_like(x32)
    rc = lib().nqo_expert_forward(_ptr(Wgu), _ptr(Wdn), _ptr(np.ascontiguousarray(ex.scales).view(np.uint16)), ex.H, ex.I,
                                  int(ex.had_dn), _ptr(None if ex.lr is None else np.ascontiguousarray(ex.lr).view(np.uint16)),
                                  _ptr(None if ex.lr4 is None else np.ascontiguousarray(ex.lr4).view(np.uint16)),
                                  int(ex.rg), int(ex.rd), int(level), _ptr(x32), x32.shape[0], _ptr(y))
    if rc:
        raise ValueError(f"nqo_expert_forward failed with {rc}")
    return y


def moe_ref(experts, levels, x16: np.ndarray, sel: np.ndarray, rw16: np.ndarray, keep_cache=True) -> np.ndarray:
    """Layer reference (sm120/moe.py:344-351): out[b] = sum_k rw[b,k] * expert(sel[b,k])(x[b]); picks with rw == 0 or
    level <= 0 add nothing.  x16 / rw16 are float16 arrays.  Tokens of one expert are run as one batch."""
    x32 = x16.astype(np.float32)
    T, H = x32.shape
    out = np.zeros((T, H), np.float32)
    rw = rw16.astype(np.float32)
    for e in np.unique(sel):
        lv = levels[int(e)]
        if lv <= 0:
            continue
        tk = [(b, k) for b in range(T) for k in range(sel.shape[1]) if sel[b, k] == e and rw[b, k] != 0]
        if not tk:
            continue
        toks = sorted({b for b, _ in tk})
        y = expert_forward(experts[int(e)], lv, x32[toks])
        if not keep_cache:
            experts[int(e)]._cache.clear()
        for b, k in tk:
            out[b] += rw[b, k] * y[toks.index(b)]
    return out


def salience_ref(x, rw16, sel, rsf, E):
    """salience added by one decode call (sm120/nqsal.cu:3-5): sal[e] = sum over picks (t, k) of e with weight != 0 of
    (rsf * w)^2 * sum_i x[t, i]^2; x [T, H] float, rw16 fp16 [T, topk], sel int [T, topk] -> float64 [E].
    The weight product follows the kernel's fp32 order; the norm is summed in float64 (the kernel sums fp32 partials)."""
    xn = (np.asarray(x, np.float64) ** 2).sum(1)
    out = np.zeros(E, np.float64)
    for t in range(sel.shape[0]):
        for k in range(sel.shape[1]):
            w = np.float32(rw16[t, k])
            if w != 0 and 0 <= sel[t, k] < E:
                w = np.float32(w * np.float32(rsf))
                out[int(sel[t, k])] += float(np.float32(w * w)) * xn[t]
    return out


# ------------------------------------------------------------------ numpy second opinion (one unit)
def _step_off(p, KA, MASK):
    per = np.array([sum(KA + ((MASK >> i) & 1) for i in range(r)) for r in range(16)])
    width = 16 * KA + bin(MASK).count("1")
    p = np.asarray(p)
    return (p >> 4) * width + per[p & 15]


def ring_sums_numpy(words, bits, code):
    """words: uint32 [32, nw] lane records of one unit -> byte-sums [8 rings, 256 positions]."""
    KA, MASK = PATTERNS[code]
    b = ((words[:, :, None].astype(np.uint64) >> np.arange(32, dtype=np.uint64)) & 1).reshape(32, -1)[:, :bits]
    ring = b.reshape(8, 4 * bits).astype(np.int64)
    off = _step_off(np.arange(256), KA, MASK)
    idx = (off[:, None] + np.arange(16)[None, :]) % (4 * bits)
    st = (ring[:, idx] << np.arange(16)).sum(-1)
    x = (st * HASH_MUL) & 0xFFFFFFFF
    return (x & 255) + ((x >> 8) & 255) + ((x >> 16) & 255) + ((x >> 24) & 255)


def decode_unit_numpy(base_words, res_words, rk, Mb, N, signs=None, bk=0):
    """One 16x128 unit.  base_words uint32 [32, nwb], res_words uint32 [32, nwr] or None (level 2).
    Returns fp16 array [16, 128].  signs: optional 8 booleans (ring negated)."""
    Sb = ring_sums_numpy(base_words, rbits(bk), bk)
    A = np.array([0x1eee], np.uint16).view(np.float16).astype(np.float64)[0]
    B = np.array([0xc931], np.uint16).view(np.float16).astype(np.float64)[0]
    if res_words is None:
        q = (A * (1024 + Sb) + B).astype(np.float16)
    else:
        Sr = ring_sums_numpy(res_words, rbits(rk), rk)
        rc = np.float32(1) / np.float32(Mb)
        Ah = np.float16(np.float32(1.732421875) * rc)
        t = np.float32(np.float32(N) * rc) * np.float32(-3.453125)
        t = np.float32(t + np.float32(-3.453125))
        Ch = np.float16(np.float32(t - np.float32(1024) * np.float32(Ah)))
        F = (Mb * Sb + N * Sr + 128) >> 8
        q = (np.float64(Ah) * (1024 + F) + np.float64(Ch)).astype(np.float16)
    if signs is not None:
        q = np.where(np.asarray(signs, bool)[:, None], -q, q)
    out = np.zeros((16, 128), np.float16)
    p = np.arange(256)
    t4, j = p >> 6, p & 63
    pp, e = j >> 1, j & 1
    t, r = pp >> 2, pp & 3
    k = 16 * t + 2 * t4 + 8 * (r >> 1) + e
    for g in range(8):
        out[g + 8 * (r & 1), k] = q[g]
    return out
