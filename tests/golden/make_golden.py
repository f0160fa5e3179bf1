"""Generates the golden fixtures in this folder by IMPORTING the reference's own CPU implementation.

Run once in a container that has the reference checkout (it is not needed to run the tests):

    python tests/golden/make_golden.py /path/to/nestquant

What is imported, unmodified: sm120/moe.py (Proj, Expert, pack_words, fold_vals, dense_W, moe_ref) and
sm120/ref15_spec.py (consts).  Two shims are needed to import moe.py without a GPU: a stub `build` module
(moe.py JIT-compiles its CUDA extension at import) and `Proj.bw = None` (Proj.to reads an attribute that is only
set for non-default base codes).  Nothing from the reference is copied into the fixtures except the numbers it
computes: packed planes drawn by its generators and the decoded weights / layer outputs it derives from them.

Fixtures written (all numpy .npz, little-endian):
  pack.npz      pack_words() of random record words, every window code 0..9            (plane layout)
  consts.npz    fold_vals() samples for every valid block word (+ ref15_spec.consts())   (level-4 arithmetic)
  decode.npz    small projections: planes + dense_W() at level 2 and 4, all codes, signs, mask mode, base code 1
  layer.npz     5-expert layer, mixed levels 0/2/4/4-masked: planes, scales, x, sel, rw and moe_ref() output
  layer_lr.npz  2-expert layer with the low-rank plane and the 512-wide down-input rotation
"""
import os
import sys
import types

import numpy as np
import torch

if len(sys.argv) < 2:
    raise SystemExit(__doc__)
REF = sys.argv[1]
OUT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(REF, "sm120"))
sys.modules["build"] = types.SimpleNamespace(get=lambda *a, **k: None, get_sal=lambda *a, **k: None)
import moe  # noqa: E402
import ref15_spec as spec  # noqa: E402

moe.Proj.bw = None
torch.set_num_threads(8)


def u16(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def proj_arrays(p, prefix, d):
    d[prefix + "base"] = p.base.numpy().copy()
    d[prefix + "p4"] = p.p4.numpy().copy()
    d[prefix + "d4"] = p.d4.numpy().copy()
    d[prefix + "flags"] = np.zeros(0, np.int64) if p.flags is None else p.flags.numpy().copy()
    d[prefix + "var"] = np.zeros(0, np.uint8) if p.var is None else p.var.numpy().copy()
    d[prefix + "meta"] = np.array([p.N, p.K, -1 if p.z["nm"] is None else p.z["nm"], p.rk, p.bk], np.int64)


# ---------------------------------------------------------------- pack.npz
d = {}
g = torch.Generator().manual_seed(11)
for c in sorted(moe.RKP):
    b = moe.rbits(c); nw = (b + 31) // 32
    for nrec in (32, 160):
        w = torch.randint(0, 2**32, (nrec, nw), generator=g, dtype=torch.int64)
        if b % 32:
            w[:, -1] &= (1 << (b % 32)) - 1
        d[f"c{c}.n{nrec}.words"] = w.numpy().astype(np.uint32)
        d[f"c{c}.n{nrec}.packed"] = moe.pack_words(w, b).numpy().view(np.uint8).copy()
np.savez_compressed(os.path.join(OUT, "pack.npz"), **d)

# ---------------------------------------------------------------- consts.npz
# Note: ref15_spec.consts() does its last subtraction in float64 while moe.fold_vals() and the CUDA kernel
# (nqmoe.cu:267) stay in fp32; they differ by one fp16 ulp of C for 11 of the 33,149 block words.  The kernel
# contract is the fp32 form, so the fixture stores fold_vals() outputs, and the 11 words for the record.
L = moe.all_MbN().numpy()
Ah_s, Ch_s = spec.consts(L[:, 0], L[:, 1])
g = torch.Generator().manual_seed(12)
Sb = torch.randint(0, 1021, (len(L), 4), generator=g)
Sr = torch.randint(0, 1021, (len(L), 4), generator=g)
Sb[:64, 0] = 0; Sr[:64, 0] = 0; Sb[64:128, 0] = 1020; Sr[64:128, 0] = 1020
Lt = torch.from_numpy(L)
q_pos = moe.fold_vals(Sb, Sr, Lt[:, :1], Lt[:, 1:], 1.0)
q_neg = moe.fold_vals(Sb, Sr, Lt[:, :1], Lt[:, 1:], -1.0)
Sq = torch.arange(0, 1021)
q2 = ((1.0 * moe.A_) * (1024 + Sq.double()) + 1.0 * moe.B_).half()
np.savez_compressed(os.path.join(OUT, "consts.npz"), MbN=L.astype(np.int32),
                    Ah_spec=Ah_s.astype(np.float16).view(np.uint16), Ch_spec=Ch_s.astype(np.float16).view(np.uint16),
                    Sb=Sb.numpy().astype(np.int16), Sr=Sr.numpy().astype(np.int16), q4=u16(q_pos), q4_neg=u16(q_neg), q2=u16(q2))

# ---------------------------------------------------------------- decode.npz
d = {}; cases = []
N_, K_ = 32, 384                                          # 2 strips x 3 chunks = 6 units
for i, (rk, bk, var, nm, mbn) in enumerate([
        (0, 0, False, None, "rand"), (0, 0, True, None, ("exh", 0)), (1, 0, True, None, ("exh", 500)),
        (2, 0, False, None, ("exh", 1000)), (3, 0, True, None, ("exh", 5000)), (4, 0, False, None, ("exh", 9000)),
        (5, 0, True, None, ("exh", 13000)), (6, 0, True, None, ("exh", 17000)), (7, 0, True, None, ("exh", 21000)),
        (8, 0, False, None, ("exh", 25000)), (9, 0, True, None, ("exh", 29000)), (0, 0, True, 2, "rand"),
        (7, 0, True, 1, ("exh", 33000)), (6, 0, False, 2, "rand"), (3, 1, True, None, "rand"), (9, 1, True, 1, "rand")]):
    gen = torch.Generator().manual_seed(1000 + i)
    p = moe.Proj(N_, K_, gen, nm, rk, mbn, var, bk)
    name = f"case{i}."
    proj_arrays(p, name, d)
    d[name + "W2"] = u16(moe.dense_W(p, 2, 4, torch.float16))
    d[name + "W4"] = u16(moe.dense_W(p, 4, 4, torch.float16))
    cases.append(i)
d["ncases"] = np.array([len(cases)])
np.savez_compressed(os.path.join(OUT, "decode.npz"), **d)


# ---------------------------------------------------------------- layer.npz / layer_lr.npz
def expert_arrays(ex, prefix, d):
    proj_arrays(ex.gu, prefix + "gu.", d); proj_arrays(ex.dn, prefix + "dn.", d)
    d[prefix + "scales"] = u16(ex.signs)
    d[prefix + "had_dn"] = np.array([moe.had_dn(ex)])
    if ex.lr is not None:
        d[prefix + "lr"] = u16(ex.lr); d[prefix + "lr4"] = u16(ex.lr4); d[prefix + "r"] = np.array([ex.rg, ex.rd])


def scales_for(ex, gen):
    """[su_g | sv_g | sv_u | su_d | sv_o | su_u]: +-1 input signs, |N(0, 0.02)| output scales"""
    H, I = ex.H, ex.I
    s = ex.signs.clone().float()
    for a, b in ((H, H + 2 * I), (H + 3 * I, 2 * H + 3 * I)):
        s[a:b] = (torch.randn(b - a, generator=gen) * 0.02).abs()
    ex.signs = s.half()


H, I, E, topk, B = 256, 256, 5, 2, 6
levels = [2, 4, 4, 0, 4]
gen = torch.Generator().manual_seed(77)
exs = []
for e in range(E):
    masked = e == 2
    ex = moe.Expert(H, I, seed=300 + e, nm_gu=1 if masked else None, nm_dn=1 if masked else None, dev="cpu",
                    rk_gu=(0, 6, 0, 0, 3)[e], rk_dn=(7, 7, 8, 0, 7)[e], var=e != 4)
    scales_for(ex, gen); exs.append(ex)
x = torch.randn(B, H, generator=gen).bfloat16().half()
logits = torch.randn(B, E, generator=gen)
tv, sel = logits.topk(topk, dim=1)
rw = torch.softmax(tv, 1).half()
rw[5, 1] = 0                                              # a pick with zero weight is skipped
sel[4] = torch.tensor([3, 3])                             # a token whose picks are all at level 0
out = moe.moe_ref(exs, levels, x, sel, rw)
d = {"shape": np.array([H, I, E, topk, B]), "levels": np.array(levels), "x": u16(x), "sel": sel.numpy(), "rw": u16(rw),
     "out": out.numpy()}
for e in range(E):
    if levels[e] > 0:
        expert_arrays(exs[e], f"e{e}.", d)
np.savez_compressed(os.path.join(OUT, "layer.npz"), **d)

H, I, E, topk, B = 256, 512, 2, 2, 3
levels = [4, 2]
gen = torch.Generator().manual_seed(78)
exs = []
for e in range(E):
    ex = moe.Expert(H, I, seed=400 + e, dev="cpu", rk_gu=0, rk_dn=7, var=True)
    scales_for(ex, gen)
    rg, rd = (2, 1) if e == 0 else (1, 3)
    r = lambda *s: torch.randn(*s, generator=gen) * 0.02
    ex.set_lr(r(rg, H), r(rg, I), r(rg, I), r(rg, I), r(rg, I), r(rd, I), r(rd, H), r(rd, H))
    ex.lrT = tuple(t.half().float() for t in ex.lrT)       # the reference reads the fp32 originals; round them like the plane
    if e == 0:
        ex.had_dn = 512
    exs.append(ex)
x = torch.randn(B, H, generator=gen).bfloat16().half()
sel = torch.tensor([[0, 1], [1, 0], [0, 1]])
rw = torch.softmax(torch.randn(B, topk, generator=gen), 1).half()
out = moe.moe_ref(exs, levels, x, sel, rw)
d = {"shape": np.array([H, I, E, topk, B]), "levels": np.array(levels), "x": u16(x), "sel": sel.numpy(), "rw": u16(rw),
     "out": out.numpy()}
for e in range(E):
    expert_arrays(exs[e], f"e{e}.", d)
np.savez_compressed(os.path.join(OUT, "layer_lr.npz"), **d)
for f in sorted(os.listdir(OUT)):
    if f.endswith(".npz"):
        print(f, os.path.getsize(os.path.join(OUT, f)))
