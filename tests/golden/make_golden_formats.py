"""Generates the serving-file fixtures by IMPORTING the reference's own writers (streaming/resident.py, streaming/p4rec.py).

    python tests/golden/make_golden_formats.py /path/to/nestquant

Fixtures:
  resident_L5.pt   an nq-res-v1 file written by the reference's resident.save for a 3-expert layer (one with a low-rank
                   plane), 512-wide down-input rotation
  records.npz      the same experts' records packed by the reference's p4rec.pack, its layout, and the level-4 rows
                   p4rec.row derives for a made-up slot address
The experts come from the reference's sm120/moe.py generators (same shims as make_golden.py).
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
sys.path[:0] = [os.path.join(REF, "sm120"), os.path.join(REF, "streaming")]
sys.modules["build"] = types.SimpleNamespace(get=lambda *a, **k: None, get_sal=lambda *a, **k: None)
import moe  # noqa: E402
import p4rec  # noqa: E402
import resident  # noqa: E402

moe.Proj.bw = None
H, I = 256, 512
gen = torch.Generator().manual_seed(91)
ex = {}
for e in (2, 5, 7):
    x = moe.Expert(H, I, seed=500 + e, dev="cpu", rk_gu=0, rk_dn=7, var=True)
    x.sc = {2: x.signs, 4: (torch.randn(3 * H + 3 * I, generator=gen) * 0.02).abs().half()}
    if e == 5:
        r = lambda *s: torch.randn(*s, generator=gen) * 0.02
        x.set_lr(r(2, H), r(2, I), r(2, I), r(2, I), r(2, I), r(1, I), r(1, H), r(1, H))
    x.had_dn = 512                                       # as nqload.RankLayer sets it on every expert of the layer
    ex[e] = x
RL = types.SimpleNamespace(L=5, rank=1, tp=4, H=H, I=I, experts=list(ex), ex=ex, had_dn=512)
resident.save(RL, os.path.join(OUT, "resident_L5.pt"))
lay = p4rec.layout(ex[2], H, I)
d = {"rec_bytes": np.array([lay["rec_bytes"]]), "seg": np.array([list(lay["seg"][k]) for k in p4rec.SEGS])}
SLOT = 0x7F0000001000
for e, x in ex.items():
    d[f"rec{e}"] = np.frombuffer(p4rec.pack(x, lay), dtype=np.uint8).copy()
    row = p4rec.row(x, lay, SLOT, moe.entry)
    ptrs = {"gu.base": x.gu.base.data_ptr(), "dn.base": x.dn.base.data_ptr(), "sc4": x.sc[4].data_ptr(), "gu.var": x.gu.var.data_ptr(),
            "dn.var": x.dn.var.data_ptr(), "lr": 0 if x.lr is None else x.lr.data_ptr()}
    # rows hold process addresses: store them relative to what they point at
    rel = [int(v) for v in row]
    d[f"row{e}.slot_rel"] = np.array([rel[2] - SLOT, rel[3] - SLOT, rel[6] - SLOT, rel[7] - SLOT, (rel[15] - SLOT) if x.rg + x.rd else -1])
    d[f"row{e}.same"] = np.array([rel[1] == ptrs["gu.base"], rel[5] == ptrs["dn.base"], rel[9] == ptrs["sc4"], rel[12] == ptrs["gu.var"],
                                  rel[13] == ptrs["dn.var"], rel[14] == ptrs["lr"]])
    d[f"row{e}.plain"] = np.array([rel[0], rel[4], rel[8], rel[10], rel[11], rel[16], rel[17], rel[18], rel[19]])
np.savez_compressed(os.path.join(OUT, "records.npz"), **d)
for f in ("resident_L5.pt", "records.npz"):
    print(f, os.path.getsize(os.path.join(OUT, f)))
