"""Serving file formats against fixtures written by the reference's own tools (tests/golden/make_golden_formats.py):
the resident-plane file of a rank and layer (nq-res-v1) and the record layout / level-4 row of the slot pool."""
import json
import os
import types

import numpy as np
import torch

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
SLOT = 0x7F0000001000


def _reference_dict():
    return torch.load(os.path.join(GOLD, "resident_L5.pt"), map_location="cpu", weights_only=True)


def test_resident_file_loads_and_rewrites_identically(tmp_path):
    from nestquant_b200 import resident
    ref = _reference_dict()
    assert ref["format"] == "nq-res-v1" and ref["experts"] == [2, 5, 7] and ref["in_had_down"] == 512
    ex, H, I = resident.load(os.path.join(GOLD, "resident_L5.pt"), dev="cpu")
    assert (H, I) == (256, 512) and sorted(ex) == [2, 5, 7]
    for i, e in enumerate(ref["experts"]):
        x = ex[e]
        assert torch.equal(x.gu.base, ref["gu_base"][i]) and torch.equal(x.dn.var, ref["dn_var"][i])
        assert torch.equal(x.sc[2], ref["sc2"][i]) and torch.equal(x.sc[4], ref["sc4"][i]) and x.signs is x.sc[2]
        assert (x.gu.rk, x.dn.rk, x.gu.bk, x.dn.bk, x.had_dn) == (0, 7, 0, 0, 512)
        assert x.gu.p4 is None and x.dn.d4 is None
    assert ex[2].lr is None and (ex[5].rg, ex[5].rd) == (2, 1)
    assert ex[5].lr.numel() == resident.lr_len(H, I, 2, 1) and torch.equal(ex[5].lr, ref["lr"][1, :ex[5].lr.numel()])
    # writing the loaded layer back gives the reference's file content again
    layer = types.SimpleNamespace(L=ref["L"], rank=ref["rank"], tp=ref["tp"], H=H, I=I, experts=ref["experts"], ex=ex, had_dn=512)
    out = str(tmp_path / "L5.pt")
    resident.save(layer, out)
    mine = torch.load(out, map_location="cpu", weights_only=True)
    assert sorted(mine) == sorted(ref)
    for k, v in ref.items():
        assert torch.equal(mine[k], v) if torch.is_tensor(v) else mine[k] == v, k


def test_record_layout_and_rows_match_the_reference(tmp_path):
    from nestquant_b200 import moe, p4rec, resident
    z = np.load(os.path.join(GOLD, "records.npz"))
    ex, H, I = resident.load(os.path.join(GOLD, "resident_L5.pt"), dev="cpu")
    seg = {k: tuple(int(v) for v in z["seg"][i]) for i, k in enumerate(p4rec.SEGS)}
    full = {}
    for e, x in ex.items():                         # residual planes back from the reference's record
        rec = torch.from_numpy(z[f"rec{e}"].copy())
        for p, name in ((x.gu, "gu"), (x.dn, "dn")):
            for part in ("p4", "d4"):
                o, n = seg[f"{name}.{part}"]
                setattr(p, part, rec[o:o + n].view(torch.int32).clone())
        if x.rg + x.rd:
            n4 = (x.rg * 2 * I + x.rd * H) * 2
            x.lr4 = rec[seg["lr4"][0]:seg["lr4"][0] + n4].view(torch.float16).clone()
        full[e] = x
    lay = p4rec.layout(full[2], H, I)
    assert lay["rec_bytes"] == int(z["rec_bytes"][0]) and {k: tuple(v) for k, v in lay["seg"].items()} == seg
    for e, x in full.items():
        assert np.array_equal(p4rec.pack(x, lay, pin=False).numpy(), z[f"rec{e}"]), e
        row = [int(v) for v in p4rec.row(x, lay, SLOT, moe.entry)]
        rel = [row[2] - SLOT, row[3] - SLOT, row[6] - SLOT, row[7] - SLOT, (row[15] - SLOT) if x.rg + x.rd else -1]
        assert rel == z[f"row{e}.slot_rel"].tolist()
        same = [row[1] == x.gu.base.data_ptr(), row[5] == x.dn.base.data_ptr(), row[9] == x.sc[4].data_ptr(), row[12] == x.gu.var.data_ptr(),
                row[13] == x.dn.var.data_ptr(), row[14] == (0 if x.lr is None else x.lr.data_ptr())]
        assert same == z[f"row{e}.same"].astype(bool).tolist()
        assert [row[i] for i in (0, 4, 8, 10, 11, 16, 17, 18, 19)] == z[f"row{e}.plain"].tolist()
    # record file of a rank: record of (L, E) at ((L - L0) * NE + E) * rec_bytes, index beside it
    idx = resident.rank_index(tp=4, rank=1, L0=3, NE=8)
    resident.write_rank_file(str(tmp_path), idx, 5, full, H, I)
    raw = np.fromfile(tmp_path / "rank1.bin", dtype=np.uint8)
    for e in full:
        o = resident.record_offset(idx, 5, e)
        assert o == ((5 - 3) * 8 + e) * lay["rec_bytes"] and np.array_equal(raw[o:o + lay["rec_bytes"]], z[f"rec{e}"])
    j = json.load(open(tmp_path / "rank1.json"))
    assert j["format"] == "nq-p4rec-v1" and j["rec_bytes"] == lay["rec_bytes"] and j["layers"]["5"]["experts"] == [2, 5, 7]
    assert j["layers"]["5"]["rg"] == {"2": 0, "5": 2, "7": 0}
