"""Resident planes of one rank and layer in the serving file format, and the index of the rank's record file.

`save` / `load` read and write the reference's `nq-res-v1` / `nq-res-v2` files (streaming/resident.py:17-50): a
torch-saved dict holding, stacked over the layer's experts, the 2-bit base and ring-sign planes, the level-2 and level-4
scale vectors, the low-rank base part (V, U2; padded to rank 4), the residual window codes and, when it is not 128, the
width of the down-input rotation.  Files written here load in the reference and the other way round; v2 (a base window
code other than 0) is read and written too, although the kernels of this library only run base code 0.

`rank_index` / `record_offset` / `write_rank_file` are the record-file side (streaming/repack.py:1-6,31-44): the record
of expert E of layer L sits at ((L - L0) * NE + E) * rec_bytes of rank{r}.bin, rank{r}.json holds the layout.
"""
import json
import os
import types

import torch

from . import p4rec

RMAX = 4
FORMATS = ("nq-res-v1", "nq-res-v2")


def lr_len(H, I, rg, rd):
    return rg * (H + 2 * I) + rd * (I + H)


def save(layer, path):
    """layer: .L, .rank, .tp, .H, .I, .experts (ids), .ex {id: expert}, optional .had_dn.  An expert needs gu / dn with
    base, var, rk (bk optional), sc {2: scales, 4: scales}, lr (or None), rg, rd.
    The dictionary keys, tensor shapes and the write-then-rename step are the file format of the reference's writer
    (streaming/resident.py:17-33): files written here load there and the other way round (tests/test_formats_cpu.py)."""
    E = list(layer.experts)
    ex = [layer.ex[e] for e in E]
    H, I = layer.H, layer.I
    stack = lambda f: torch.stack([f(x).cpu() for x in ex])
    lr = torch.zeros(len(E), lr_len(H, I, RMAX, RMAX), dtype=torch.float16)
    for i, x in enumerate(ex):
        if x.lr is not None:
            lr[i, :x.lr.numel()] = x.lr.cpu()
    d = dict(format="nq-res-v1", L=layer.L, rank=layer.rank, tp=layer.tp, H=H, I=I, experts=E,
             rk_gu=[x.gu.rk for x in ex], rk_dn=[x.dn.rk for x in ex], rg=[x.rg for x in ex], rd=[x.rd for x in ex],
             gu_base=stack(lambda x: x.gu.base), gu_var=stack(lambda x: x.gu.var), dn_base=stack(lambda x: x.dn.base),
             dn_var=stack(lambda x: x.dn.var), sc2=stack(lambda x: x.sc[2]), sc4=stack(lambda x: x.sc[4]), lr=lr)
    bk_gu = [int(getattr(x.gu, "bk", 0) or 0) for x in ex]
    bk_dn = [int(getattr(x.dn, "bk", 0) or 0) for x in ex]
    if any(bk_gu) or any(bk_dn):
        d.update(format="nq-res-v2", bk_gu=bk_gu, bk_dn=bk_dn)
    w = int(getattr(layer, "had_dn", 128))
    if w != 128:
        d["in_had_down"] = w
    torch.save(d, path + ".tmp")
    os.replace(path + ".tmp", path)


def load(path, dev="cuda"):
    """-> ({expert id: expert}, H, I).  The experts carry what moe.entry and p4rec.row read at level 2; their residual
    planes (p4, d4) are None until a record is promoted into a slot, lr4 is a placeholder (U4 is read from the slot)."""
    d = torch.load(path, map_location="cpu", weights_only=True)
    if d.get("format") not in FORMATS:
        raise ValueError(f"{path}: format {d.get('format')!r} is not one of {FORMATS}")
    H, I = d["H"], d["I"]
    g = {k: d[k].to(dev) for k in ("gu_base", "gu_var", "dn_base", "dn_var", "sc2", "sc4", "lr")}
    dummy = torch.zeros(1, dtype=torch.float16, device=dev)
    hw = had_width(path, d)
    n = len(d["experts"])
    bkg, bkd = d.get("bk_gu", [0] * n), d.get("bk_dn", [0] * n)
    out = {}
    for i, e in enumerate(d["experts"]):
        proj = lambda k, rk, bk: types.SimpleNamespace(base=g[k + "_base"][i], var=g[k + "_var"][i], p4=None, d4=None, flags=None,
                                                       fl=None, rk=rk, bk=bk)
        rg, rd = d["rg"][i], d["rd"][i]
        has = rg + rd > 0
        x = types.SimpleNamespace(gu=proj("gu", d["rk_gu"][i], bkg[i]), dn=proj("dn", d["rk_dn"][i], bkd[i]), H=H, I=I, rg=rg, rd=rd,
                                  sc={2: g["sc2"][i], 4: g["sc4"][i]}, lr=g["lr"][i, :lr_len(H, I, rg, rd)] if has else None,
                                  lr4=dummy if has else None)
        x.signs = x.sc[2]
        x.had_dn = hw
        out[e] = x
    return out, H, I


def had_width(path, d):
    """width of the down-input rotation of a resident file: its own key, else the layer entry of the rank index three
    directories up (<repack>/rank{r}.json), else 128"""
    if "in_had_down" in d:
        return int(d["in_had_down"])
    ip = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(path)))), f"rank{d['rank']}.json")
    if not os.path.exists(ip):
        return 128
    return int(json.load(open(ip))["layers"].get(str(d["L"]), {}).get("in_had_down", 128))


# ---------------------------------------------------------------- record file of a rank
def rank_index(tp, rank, L0=3, NE=256):
    return dict(format="nq-p4rec-v1", tp=tp, rank=rank, L0=L0, NE=NE, layers={})


def record_offset(idx, L, E):
    """byte offset of the record of expert E of layer L in rank{r}.bin"""
    return ((L - idx["L0"]) * idx["NE"] + E) * idx["rec_bytes"]


def write_rank_file(out_dir, idx, L, experts, H, I):
    """Write the records of one layer (experts: {id: expert with residual planes}) into out_dir/rank{r}.bin and enter the
    layer in out_dir/rank{r}.json.  Returns the record layout.  Every layer of a file must have the same layout."""
    os.makedirs(out_dir, exist_ok=True)
    lay = p4rec.layout(next(iter(experts.values())), H, I)
    seg = json.loads(json.dumps(lay["seg"]))
    if "rec_bytes" not in idx:
        idx["rec_bytes"], idx["seg"] = lay["rec_bytes"], seg
    if seg != idx["seg"] or lay["rec_bytes"] > idx["rec_bytes"]:
        raise ValueError(f"layer {L}: record layout differs from the file's")
    lay["rec_bytes"] = idx["rec_bytes"]
    fd = os.open(os.path.join(out_dir, f"rank{idx['rank']}.bin"), os.O_WRONLY | os.O_CREAT, 0o644)
    try:
        for e, ex in experts.items():
            os.pwrite(fd, p4rec.pack(ex, lay, pin=False).numpy().tobytes(), record_offset(idx, L, e))
        os.fsync(fd)
    finally:
        os.close(fd)
    idx["layers"][str(L)] = dict(experts=list(experts), rg={e: x.rg for e, x in experts.items()}, rd={e: x.rd for e, x in experts.items()})
    ip = os.path.join(out_dir, f"rank{idx['rank']}.json")
    json.dump(idx, open(ip + ".tmp", "w"))
    os.replace(ip + ".tmp", ip)
    return lay
