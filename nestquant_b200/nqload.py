"""Loader for the production shard format (nestquant-v1): one directory per layer holding manifest.json and eight
tensor-parallel shard files tp{s}.pt (or tp{s}.safetensors), each {expert: {gate | up | down: planes}}.

Mirrors the reference's sm120/nqload.py (same names, arguments and results), which the serving scripts call:
  group_art(parts, man, E, ss)        the artifact of expert E restricted to the shard group ss        nqload.py:19-38
  repack(P, dev, want_Q)              one projection: encoder planes -> kernel planes                   nqload.py:40-65
  cat_proj(a, b, dev)                 gate and up as one 2I-row projection                              nqload.py:67-75
  kernel_expert(art, dev, want_Q)     -> (expert, scales(level), (Qgate, Qup, Qdown))                   nqload.py:77-93
  had_width, p4_bytes, layer_dir, load_part, RankLayer                                                  nqload.py:95-136
Rank r of a TP = tp run owns the shards r * 8 / tp .. (r + 1) * 8 / tp - 1; the format stores units shard-major, so a group
of shards is a self-contained expert with I = 256 * 8 / tp.

What the loader does is move bits: the encoder writes, per unit, the eight ring streams back to back (LSB first, units in
shard order then strip-major); the kernels read one record per lane (a quarter of a ring stream) with the records in
(strip, chunk, lane) order, the residual plane in the sub-array layout (moe.pack_words).  Everything here is host-side
numpy; the result tensors are moved to `dev` at the end.  The dense matrices asked for by want_Q come from this library's
own dense decode kernel (ext.pf_decode) and therefore need the GPU; the reference takes them from the encoder-side decoder.
"""
import json
import os
import struct
import types

import numpy as np
import torch

from . import ext as _ext
from .moe import RK_OF, TBL_W, entry, pack_words, proj_sizes, rbits

PROJ = ("gate", "up", "down")
NSH = 8
ST_FORMAT = "nestquant-v1-tp-safetensors"
_ST_DTYPES = {"U8": torch.uint8, "I8": torch.int8, "I16": torch.int16, "I32": torch.int32, "I64": torch.int64, "F16": torch.float16,
              "BF16": torch.bfloat16, "F32": torch.float32, "F64": torch.float64, "BOOL": torch.bool}


def _cat(ts, dim=0):
    return torch.cat(list(ts), dim)


def group_art(parts, man, E, ss):
    """parts[s] = the loaded shard file s; ss = contiguous shard ids.  Returns {proj: {base, p4, meta}} with the group's
    dimensions in meta: down is sharded along its inputs (k), gate and up along their outputs (n); the scale vector of the
    sharded side is the concatenation over the group, the other side is replicated in every shard."""
    g = len(ss)
    art = {}
    for pn in PROJ:
        meta = dict(man["proj_meta"][pn])
        ps = [parts[s][E][pn] for s in ss]
        along_k = pn == "down"
        if along_k:
            meta.update(k=meta["k"] * g // NSH, tk=meta["tk"] * g // NSH)
        else:
            meta.update(n=meta["n"] * g // NSH, tn=meta["tn"] * g // NSH)
        vec = {}
        for key in ("suh2", "svh2", "suh4", "svh4"):
            sharded = key.startswith("suh") == along_k
            vec[key] = _cat(p[key] for p in ps) if sharded else ps[0][key]
        art[pn] = dict(base=dict(shards=[p["base"] for p in ps], var=[p["var"] for p in ps], suh=vec["suh2"], svh=vec["svh2"]),
                       p4=dict(shards=[p["p4"] for p in ps], word=[p["word"] for p in ps], suh=vec["suh4"], svh=vec["svh4"]), meta=meta)
        if "lrU2" in ps[0]:
            if along_k:        # V is cut along the inputs, U is whole in every shard
                V, U2, U4 = _cat((p["lrV"] for p in ps), 1), ps[0]["lrU2"], ps[0]["lrU4"]
            else:              # V is whole (up may point at gate's), U is cut along the outputs
                V = parts[ss[0]][E][ps[0].get("lrV_from", pn)]["lrV"]
                U2, U4 = _cat((p["lrU2"] for p in ps), 1), _cat((p["lrU4"] for p in ps), 1)
            art[pn]["base"]["lr"] = dict(V=V, U2=U2)
            art[pn]["p4"]["lr"] = dict(U4=U4)
    return art


def _storage_to_record_order(tk, tn, shard_axis):
    """position in the file of the unit that becomes record-unit i (i = strip * tk + chunk).  The file holds the units
    shard by shard (a shard = 16 strips of an n-sharded projection, 2 chunks of a k-sharded one), strip-major inside."""
    strip, chunk = np.divmod(np.arange(tk * tn), tk)
    shard = strip // 16 if shard_axis == "n" else chunk // 2
    file_rank = np.argsort((shard * tn + strip) * tk + chunk, kind="stable")     # file_rank[j] = record-unit stored j-th
    pos = np.empty(tk * tn, dtype=np.int64)
    pos[file_rank] = np.arange(tk * tn)
    return pos


def _lane_words(raw, units, bits, pos):
    """raw: the units' ring streams as stored (uint8; per unit 8 rings x 4 lanes x `bits` bits, LSB first).  Returns
    int64 [units * 32, words] of uint32 values: record (unit, ring g, lane t4) = bits [t4 * bits, (t4 + 1) * bits) of ring g."""
    per_unit = 4 * bits                                    # bytes: 32 lanes x bits / 8
    by = np.ascontiguousarray(raw.numpy().reshape(units, per_unit)[pos])
    b = np.unpackbits(by, axis=1, bitorder="little").reshape(units * 32, bits)
    nw = (bits + 31) // 32
    if nw * 32 != bits:
        b = np.concatenate([b, np.zeros((units * 32, nw * 32 - bits), dtype=np.uint8)], axis=1)
    words = np.packbits(b, axis=1, bitorder="little").view("<u4")
    return torch.from_numpy(words.astype(np.int64))


def repack(P, dev="cuda", want_Q=False):
    """Encoder planes of one projection -> an object with the fields the table row is built from (N, K, rk, bk, z, base,
    p4, d4, var, Mb, Nn, flags) plus the record words (p4w, and bw for a pattern-rate base) that cat_proj needs.
    The second result is always None here: dense matrices are made per expert in kernel_expert."""
    m = P["meta"]
    tk, tn = m["tk"], m["tn"]
    units = tk * tn
    rule = m["res_rule"]
    if rule["kind"] != "uniform":
        raise ValueError(f"res_rule {rule}: the kernels take one residual code per projection")
    rk, bk = RK_OF[float(rule["K"])], RK_OF[float(m.get("base_K", 2))]
    if m.get("base_var") != "sign":
        raise ValueError(f"base_var {m.get('base_var')!r}: only the 1-bit ring sign is a kernel plane")
    pos = _storage_to_record_order(tk, tn, m["shard_axis"])
    wb = _lane_words(_cat(t.cpu() for t in P["base"]["shards"]), units, rbits(bk), pos)
    wr = _lane_words(_cat(t.cpu() for t in P["p4"]["shards"]), units, rbits(rk), pos)
    p = types.SimpleNamespace(N=m["n"], K=m["k"], rk=rk, bk=bk, z=proj_sizes(m["n"], m["k"], None, rk, bk), flags=None, fl=None)
    if bk == 0:
        p.base = torch.from_numpy(wb.numpy().astype(np.uint32).view(np.int32).reshape(-1)).to(dev)
    else:
        p.bw = wb
        p.base = pack_words(wb, rbits(bk)).to(dev)
    p.p4w = wr
    p.p4 = pack_words(wr, rbits(rk)).to(dev)
    word = _cat(t.cpu() for t in P["p4"]["word"]).long()[torch.from_numpy(pos)]
    p.Mb, p.Nn = (word & 255).to(dev), ((word >> 8) & 255).to(dev)
    p.d4 = (p.Mb | (p.Nn << 8)).to(torch.int32)
    ring_sign = _cat(t.cpu() for t in P["base"]["var"]).long().view(units, 8)[torch.from_numpy(pos)] & 1
    p.var = (ring_sign << torch.arange(8)).sum(1).to(torch.uint8).to(dev)
    return p, None


def cat_proj(a, b, dev="cuda"):
    """gate (a) on top of up (b): one projection of 2I rows.  The sub-arrays of a plane span all its records, so the
    residual plane (and a pattern-rate base plane) is packed again from the joined record words."""
    if a.rk != b.rk:
        raise AssertionError("gate and up must share the residual code (one code per kernel launch)")
    if a.bk != b.bk:
        raise AssertionError("gate and up must share the base code")
    p = types.SimpleNamespace(N=a.N + b.N, K=a.K, rk=a.rk, bk=a.bk, z=proj_sizes(a.N + b.N, a.K, None, a.rk, a.bk), flags=None, fl=None)
    if a.bk == 0:
        p.base = torch.cat([a.base, b.base])
    else:
        p.bw = torch.cat([a.bw, b.bw])
        p.base = pack_words(p.bw, rbits(a.bk)).to(dev)
    p.p4w = torch.cat([a.p4w, b.p4w])
    p.p4 = pack_words(p.p4w, rbits(a.rk)).to(dev)
    for k in ("Mb", "Nn", "d4", "var"):
        setattr(p, k, torch.cat([getattr(a, k), getattr(b, k)]))
    return p


def _dense(ex, scales):
    """{level: (Wgu [2I, H], Wdn [H, I])} fp16, rotated basis, decoded by the library's dense decode kernel."""
    if ex.gu.base.device.type != "cuda":
        raise RuntimeError("want_Q needs the expert on a CUDA device: the dense matrices come from the decode kernel")
    out = {}
    dev = ex.gu.base.device
    for lv in (2, 4):
        ex.signs = scales(lv)
        table = torch.zeros(1, TBL_W, dtype=torch.int64)
        table[0] = entry(ex, lv)
        table = table.to(dev)
        Wgu = torch.empty(1, 2 * ex.I, ex.H, dtype=torch.float16, device=dev)
        Wdn = torch.empty(1, ex.H, ex.I, dtype=torch.float16, device=dev)
        _ext.pf_decode(table, torch.zeros(1, dtype=torch.int32, device=dev), Wgu, Wdn, ex.H, ex.I, 0, 0)
        torch.cuda.synchronize(dev)
        out[lv] = (Wgu[0], Wdn[0])
    del ex.signs
    return out


def kernel_expert(art, dev="cuda", want_Q=False):
    """-> (ex, scales, (Qgate, Qup, Qdown)): ex has gu / dn (kernel planes), H, I, the low-rank plane (lr, lr4, rg, rd) and
    sc = {2: ..., 4: ...}, the scale vector [su_g | sv_g | sv_u | su_d | sv_o | su_u] of each level (set ex.signs = ex.sc[level]
    before MoELayer.set).  Q* = {level: fp16 [N, K]} when want_Q, else None."""
    g, u, d = (repack(art[pn], dev)[0] for pn in PROJ)
    ex = types.SimpleNamespace(gu=cat_proj(g, u, dev), dn=d, H=d.N, I=d.K, lr=None, lr4=None, rg=0, rd=0)
    for p in (ex.gu, ex.dn):
        del p.p4w
        if hasattr(p, "bw"):
            del p.bw

    def lr_of(pn):                                     # a projection of rank 0 has no 'lr' entry
        P = art[pn]
        n, k = P["meta"]["n"], P["meta"]["k"]
        if "lr" not in P["base"]:
            return [torch.zeros(0, c, dtype=torch.float16) for c in (k, n, n)]
        return [P["base"]["lr"]["V"].cpu(), P["base"]["lr"]["U2"].cpu(), P["p4"]["lr"]["U4"].cpu()]

    (Vg, U2g, U4g), (Vu, U2u, U4u), (Vd, U2d, U4d) = (lr_of(pn) for pn in PROJ)
    if not torch.equal(Vg, Vu):
        raise AssertionError("the kernels need gate and up to share V")
    ex.rg, ex.rd = Vg.shape[0], Vd.shape[0]
    flat = lambda *ts: torch.cat([t.reshape(-1) for t in ts]).half().contiguous().to(dev)
    if ex.rg + ex.rd:
        ex.lr, ex.lr4 = flat(Vg, U2g, U2u, Vd, U2d), flat(U4g, U4u, U4d)

    def scales(lv):
        plane = {2: "base", 4: "p4"}[lv]
        v = lambda pn, key: art[pn][plane][key].half().to(dev)
        return torch.cat([v("gate", "suh"), v("gate", "svh"), v("up", "svh"), v("down", "suh"), v("down", "svh"), v("up", "suh")])

    ex.sc = {lv: scales(lv) for lv in (2, 4)}
    Q = (None, None, None)
    if want_Q:
        W = _dense(ex, lambda lv: ex.sc[lv])
        Q = ({lv: W[lv][0][:ex.I] for lv in W}, {lv: W[lv][0][ex.I:] for lv in W}, {lv: W[lv][1] for lv in W})
    return ex, scales, Q


def had_width(man):
    """width of the down projection's input rotation of a layer (manifest config.in_had_down; absent = 128)"""
    return int(man.get("config", {}).get("in_had_down", 128))


def p4_bytes(ex):
    """bytes of the level-4 part of one expert that a promotion streams: residual planes + block words (+ lr4)"""
    b = sum(p.p4.numel() * 4 + p.d4.numel() * 4 for p in (ex.gu, ex.dn))
    return b + (0 if ex.lr4 is None else ex.lr4.numel() * 2)


def layer_dir(root, L):
    """root/L{L} (the encoder's output) or root/layers/L{L} (the hub layout)"""
    d = f"{root}/L{L}"
    return d if os.path.exists(f"{d}/manifest.json") else f"{root}/layers/L{L}"


def _load_safetensors(path):
    """The shard dict from the safetensors container: tensors under flat keys, the dict skeleton (key order and types,
    non-tensor values) as JSON in the metadata field 'tree': {"D": [[key, node], ...]} | {"T": tensor key} | {"V": value}.
    One sequential read of the file."""
    with open(path, "rb") as f:
        blob = f.read()
    n = struct.unpack("<Q", blob[:8])[0]
    head = json.loads(blob[8:8 + n])
    meta = head.pop("__metadata__", {})
    if meta.get("format") != ST_FORMAT:
        raise ValueError(f"{path}: format {meta.get('format')!r}, expected {ST_FORMAT}")
    data = memoryview(blob)[8 + n:]

    def tensor(key):
        h = head[key]
        lo, hi = h["data_offsets"]
        dt = _ST_DTYPES[h["dtype"]]
        if hi == lo:
            return torch.zeros(h["shape"], dtype=dt)
        return torch.frombuffer(bytearray(data[lo:hi]), dtype=dt).reshape(h["shape"])

    def build(node):
        if "D" in node:
            return {k: build(v) for k, v in node["D"]}
        return tensor(node["T"]) if "T" in node else node["V"]

    return build(json.loads(meta["tree"]))


def load_part(d, i):
    """shard i of the layer directory d: tp{i}.pt, else tp{i}.safetensors (the same dict)"""
    if os.path.exists(f"{d}/tp{i}.pt"):
        return torch.load(f"{d}/tp{i}.pt", weights_only=False)
    return _load_safetensors(f"{d}/tp{i}.safetensors")


class RankLayer:
    """Every expert of MoE layer L that rank `rank` of a TP = tp run holds, as kernel planes on `dev`."""

    def __init__(s, root, L, rank, tp=4, experts=None, dev="cuda"):
        if NSH % tp or not 0 <= rank < tp:
            raise AssertionError(f"tp = {tp} must divide {NSH} and rank = {rank} lie below it")
        d = layer_dir(root, L)
        with open(f"{d}/manifest.json") as f:
            s.man = json.load(f)
        if s.man["format"] != "nestquant-v1":
            raise AssertionError(f"{d}: format {s.man['format']!r}")
        g = NSH // tp
        s.ss = list(range(rank * g, (rank + 1) * g))
        s.L, s.rank, s.tp, s.dev = L, rank, tp, dev
        s.parts = {i: load_part(d, i) for i in s.ss}
        s.experts = [E for E in s.man["experts"] if experts is None or E in experts]
        s.ex = {E: kernel_expert(group_art(s.parts, s.man, E, s.ss), dev)[0] for E in s.experts}
        down = s.man["proj_meta"]["down"]
        s.H, s.I = down["n"], down["k"] * g // NSH
        s.had_dn = had_width(s.man)
        if s.I % s.had_dn:
            raise AssertionError(f"layer {L}: I = {s.I} is not a multiple of the rotation width {s.had_dn}")
        for x in s.ex.values():
            x.had_dn = s.had_dn

    def art(s, E):
        return group_art(s.parts, s.man, E, s.ss)

    def slot_bytes(s, align=256):
        """size of a promotion slot: the largest p4_bytes over this layer's experts, rounded up to `align`"""
        m = max(p4_bytes(e) for e in s.ex.values())
        return (m + align - 1) // align * align
