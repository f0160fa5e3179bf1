"""Generates the production-shard fixtures and what the reference's own loader (sm120/nqload.py) makes of them.

    python tests/golden/make_golden_nqload.py /path/to/nestquant

Inputs (written here from a seeded torch generator, no encoder run: the loader only moves bits, so random streams do):
  nqload/L3/{manifest.json, tp0.pt, tp1.pt}   nestquant-v1 layer, H 128, 2 of the 8 TP shards (I 256 each), experts 0 and 3,
                                              base K 2, residual K 2 (gate, up) / 2.3125 (down); expert 3 carries a
                                              rank-2 / rank-1 low-rank plane with gate and up sharing V
  nqload/L4/{manifest.json, tp0.pt}           the pattern-rate format: base K 1.75, residual K 2.25 / 2.5625, expert 1
  nqload_st/layers/L4/{manifest.json, tp0.safetensors}   the same shard in the safetensors container, written by the
                                              reference's threads/25-campaign/nq25_st.save_shard, in the hub's directory layout
Outputs, from the reference (nqload.RankLayer / kernel_expert on CPU, torch shims as in make_golden.py):
  nqload.npz   for every (layer, tp, rank, expert): SHA-256 of the bytes of each kernel plane (base, p4, d4, var of gate|up
               and down, both scale vectors, lr, lr4), the plane sizes, slot_bytes(); the planes themselves for the smallest
               case; and, for that case, the dense matrices Q2 / Q4 that the ENCODER-side decoder (threads/12
               nq_decode.ring_levels) derives from the same streams: their SHA-256 (fp16 bit patterns, -0 folded into
               +0) and their first 32 rows (layer L3 only: that decoder has no pattern-rate base).
"""
import hashlib
import json
import os
import sys
import types

import numpy as np
import torch

if len(sys.argv) < 2:
    raise SystemExit(__doc__)
REF = sys.argv[1]
OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "nqload")
sys.path[:0] = [os.path.join(REF, "sm120")]
sys.modules["build"] = types.SimpleNamespace(get=lambda *a, **k: None, get_sal=lambda *a, **k: None)
import nqload  # noqa: E402  (adds the encoder thread to sys.path itself)

NSH, H, ISH = 8, 128, 256           # shards of the format, hidden size, intermediate columns per shard
RING_BYTES = {2: 64, 1.75: 56, 2.25: 72, 2.3125: 74, 2.5625: 82}      # 256 steps of K bits


def make_layer(L, shards, experts, base_K, K_gu, K_dn, lr_of, seed):
    g = torch.Generator().manual_seed(seed)
    rb = lambda n: torch.randint(0, 256, (n,), generator=g, dtype=torch.uint8)
    sc = lambda n: (torch.randn(n, generator=g) * 0.05).abs().half() + 0.01
    sg = lambda n: (torch.randint(0, 2, (n,), generator=g) * 2 - 1).half()
    meta = {}
    for pn in ("gate", "up", "down"):
        k, n = (ISH * NSH, H) if pn == "down" else (H, ISH * NSH)
        m = dict(k=k, n=n, tk=k // 128, tn=n // 16, shard_axis="k" if pn == "down" else "n", base_var="sign",
                 res_rule=dict(kind="uniform", K=K_dn if pn == "down" else K_gu))
        if base_K != 2:
            m["base_K"] = base_K
        meta[pn] = m
    parts = {s: {} for s in shards}
    for E in experts:
        rg, rd = lr_of.get(E, (0, 0))
        Vg = (torch.randn(rg, H, generator=g) * 0.05).half()
        for s in shards:
            d = {}
            for pn in ("gate", "up", "down"):
                U = 16                                   # units of one shard: 16 strips x 1 chunk, or 8 strips x 2 chunks
                Kr = K_dn if pn == "down" else K_gu
                word_m = torch.randint(100, 256, (U,), generator=g)
                word_n = torch.minimum((torch.rand(U, generator=g) * 0.8 * word_m).long(), 257 - word_m)
                p = dict(base=rb(U * 8 * RING_BYTES[base_K]), p4=rb(U * 8 * RING_BYTES[Kr]), word=(word_m | (word_n << 8)).to(torch.int32),
                         var=torch.randint(0, 2, (U * 8,), generator=g).to(torch.uint8))
                kin, nout = (ISH, H) if pn == "down" else (H, ISH)
                p.update(suh2=sg(kin), svh2=sc(nout), suh4=sg(kin), svh4=sc(nout))
                if pn == "down" and rd:
                    p.update(lrV=(torch.randn(rd, ISH, generator=g) * 0.05).half(), lrU2=None, lrU4=None)
                elif pn != "down" and rg:
                    p.update(lrU2=(torch.randn(rg, ISH, generator=g) * 0.05).half(), lrU4=(torch.randn(rg, ISH, generator=g) * 0.05).half())
                    if pn == "gate":
                        p["lrV"] = Vg
                    else:
                        p["lrV_from"] = "gate"
                d[pn] = p
            parts[s][E] = d
        if rd:                                            # replicated parts of the down plane: the same tensors in every shard
            U2, U4 = (torch.randn(rd, H, generator=g) * 0.05).half(), (torch.randn(rd, H, generator=g) * 0.05).half()
            for s in shards:
                parts[s][E]["down"].update(lrU2=U2, lrU4=U4)
        for s in shards:                                  # replicated scale vectors: gate/up input side, down output side
            for pn in ("gate", "up", "down"):
                for key in (("suh2", "suh4") if pn != "down" else ("svh2", "svh4")):
                    parts[s][E][pn][key] = parts[shards[0]][E][pn][key]
    d = os.path.join(OUT, f"L{L}")
    os.makedirs(d, exist_ok=True)
    for s in shards:
        torch.save(parts[s], os.path.join(d, f"tp{s}.pt"))
    man = dict(format="nestquant-v1", layer=L, experts=list(experts), tp=NSH, proj_meta=meta, config=dict(base_var="sign", in_had_down=128))
    json.dump(man, open(os.path.join(d, "manifest.json"), "w"), indent=1)


make_layer(3, (0, 1), (0, 3), 2, 2, 2.3125, {3: (2, 1)}, seed=4103)
make_layer(4, (0,), (1,), 1.75, 2.25, 2.5625, {}, seed=4104)

sys.path.append(os.path.join(REF, "threads", "25-campaign"))
import nq25_st  # noqa: E402

ST = os.path.join(os.path.dirname(OUT), "nqload_st", "layers", "L4")
os.makedirs(ST, exist_ok=True)
nq25_st.save_shard(torch.load(os.path.join(OUT, "L4", "tp0.pt"), weights_only=False), os.path.join(ST, "tp0.safetensors"), 4, 0)
with open(os.path.join(ST, "manifest.json"), "w") as f:
    f.write(open(os.path.join(OUT, "L4", "manifest.json")).read())

sha = lambda t: hashlib.sha256(t.contiguous().cpu().numpy().tobytes()).hexdigest()
out = {}


def fp16_bits(q):
    b = q.contiguous().view(torch.int16).clone()
    b[b == -32768] = 0                                    # -0 -> +0
    return b


def record(tag, ex, full):
    for pj, p in (("gu", ex.gu), ("dn", ex.dn)):
        for k in ("base", "p4", "d4", "var"):
            t = getattr(p, k)
            out[f"{tag}.{pj}.{k}.sha"] = np.array(sha(t))
            out[f"{tag}.{pj}.{k}.numel"] = np.array([t.numel(), t.element_size()])
            if full:
                out[f"{tag}.{pj}.{k}"] = t.cpu().numpy()
        out[f"{tag}.{pj}.codes"] = np.array([p.N, p.K, p.rk, p.bk])
    for lv in (2, 4):
        out[f"{tag}.sc{lv}.sha"] = np.array(sha(ex.sc[lv]))
        if full:
            out[f"{tag}.sc{lv}"] = ex.sc[lv].cpu().view(torch.int16).numpy()
    out[f"{tag}.ranks"] = np.array([ex.rg, ex.rd, ex.H, ex.I])
    if ex.lr is not None:
        out[f"{tag}.lr.sha"], out[f"{tag}.lr4.sha"] = np.array(sha(ex.lr)), np.array(sha(ex.lr4))
    out[f"{tag}.p4_bytes"] = np.array([nqload.p4_bytes(ex)])


for L, tp, rank in ((3, 8, 0), (3, 8, 1), (3, 4, 0), (4, 8, 0)):
    RL = nqload.RankLayer(OUT, L, rank, tp=tp, dev="cpu")
    out[f"L{L}.tp{tp}.r{rank}.slot_bytes"] = np.array([RL.slot_bytes(), RL.H, RL.I, RL.had_dn])
    for E in RL.experts:
        tag = f"L{L}.tp{tp}.r{rank}.E{E}"
        record(tag, RL.ex[E], full=(L, tp, rank, E) in ((3, 8, 0, 0), (4, 8, 0, 1)))
        if (L, tp, rank) == (3, 8, 0):                    # dense matrices by the encoder-side decoder (it knows base K 2 only)
            ex, _, (Qg, Qu, Qd) = nqload.kernel_expert(RL.art(E), "cpu", want_Q=True)
            for lv in (2, 4):
                gu = fp16_bits(torch.cat([Qg[lv], Qu[lv]]))
                dn = fp16_bits(Qd[lv])
                out[f"{tag}.Q{lv}.gu.sha"], out[f"{tag}.Q{lv}.dn.sha"] = np.array(sha(gu)), np.array(sha(dn))
                out[f"{tag}.Q{lv}.gu.head"], out[f"{tag}.Q{lv}.dn.head"] = gu[:32].numpy(), dn[:32].numpy()
np.savez_compressed(os.path.join(os.path.dirname(OUT), "nqload.npz"), **out)
for root, _, files in list(os.walk(OUT)) + list(os.walk(os.path.dirname(os.path.dirname(ST)))):
    for f in files:
        print(os.path.join(root, f), os.path.getsize(os.path.join(root, f)))
print("nqload.npz", os.path.getsize(os.path.join(os.path.dirname(OUT), "nqload.npz")), len(out), "entries")
