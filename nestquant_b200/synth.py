"""Seeded synthetic workloads with the shapes, sizes and value distributions of the GLM-5-shaped MoE layer the
reference is measured on (no checkpoint or dataset is needed or used):

  planes     uniform random packed words (Proj / Expert in nestquant_b200.moe), block words from the 'rand' recipe,
             ring signs on, gate|up residual K = 2 (code 0), down residual K = 2.3125 (code 7): the 4.1-bpw layout
  scales     +-1 input signs, |N(0, 0.02)| output scales
  level map  the `n4` most frequently routed experts at level 4, the rest at level 2
  routing    logits N(0,1) (bf16) + beta * log Zipf(1.1) per-expert bias, top-k, softmax over the k
  tokens     bf16 N(0,1), cast to fp16 at the boundary
"""
import math

import torch

from . import moe

GLM = dict(E=256, topk=8, H=6144, I=2048)
C0 = dict(E=64, topk=4, H=1024, I=512)


def zipf_bias(E, seed, alpha=1.1):
    """log-probabilities of a Zipf(alpha) law over a seeded random permutation of the experts"""
    g = torch.Generator().manual_seed(seed)
    rank = torch.randperm(E, generator=g).float() + 1.0
    p = rank.pow(-alpha)
    return (p / p.sum()).log()


def routing(T, E, topk, seed, bias=None, beta=1.0):
    """-> sel int64 [T, topk], rw fp16 [T, topk] (CPU tensors)"""
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g).bfloat16().float()
    if bias is not None:
        logits = logits + beta * bias
    tv, sel = logits.topk(topk, dim=1)
    return sel, torch.softmax(tv, 1).half()


def tokens(T, H, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(T, H, generator=g).bfloat16().half()


def level_map(E, bias, n4):
    """level 4 for the n4 experts with the largest routing bias, level 2 for the rest"""
    lv = [2] * E
    for e in torch.argsort(bias, descending=True)[:n4].tolist():
        lv[e] = 4
    return lv


def share_at_level4(levels, bias, beta, E, topk, samples=2048, seed=1234):
    sel, _ = routing(samples, E, topk, seed, bias, beta)
    l4 = torch.tensor([lv == 4 for lv in levels])
    return float(l4[sel].float().mean())


def fit_beta(levels, bias, E, topk, target=0.63):
    """bias strength for which about `target` of the activated picks land on level-4 experts"""
    lo, hi = 0.0, 4.0
    for _ in range(20):
        mid = 0.5 * (lo + hi)
        if share_at_level4(levels, bias, mid, E, topk) < target:
            lo = mid
        else:
            hi = mid
    return 0.5 * (lo + hi)


def fixed_bias(E, n_fixed, seed):
    """indicator (1 / 0) of n_fixed seeded 'fixed' experts, to be scaled by fit_share"""
    g = torch.Generator().manual_seed(seed)
    b = torch.zeros(E)
    b[torch.randperm(E, generator=g)[:n_fixed]] = 1.0
    return b


def fit_share(bias, E, topk, target=0.5, samples=2048, seed=4321):
    """bias strength for which the experts with bias > 0 take about `target` of the picks"""
    lo, hi = 0.0, 8.0
    hot = bias > 0
    for _ in range(20):
        mid = 0.5 * (lo + hi)
        sel, _ = routing(samples, E, topk, seed, bias, mid)
        if float(hot[sel].float().mean()) < target:
            lo = mid
        else:
            hi = mid
    return 0.5 * (lo + hi)


def build_layer(cfg, levels, seed=0, dev="cuda", Bmax=4, owned=None, masked=(), nm_frac=0.5):
    """Experts + MoELayer.  owned: expert ids resident on this GPU (others stay at level 0 and get no planes)."""
    E, topk, H, I = cfg["E"], cfg["topk"], cfg["H"], cfg["I"]
    nm_gu, nm_dn = max(1, int(H // 128 * nm_frac)), max(1, int(I // 128 * nm_frac))
    L = moe.MoELayer(E, H, I, nm_gu if masked else 0, nm_dn if masked else 0, Bmax=Bmax, topk=topk, dev=dev,
                     share=1.0 if owned is None else len(owned) / E)
    experts = {}
    for e in (range(E) if owned is None else owned):
        if levels[e] <= 0:
            continue
        m = e in masked
        ex = moe.Expert(H, I, seed=seed * 100003 + e, nm_gu=nm_gu if m else None, nm_dn=nm_dn if m else None, dev=dev,
                        rk_gu=0, rk_dn=7, var=True, sv=0.02, gen_device=dev if str(dev).startswith("cuda") else "cpu")
        experts[e] = ex
        L.set(e, ex, levels[e])
    return L, experts


def plane_bytes(experts, levels, sel, H, I):
    """algorithmic bytes of a decode-path call: packed planes + scales of the distinct activated resident experts"""
    n = 0
    for e in set(sel.reshape(-1).tolist()):
        if e in experts and levels[e] > 0:
            n += experts[e].bytes(levels[e]) + (3 * H + 3 * I) * 2
    return n
