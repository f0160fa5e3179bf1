"""Cross-check of the fused prefill GEMM: the same prefill computed the way the reference does it (sm120/moe.py:282-327) -
decode groups of experts to dense fp16 with pf_decode, multiply with library GEMMs (aten.mm), and run the same pf_pre /
pf_mid / pf_post / pf_combine passes around them.  Test infrastructure only: nothing in the package uses it."""
import torch


def prefill_library(L, x, sel, rw, R=8192, G=16, deterministic=True):
    """L: MoELayer.  x fp16 [T,H], sel int64 [T,topk], rw fp16 [T,topk] -> fp32 [T,H].
    R: pairs per scratch chunk, G: experts decoded per group.  deterministic: sum each token's picks in pick order
    (pf_combine over one pairs-sized buffer) instead of atomic adds (pf_post)."""
    T, k = sel.shape
    H, I, E, M, dev, tb = L.H, L.I, L.E, L.M, x.device, L.table
    f16, f32, i32 = torch.float16, torch.float32, torch.int32
    out = torch.empty(T, H, dtype=f32, device=dev)
    flat, rwf = sel.reshape(-1), rw.reshape(-1)
    order = torch.argsort(flat, stable=True)
    pe, pt, prw = flat[order].to(i32), (order // k).to(i32), rwf[order].contiguous()
    cnt = torch.bincount(flat, minlength=E).cpu().tolist()
    start, o = [0] * E, 0
    for e in range(E):
        start[e] = o; o += cnt[e]
    live = [e for e in range(E) if cnt[e]]
    P = T * k
    if deterministic:
        y_all = torch.empty(P, H, dtype=f32, device=dev)
        zd_all = torch.zeros(P, 4, dtype=f32, device=dev)
        pos = torch.empty(P, dtype=i32, device=dev)
        pos[order] = torch.arange(P, dtype=i32, device=dev)
    else:
        out.zero_()
    Wgu = torch.empty(G, 2 * I, H, dtype=f16, device=dev)
    Wdn = torch.empty(G, H, I, dtype=f16, device=dev)
    xg, xu = torch.empty(R, H, dtype=f16, device=dev), torch.empty(R, H, dtype=f16, device=dev)
    acc = torch.empty(2, R, I, dtype=f32, device=dev)
    hbuf = torch.empty(R, I, dtype=f16, device=dev)
    zg = torch.zeros(R, 4, dtype=f32, device=dev)
    zd = torch.zeros(R, 4, dtype=f32, device=dev)
    ybuf = None if deterministic else torch.empty(R, H, dtype=f32, device=dev)
    ids = torch.tensor(live, dtype=i32, device=dev)
    mm = torch.ops.aten.mm.dtype_out
    for g0 in range(0, len(live), G):
        grp = live[g0:g0 + G]
        M.pf_decode(tb, ids[g0:g0 + len(grp)], Wgu, Wdn, H, I, L.nm_gu, L.nm_dn)
        a, b = start[grp[0]], start[grp[-1]] + cnt[grp[-1]]
        for c in range(a, b, R):
            d = min(b, c + R)
            n = d - c
            M.pf_pre(x, pt[c:d], pe[c:d], tb, xg, xu, zg, I)
            y = y_all[c:d] if deterministic else ybuf[:n]
            segs = []
            for j, e in enumerate(grp):
                u, v = max(start[e], c) - c, min(start[e] + cnt[e], d) - c
                if v > u:
                    segs.append((j, u, v))
            for j, u, v in segs:
                mm(xg[u:v], Wgu[j, :I].t(), f32, out=acc[0, u:v]); mm(xu[u:v], Wgu[j, I:].t(), f32, out=acc[1, u:v])
            M.pf_mid(acc[0], acc[1], zg, pe[c:d], tb, hbuf, zd_all[c:d] if deterministic else zd, H, I)
            for j, u, v in segs:
                mm(hbuf[u:v], Wdn[j].t(), f32, out=y[u:v])
            if not deterministic:
                M.pf_post(y, zd, pt[c:d], pe[c:d], prw[c:d], tb, out, I)
    if deterministic:
        M.pf_combine(y_all, zd_all, pos, sel, rw, tb, out, I)
    return out
