"""The operator module of the NestQuant MoE layer: same Python-visible functions as the reference's torch extension
(sm120/nqmoe.cu:1294-1295 exports moe_forward, rk_codes, occ, mailbox, set_wdump, pf_decode, pf_pre, pf_mid, pf_post,
pf_hits), implemented over the C ABI of libnestquant_b200.so.  Tensors are caller-owned torch CUDA tensors; every call is
enqueued on the current torch CUDA stream and errors surface as RuntimeError (NestQuantError), as TORCH_CHECK did.
"""
import ctypes as C

import torch

from . import capi
from .capi import NestQuantError, check, current_stream, lib, ptr


def _need(t, dtype, name):
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == dtype and t.is_contiguous()):
        raise NestQuantError(f"{name}: expected a contiguous CUDA tensor of {dtype}")


def rk_codes():
    """[gate|up mask, down mask] of compiled residual window codes (bit c = code c)"""
    out = (C.c_int64 * 2)()
    check(lib().nq_rk_codes(out), "rk_codes")
    return [int(out[0]), int(out[1])]


def bk_codes():
    out = (C.c_int64 * 2)()
    check(lib().nq_bk_codes(out), "bk_codes")
    return [int(out[0]), int(out[1])]


def mailbox(table, stage, seq, applied, applied_host):
    """table[e] = stage[e] where seq[e] != applied[e]; applied_host: raw pointer of a pinned int32 [E] mirror or 0"""
    _need(table, torch.int64, "table"); _need(stage, torch.int64, "stage")
    _need(seq, torch.int32, "seq"); _need(applied, torch.int32, "applied")
    check(lib().nq_mailbox(ptr(table), ptr(stage), ptr(seq), ptr(applied), ptr(applied_host), table.shape[0],
                           current_stream()), "mailbox")


def pf_decode(table, experts, Wgu, Wdn, H, I, nm_gu, nm_dn, force_level=0):
    """Decode the listed experts (int32 ids, device) to dense fp16: Wgu [G,2I,H], Wdn [G,H,I] (None skips one)."""
    _need(table, torch.int64, "table"); _need(experts, torch.int32, "experts")
    G = experts.numel()
    for t, n, name in ((Wgu, G * 2 * I * H, "Wgu"), (Wdn, G * H * I, "Wdn")):
        if t is not None:
            _need(t, torch.float16, name)
            if t.numel() < n:
                raise NestQuantError(f"pf_decode sizes: {name} has {t.numel()} elements, needs {n}")
    check(lib().nq_pf_decode(ptr(table), ptr(experts), G, ptr(Wgu), ptr(Wdn), H, I, nm_gu, nm_dn, force_level,
                             current_stream()), "pf_decode")


def pf_pre(x, pt, pe, table, xg, xu, zg, I, kperm=False):
    """per pair (sorted by expert): xg / xu = fp16(WHT128(x * su_g / su_u)) [R,H], zg = x V_gu^T [R,4].
    kperm: write the k order the fused pf_gemm reads (see the header); False = the reference's plain order"""
    _need(x, torch.float16, "x"); _need(pt, torch.int32, "pt"); _need(pe, torch.int32, "pe"); _need(table, torch.int64, "table")
    _need(xg, torch.float16, "xg"); _need(xu, torch.float16, "xu"); _need(zg, torch.float32, "zg")
    R, H = pt.numel(), x.shape[1]
    if pe.numel() < R or xg.numel() < R * H or xu.numel() < R * H or zg.numel() < R * 4:
        raise NestQuantError("pf_pre sizes")
    check(lib().nq_pf_pre(ptr(x), ptr(pt), ptr(pe), R, ptr(table), table.shape[0], ptr(xg), ptr(xu), ptr(zg), H, I, int(bool(kperm)), current_stream()), "pf_pre")


def pf_pre_ep(peer_ptrs, tokens_per_rank, H, pt, pe, table, xg, xu, zg, I, kperm=False):
    """pf_pre with the input rows read from the ranks' buffers: peer_ptrs = device addresses (ints) of every rank's fp16
    [tokens_per_rank, H] input buffer as seen from this GPU; pt holds global token ids (rank * tokens_per_rank + t)"""
    _need(pt, torch.int32, "pt"); _need(pe, torch.int32, "pe"); _need(table, torch.int64, "table")
    _need(xg, torch.float16, "xg"); _need(xu, torch.float16, "xu"); _need(zg, torch.float32, "zg")
    R = pt.numel()
    if pe.numel() < R or xg.numel() < R * H or xu.numel() < R * H or zg.numel() < R * 4:
        raise NestQuantError("pf_pre_ep sizes")
    arr = (C.c_void_p * len(peer_ptrs))(*peer_ptrs)
    check(lib().nq_pf_pre_ep(arr, len(peer_ptrs), tokens_per_rank, ptr(pt), ptr(pe), R, ptr(table), table.shape[0], ptr(xg), ptr(xu),
                             ptr(zg), H, I, int(bool(kperm)), current_stream()), "pf_pre_ep")


def pf_mid(acc_g, acc_u, zg, pe, table, h, zd, H, I, kperm=False):
    """acc_g / acc_u fp32 [R,I] -> h fp16 [R,I] (rotations, scales, SwiGLU), zd [R,4]"""
    _need(acc_g, torch.float32, "acc_g"); _need(acc_u, torch.float32, "acc_u"); _need(zg, torch.float32, "zg")
    _need(pe, torch.int32, "pe"); _need(table, torch.int64, "table"); _need(h, torch.float16, "h"); _need(zd, torch.float32, "zd")
    R = pe.numel()
    if acc_g.numel() < R * I or acc_u.numel() < R * I or h.numel() < R * I or zd.numel() < R * 4 or zg.numel() < R * 4:
        raise NestQuantError("pf_mid sizes")
    check(lib().nq_pf_mid(ptr(acc_g), ptr(acc_u), ptr(zg), ptr(pe), R, ptr(table), table.shape[0], ptr(h), ptr(zd), H, I, int(bool(kperm)), current_stream()), "pf_mid")


def pf_post(y, zd, pt, pe, prw, table, out, I):
    """out[pt[p]] += prw[p] * (WHT128(y[p]) * sv_o + low rank); out fp32 [T,H], zeroed by the caller"""
    _need(y, torch.float32, "y"); _need(zd, torch.float32, "zd"); _need(pt, torch.int32, "pt"); _need(pe, torch.int32, "pe")
    _need(prw, torch.float16, "prw"); _need(table, torch.int64, "table"); _need(out, torch.float32, "out")
    R, H = pt.numel(), out.shape[1]
    if y.numel() < R * H or zd.numel() < R * 4 or prw.numel() < R or pe.numel() < R:
        raise NestQuantError("pf_post sizes")
    check(lib().nq_pf_post(ptr(y), ptr(zd), ptr(pt), ptr(pe), ptr(prw), R, ptr(table), table.shape[0], ptr(out), H, I, current_stream()), "pf_post")


def pf_combine(y, zd, pos, sel, rw, table, out, I, pair0=0, npairs=None, accumulate=False):
    """out[t] (+)= sum over the picks k of token t whose pair index pos[t,k] lies in [pair0, pair0 + npairs), in pick order, of
    rw[t,k] * (WHT128(y[pos[t,k] - pair0]) * sv_o + low rank).  y fp32 [npairs,H] and zd [npairs,4] hold that window of the
    expert-sorted pairs; npairs=None: the window is every pair.  accumulate=False overwrites out fp32 [T,H]."""
    _need(y, torch.float32, "y"); _need(zd, torch.float32, "zd"); _need(pos, torch.int32, "pos"); _need(sel, torch.int64, "sel")
    _need(rw, torch.float16, "rw"); _need(table, torch.int64, "table"); _need(out, torch.float32, "out")
    T, topk = sel.shape
    H = out.shape[1]
    npairs = T * topk if npairs is None else npairs
    if pos.numel() < T * topk or rw.numel() < T * topk or out.numel() < T * H or y.numel() < npairs * H or zd.numel() < npairs * 4:
        raise NestQuantError("pf_combine sizes")
    check(lib().nq_pf_combine(ptr(y), ptr(zd), ptr(pos), ptr(sel), ptr(rw), T, topk, ptr(table), table.shape[0], ptr(out), H, I,
                              pair0, npairs, int(bool(accumulate)), current_stream()), "pf_combine")


def pf_sort_scratch_ints(pairs, E):
    return int(lib().nq_pf_sort_scratch_ints(pairs, E))


def pf_sort(sel, rw, table, pe, pt, pos, start, hit_counts, scratch):
    """the (token, pick) pairs sorted by expert on the device (stable counting sort, no host sync): pe / pt int32 [T*topk]
    expert (E = contributes nothing) and token of each sorted pair, pos int32 [T*topk] sorted index of each pick, start int32
    [E+2] first pair of each bin; hit_counts int32 [E] (zeroed by the caller) or None; scratch int32 [pf_sort_scratch_ints]"""
    _need(sel, torch.int64, "sel"); _need(rw, torch.float16, "rw"); _need(table, torch.int64, "table")
    for t, n in ((pe, "pe"), (pt, "pt"), (pos, "pos"), (start, "start"), (scratch, "scratch")):
        _need(t, torch.int32, n)
    T, topk = sel.shape
    E, P = table.shape[0], T * topk
    if rw.numel() < P or pe.numel() < P or pt.numel() < P or pos.numel() < P or start.numel() < E + 2 or (hit_counts is not None and hit_counts.numel() < E):
        raise NestQuantError("pf_sort sizes")
    check(lib().nq_pf_sort(ptr(sel), ptr(rw), ptr(table), T, topk, E, ptr(pe), ptr(pt), ptr(pos), ptr(start), ptr(hit_counts), ptr(scratch),
                           scratch.numel(), current_stream()), "pf_sort")


def pf_plan_window(start, table, plan, pair0, npairs):
    """pass list of the fused prefill GEMM for the pairs [pair0, pair0 + npairs) of a sorted window (start from pf_sort)"""
    _need(start, torch.int32, "start"); _need(table, torch.int64, "table"); _need(plan, torch.int32, "plan")
    check(lib().nq_pf_plan_window(ptr(start), ptr(table), table.shape[0], pair0, npairs, ptr(plan), plan.numel(), current_stream()), "pf_plan_window")


def pf_plan_ints(E, pairs):
    return int(lib().nq_pf_plan_ints(E, pairs))


def pf_plan(counts, table, plan, pairs):
    """pass list of the fused prefill GEMM from per-expert pair counts (int32 [E], device); plan int32 [pf_plan_ints]"""
    _need(counts, torch.int32, "counts"); _need(table, torch.int64, "table"); _need(plan, torch.int32, "plan")
    check(lib().nq_pf_plan(ptr(counts), ptr(table), table.shape[0], pairs, ptr(plan), plan.numel(), current_stream()), "pf_plan")


def pf_gemm(table, plan, act0, act1, out0, out1, H, I, nm_gu, nm_dn, down, status):
    """fused decode + grouped GEMM of one projection over the expert-sorted pairs (see nq_pf_gemm)"""
    _need(table, torch.int64, "table"); _need(plan, torch.int32, "plan"); _need(act0, torch.float16, "act0")
    _need(out0, torch.float32, "out0"); _need(status, torch.int32, "status")
    pairs, K, N = act0.shape[0], (I if down else H), (H if down else I)
    if act0.dim() != 2 or act0.shape[1] != K or out0.numel() < pairs * N:
        raise NestQuantError("pf_gemm sizes")
    if not down:
        _need(act1, torch.float16, "act1"); _need(out1, torch.float32, "out1")
        if act1.shape != act0.shape or out1.numel() < pairs * N:
            raise NestQuantError("pf_gemm sizes")
    check(lib().nq_pf_gemm(ptr(table), ptr(plan), ptr(act0), ptr(act1), pairs, ptr(out0), ptr(out1), H, I, nm_gu, nm_dn,
                           1 if down else 0, ptr(status), current_stream()), "pf_gemm")


def pf_hits(counts, hits_ptr):
    """hits[e] += counts[e]; hits_ptr: raw (host-mapped) int32 [E] pointer or 0"""
    if not hits_ptr:
        return
    _need(counts, torch.int32, "counts")
    check(lib().nq_pf_hits(ptr(counts), hits_ptr, counts.numel(), current_stream()), "pf_hits")


def operand_order(K):
    """int64 [K]: position of element k of a row in the "operand order" of the decode path's internal fp16 rows (h and the
    rotated inputs): inside every 128 consecutive k, k = 16 T + 2 t4 + 8 hi + e sits at 32 t4 + 4 T + 2 hi + e"""
    k = torch.arange(K)
    kk = k % 128
    T, q = kk >> 4, kk & 15
    return (k - kk) + 32 * ((q & 7) >> 1) + 4 * T + 2 * (q >> 3) + (q & 1)


def kperm_order(K):
    """int64 [K]: position of element k of a row in the k order the fused prefill GEMM reads (pf_pre / pf_mid with
    kperm=True): inside every 16 consecutive k, position 4 i + {0, 1} holds k = 2 i + {0, 1} and 4 i + {2, 3} holds 8 + 2 i + {0, 1}"""
    k = torch.arange(K)
    q = k % 16
    return (k - q) + 4 * ((q & 7) >> 1) + 2 * (q >> 3) + (q & 1)


def default_ksplit(B, H, I, share=1.0, topk=8):
    """k-slices per strip (gate|up, down) for a B-token call.  The persistent kernel hands out pieces (a 16-row strip over
    1 / k-slices of its chunks) to ~3,000 warps: the split aims at ~8 units (16 x 128 weights) per piece, between 3,000
    and 8,192 gate|up pieces and between 1,536 and 6,144 down pieces - what sweeps of the GLM shape and of its
    tensor-parallel shards (I / 2, I / 4, I / 8) at 1, 2 and 4 tokens settled on.
    share: fraction of the layer's experts resident on this GPU (expert parallelism: 1 / ranks; 1 for one GPU and for
    tensor-parallel shards, whose I is the shard's)."""
    import math
    Cg, Cd = H // 128, I // 128
    if share < 1.0:
        # expert parallelism: a rank's load swings with the routing (0 .. topk picks of a token), and the call waits for the
        # fullest rank; the table below is what sweeps with 1 / 2, 1 / 4 and 1 / 8 of the experts resident settled on
        load = B * share
        want = (8, 4) if load <= 0.5 else (4, 2) if load <= 1 else (2, 1) if load <= 4 else (1, 1)
        fit = lambda chunks, w: max(d for d in range(1, w + 1) if chunks % d == 0)
        return fit(Cg, want[0]), fit(Cd, want[1])
    runs = max(1.0, B * topk)                              # distinct experts a call activates, roughly

    def nearest(chunks, want):
        divs = [d for d in range(1, chunks + 1) if chunks % d == 0 and d <= 24]
        return min(divs, key=lambda d: abs(math.log(d / max(want, 1e-9))))

    per_ks_gu = runs * Cd * 16                             # gate|up pieces per k-slice: strips of gate and up
    per_ks_dn = runs * Cg * 8                              # down pieces per k-slice
    want_gu = min(max(per_ks_gu * Cg / 8, 3000), 8192) / per_ks_gu
    want_dn = min(max(per_ks_dn * Cd / 8, 1536), 6144) / per_ks_dn
    return nearest(Cg, want_gu), nearest(Cd, want_dn)


def moe_workspace(B, topk, H, I, ks_gu, ks_dn):
    """element counts of the workspace tensors of moe_forward for a call shape"""
    w = capi.NqMoeWorkspace()
    check(lib().nq_moe_workspace(B, topk, H, I, ks_gu, ks_dn, C.byref(w)), "moe_workspace")
    return {n: int(getattr(w, n)) for n, _ in capi.NqMoeWorkspace._fields_}


def moe_forward(x, sel, rw, table, out, acc_gu, h, acc_d, cnt_gu, cnt_d, wq, I, nm_gu, nm_dn, cfg_gu, cfg_dn, G,
                force_level, which, hits_ptr, zd, cnt_h, ep=None):
    """One MoE layer call on the decode path, positional arguments as in the reference's moe_forward.
    cfg_gu / cfg_dn: [k-slices per strip] (entries after the first are accepted and ignored).
    ep = (world, rank, receive-buffer addresses of all ranks, counter addresses of all ranks, epoch tensor): this rank's call of
    an expert-parallel group, the partial outputs of all ranks summed inside the kernel over peer memory (nq_moe_forward_ep)."""
    _need(x, torch.float16, "x"); _need(rw, torch.float16, "rw"); _need(sel, torch.int64, "sel")
    _need(table, torch.int64, "table"); _need(out, torch.float32, "out"); _need(acc_gu, torch.float32, "acc_gu")
    _need(h, torch.float16, "h"); _need(acc_d, torch.float32, "acc_d"); _need(zd, torch.float32, "zd")
    for t, n in ((cnt_gu, "cnt_gu"), (cnt_d, "cnt_d"), (wq, "wq"), (cnt_h, "cnt_h")):
        _need(t, torch.int32, n)
    if x.dim() != 2 or sel.dim() != 2 or sel.shape[0] != x.shape[0] or rw.shape != sel.shape:
        raise NestQuantError("moe_forward: x [B,H], sel [B,topk], rw [B,topk]")
    a = capi.NqMoeForward()
    for n, t in (("x", x), ("sel", sel), ("rw", rw), ("table", table), ("out", out), ("acc_gu", acc_gu), ("h", h),
                 ("acc_d", acc_d), ("cnt_gu", cnt_gu), ("cnt_d", cnt_d), ("wq", wq), ("zd", zd), ("cnt_h", cnt_h)):
        setattr(a, n, t.data_ptr())
    a.hits = hits_ptr or None
    a.out_floats, a.acc_gu_floats, a.h_halves, a.acc_d_floats = out.numel(), acc_gu.numel(), h.numel(), acc_d.numel()
    a.cnt_gu_ints, a.cnt_d_ints, a.wq_ints, a.zd_floats, a.cnt_h_ints = (cnt_gu.numel(), cnt_d.numel(), wq.numel(),
                                                                        zd.numel(), cnt_h.numel())
    a.B, a.topk, a.E, a.H, a.I = x.shape[0], sel.shape[1], table.shape[0], x.shape[1], I
    a.nm_gu, a.nm_dn, a.ks_gu, a.ks_dn = nm_gu, nm_dn, int(cfg_gu[0]), int(cfg_dn[0])
    a.G, a.force_level, a.which = G, force_level, which
    if ep is None:
        check(lib().nq_moe_forward(C.byref(a), current_stream()), "moe_forward")
        return
    world, rank, recv_ptrs, cnt_ptrs, epoch = ep
    d = capi.NqMoeEp()
    d.world, d.rank = world, rank
    d.peer_recv, d.peer_counters = (C.c_void_p * world)(*recv_ptrs), (C.c_void_p * world)(*cnt_ptrs)
    d.epoch = epoch.data_ptr()
    check(lib().nq_moe_forward_ep(C.byref(a), C.byref(d), current_stream()), "moe_forward_ep")


def moe_forward_static(x, sel, rw, table, out, I, nm_gu, nm_dn, ks_gu, ks_dn, hits_ptr=0):
    """moe_forward for hosts that must not allocate (a plugin inside an engine that owns all device memory, a thread
    that may not call the allocator): the workspaces come from a 4 MiB array built into the library, shared by every
    call on the device.  Raises if the call shape needs more; calls that overlap on the GPU race on the array."""
    _need(x, torch.float16, "x"); _need(rw, torch.float16, "rw"); _need(sel, torch.int64, "sel")
    _need(table, torch.int64, "table"); _need(out, torch.float32, "out")
    if x.dim() != 2 or sel.dim() != 2 or sel.shape[0] != x.shape[0] or rw.shape != sel.shape or out.numel() < x.numel():
        raise NestQuantError("moe_forward_static: x [B,H], sel [B,topk], rw [B,topk], out [B,H]")
    check(lib().nq_moe_forward_static(ptr(x), ptr(sel), ptr(rw), ptr(table), ptr(out), x.shape[0], sel.shape[1], table.shape[0],
                                      x.shape[1], I, nm_gu, nm_dn, ks_gu, ks_dn, hits_ptr or None, current_stream()),
          "moe_forward_static")


def sal(x, w, ids, rsf, acc, host_ptr=0):
    """salience export of one decode call (the reference's nqsal.sal): acc[e] += (rsf * w)^2 * |x[t]|^2 over the picks of e.
    x fp16 / bf16 [T,H] (rows may be strided), w fp16 [T,topk], ids int64 [T,topk], acc fp64 [E] (device),
    host_ptr: raw address of a host-mapped fp64 [E] mirror, or 0"""
    if x.dtype not in (torch.float16, torch.bfloat16) or x.dim() != 2 or x.stride(1) != 1:
        raise NestQuantError("sal: x must be fp16 or bf16 [T, H] with unit column stride")
    _need(w, torch.float16, "w"); _need(ids, torch.int64, "ids"); _need(acc, torch.float64, "acc")
    T, H = x.shape
    if w.numel() != ids.numel() or (T and ids.numel() % T):
        raise NestQuantError("sal sizes")
    check(lib().nq_salience(ptr(x), int(x.dtype == torch.bfloat16), x.stride(0) if T else H, ptr(w), ptr(ids), T, H,
                            ids.shape[1], acc.numel(), float(rsf), ptr(acc), host_ptr or None, current_stream()), "sal")
