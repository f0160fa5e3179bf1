"""Host side of the NestQuant MoE layer on B200: plane generators, device table rows, the layer object and the mailbox.

Mirrors the operator surface of the reference's sm120/moe.py (same class and function names, argument meaning and
error behaviour) so scripts written against it run unchanged:
  RKP / rbits / proj_sizes / make_flags / pack_words / unpack_words   sm120/moe.py:10-63
  Proj, Expert, entry                                                  sm120/moe.py:76-107,174-229
  MoELayer (.set / __call__ / .prefill), Mailbox                       sm120/moe.py:231-342
Everything that computes runs in the CUDA library behind nestquant_b200.ext; there is no torch or CPU fallback here
(the dense reference decode of the original module lives in the test oracle, not in this package).
"""
import torch

from . import ext as _ext

TBL_W = 20

# window pattern per code: step p of a ring is KA + ((MASK >> (p % 16)) & 1) bits wide
RKP = {0: (2, 0x0000), 1: (1, 0xEEEE), 2: (2, 0xAAAA), 3: (2, 0x8888), 4: (3, 0x0000), 5: (1, 0xAAAA),
       6: (1, 0xFFFE), 7: (2, 0x9248), 8: (1, 0xFEFE), 9: (2, 0xD5AA)}
RK_OF = {2: 0, 1.75: 1, 2.5: 2, 2.25: 3, 3: 4, 1.5: 5, 1.9375: 6, 2.3125: 7, 1.875: 8, 2.5625: 9}


def popc(m):
    return bin(m).count("1")


def rbits(rk):
    """bits of one lane record (64 weights) for window code rk"""
    ka, mask = RKP[rk]
    return 4 * (16 * ka + popc(mask))


def split_bits(bits):
    """pieces of a record in the sub-array layout: (#128-bit, has 64, has 32, has 16, tail bits)"""
    r = bits % 128
    return bits // 128, (r >> 6) & 1, (r >> 5) & 1, (r >> 4) & 1, bits % 16


def proj_sizes(N, K, nm=None, rk=0, bk=0):
    """bytes per plane of an N x K projection; nm = flagged chunks per strip in mask mode (None = every chunk refined)"""
    S, C = N // 16, K // 128
    R = C if nm is None else nm
    plane = lambda nrec, code: nrec * rbits(code) // 8 + (4 if rbits(code) % 16 else 0)
    return dict(S=S, C=C, nm=nm, rk=rk, bk=bk, base=plane(S * C * 32, bk), p4=plane(S * R * 32, rk), d4=S * R * 4,
                flags=0 if nm is None else S * 8, nrec_r=S * R * 32)


def make_flags(S, C, nm, gen, grp=8):
    """nm flagged chunks per strip, identical over each group of `grp` strips -> (int64 [S], bool [S, C])"""
    ng = (S + grp - 1) // grp
    pick = torch.rand(ng, C, generator=gen).argsort(1)[:, :nm]
    fl = torch.zeros(ng, C, dtype=torch.bool)
    fl.scatter_(1, pick, True)
    fl = fl.repeat_interleave(grp, 0)[:S]
    return (fl.long() << torch.arange(C)).sum(1), fl


def _pieces(bits):
    """(stream bit offset, width) of each sub-array of a record, in storage order"""
    n4, n2, n1, nh, T = split_bits(bits)
    out, o = [], 0
    if n4:
        out.append((0, 128 * n4)); o = 128 * n4
    for has, w in ((n2, 64), (n1, 32), (nh, 16)):
        if has:
            out.append((o, w)); o += w
    if T:
        out.append((o, T))
    return out


def _to_bits(words, bits):
    """int64 [nrec, nw] of uint32 values -> uint8 {0,1} [nrec, bits], LSB first"""
    sh = torch.arange(32, device=words.device)
    return ((words[:, :, None] >> sh) & 1).to(torch.uint8).reshape(words.shape[0], -1)[:, :bits]


def _bits_to_bytes(b):
    b = b.reshape(-1)
    pad = (-b.numel()) % 8
    if pad:
        b = torch.cat([b, b.new_zeros(pad)])
    w = (b.view(-1, 8).to(torch.int32) << torch.arange(8, device=b.device, dtype=torch.int32)).sum(1)
    return w.to(torch.uint8)


def pack_words(w, bits):
    """w: int64 [nrec, nw] record words (uint32 values) -> int32 tensor holding the sub-array layout of the plane.
    Each piece of the record is stored contiguously over all records; the tail (bits % 16 bits per record) is
    bit-packed across records and followed by a 4-byte pad."""
    b = _to_bits(w, bits)
    parts = [_bits_to_bytes(b[:, o:o + n].contiguous()) for o, n in _pieces(bits)]
    if bits % 16:
        parts.append(torch.zeros(4, dtype=torch.uint8, device=w.device))
    out = torch.cat(parts)
    assert out.numel() % 4 == 0, "record count must keep the plane word-aligned (a multiple of 32 records does)"
    return out.view(torch.int32)


def unpack_words(t, nrec, bits):
    """inverse of pack_words -> int64 [nrec, nw]"""
    by = t.contiguous().view(torch.uint8)
    allbits = ((by[:, None].to(torch.int32) >> torch.arange(8, device=t.device, dtype=torch.int32)) & 1).reshape(-1)
    nw = (bits + 31) // 32
    rec = torch.zeros(nrec, nw * 32, dtype=torch.int64, device=t.device)
    pos = 0
    for o, n in _pieces(bits):
        rec[:, o:o + n] = allbits[pos:pos + nrec * n].view(nrec, n)
        pos += (nrec * n + 7) // 8 * 8
    return (rec.view(nrec, nw, 32) << torch.arange(32, device=t.device)).sum(-1)


_MBN = None


def all_MbN():
    """every valid block word: 1 <= Mb <= 255, 0 <= N <= 255, Mb + N <= 257"""
    global _MBN
    if _MBN is None:
        _MBN = torch.tensor([(m, n) for m in range(1, 256) for n in range(0, min(255, 257 - m) + 1)])
    return _MBN


class Proj:
    """Seeded random packed planes of one N x K projection of one expert.

    base  int32 [S*C*32*4]   one 128-bit record per lane (base code 0); for other base codes the sub-array layout at
                             rbits(bk) bits per record
    p4    int32 view of the residual plane in the sub-array layout (+ 4 B pad when the record has a bit tail)
    d4    int32 [S*R]        block word Mb | N << 8 per refined unit
    var   uint8 [S*C] or None: bit g negates ring g.   flags int64 [S] or None (mask mode, nm flagged chunks/strip)
    mbn   'rand' (Mb in [120,255], N ~ U(0,0.8) Mb, 5 % drawn from the whole valid range) or ('exh', offset) to walk
          every valid block word.
    """

    def __init__(s, N, K, gen, nm=None, rk=0, mbn="rand", var=False, bk=0):
        z = proj_sizes(N, K, nm, rk, bk)
        s.z, s.N, s.K, s.rk, s.bk = z, N, K, rk, bk
        S, C = z["S"], z["C"]
        R = C if nm is None else nm
        dev = gen.device
        if bk == 0:
            s.base = torch.randint(-2**31, 2**31 - 1, (S * C * 32 * 4,), generator=gen, dtype=torch.int32, device=dev)
        else:           # pattern-rate base: rbits(bk) bits per record in the sub-array layout (sm120/NQ_RES_V2.md:36-41)
            bb = rbits(bk)
            wb = torch.randint(0, 2**32, (S * C * 32, (bb + 31) // 32), generator=gen, dtype=torch.int64, device=dev)
            if bb % 32:
                wb[:, -1] &= (1 << (bb % 32)) - 1
            s.base = pack_words(wb.cpu(), bb).to(dev)
        nb = z["p4"]
        raw = torch.randint(0, 256, ((nb + 3) // 4 * 4,), generator=gen, dtype=torch.uint8, device=dev)
        if rbits(rk) % 16:
            raw[nb - 4:] = 0
        s.p4 = raw.view(torch.int32)
        nu = S * R
        if mbn == "rand":
            Mb = torch.randint(120, 256, (nu,), generator=gen, device=dev)
            Nn = (torch.rand(nu, generator=gen, device=dev) * 0.8 * Mb).round().long()
            wild = torch.rand(nu, generator=gen, device=dev) < 0.05
            Mw = torch.randint(1, 256, (nu,), generator=gen, device=dev)
            Nw = (torch.rand(nu, generator=gen, device=dev) * (torch.clamp(257 - Mw, max=255) + 1)).floor().long()
            Mb, Nn = torch.where(wild, Mw, Mb), torch.where(wild, Nw, Nn)
            Nn = torch.minimum(Nn, 257 - Mb)
        else:
            L = all_MbN().to(dev)
            idx = (torch.arange(nu, device=dev) + mbn[1]) % len(L)
            Mb, Nn = L[idx, 0], L[idx, 1]
        s.Mb, s.Nn = Mb, Nn
        s.d4 = (Mb | (Nn << 8)).to(torch.int32)
        s.var = torch.randint(0, 256, (S * C,), generator=gen, dtype=torch.int64, device=dev).to(torch.uint8) if var else None
        if nm is None:
            s.flags = s.fl = None
        else:
            cg = torch.Generator().manual_seed(int(torch.randint(0, 2**31 - 1, (1,), generator=gen, device=dev)))
            s.flags, s.fl = (t.to(dev) for t in make_flags(S, C, nm, cg))

    def to(s, dev):
        for k in ("base", "p4", "d4", "flags", "fl", "Mb", "Nn", "var"):
            v = getattr(s, k)
            if v is not None:
                setattr(s, k, v.to(dev))
        return s

    def nbytes(s, level):
        b = s.base.numel() * 4 + (0 if s.var is None else s.var.numel())
        if level >= 4:
            b += s.z["p4"] + s.d4.numel() * 4 + (0 if s.flags is None else s.flags.numel() * 8)
        return b


def had_dn(ex):
    """width of the down projection's input rotation (128 unless the expert says 512)"""
    return int(getattr(ex, "had_dn", 128) or 128)


class Expert:
    """Seeded synthetic expert: gate|up planes (2I x H), down planes (H x I) and the scale vector
    `signs` = fp16 [H su_g | I sv_g | I sv_u | I su_d | H sv_o | H su_u].  Input scales are +-1 (Hadamard signs);
    output scales are +-1 (sv=None, the reference's synthetic default) or |N(0, sv)|."""

    def __init__(s, H, I, seed, nm_gu=None, nm_dn=None, dev="cuda", rk_gu=0, rk_dn=0, mbn="rand", var=False, sv=None,
                 gen_device="cpu", bk_gu=0, bk_dn=0):
        gen = torch.Generator(device=gen_device).manual_seed(seed)
        s.gu = Proj(2 * I, H, gen, nm_gu, rk_gu, mbn, var, bk_gu).to(dev)
        mbn_dn = mbn if mbn == "rand" else ("exh", mbn[1] + (2 * I // 16) * (H // 128))
        s.dn = Proj(H, I, gen, nm_dn, rk_dn, mbn_dn, var, bk_dn).to(dev)
        sg = (torch.randint(0, 2, (3 * H + 3 * I,), generator=gen, device=gen_device) * 2 - 1).float()
        if sv is not None:
            mag = (torch.randn(3 * H + 3 * I, generator=gen, device=gen_device) * sv).abs()
            out = torch.zeros(3 * H + 3 * I, dtype=torch.bool, device=gen_device)
            out[H:H + 2 * I] = True
            out[H + 3 * I:2 * H + 3 * I] = True
            sg = torch.where(out, mag, sg)
        s.signs = sg.half().to(dev)
        s.H, s.I, s.lr, s.lr4, s.rg, s.rd = H, I, None, None, 0, 0

    def set_lr(s, Vg, U2g, U2u, U4g, U4u, Vd, U2d, U4d):
        """low-rank plane (fp16): Vg [rg,H], U*g/U*u [rg,I], Vd [rd,I], U*d [rd,H]"""
        cat = lambda *t: torch.cat([x.reshape(-1) for x in t]).half().contiguous()
        s.rg, s.rd = Vg.shape[0], Vd.shape[0]
        if s.rg + s.rd == 0:
            s.lr = s.lr4 = None
            return s
        s.lr = cat(Vg, U2g, U2u, Vd, U2d).to(s.signs.device)
        s.lr4 = cat(U4g, U4u, U4d).to(s.signs.device)
        return s

    def bytes(s, level):
        """packed plane bytes a kernel reads for this expert at `level` (scales not included)"""
        return s.gu.nbytes(level) + s.dn.nbytes(level)


def base_code(p):
    return int(getattr(p, "bk", 0) or 0)


def entry(ex, level):
    """device table row (int64 [20]) of an expert at a level.  The field order is the table contract the kernels and the
    serving side share (sm120/nqmoe.cu:26-45, sm120/moe.py:216-229): this function fills the fields in that order."""
    e = torch.zeros(TBL_W, dtype=torch.int64)
    e[0] = level
    for off, p in ((1, ex.gu), (5, ex.dn)):
        for i, k in enumerate(("base", "p4", "d4", "flags")):
            t = getattr(p, k)
            e[off + i] = 0 if t is None else t.data_ptr()
    e[9] = ex.signs.data_ptr()
    e[10], e[11] = ex.gu.rk, ex.dn.rk
    for i, p in ((12, ex.gu), (13, ex.dn)):
        v = getattr(p, "var", None)
        e[i] = 0 if v is None else v.data_ptr()
    if getattr(ex, "lr", None) is not None:
        e[14], e[15], e[16], e[17] = ex.lr.data_ptr(), ex.lr4.data_ptr(), ex.rg, ex.rd
    w = had_dn(ex)
    e[18] = 0 if w == 128 else w
    e[19] = base_code(ex.gu) | base_code(ex.dn) << 8
    return e


class MoELayer:
    """Device table [E, 20] plus the workspaces of the decode path for up to Bmax tokens (Bmax <= 32).

    Rows are flipped in place (`set`, or a Mailbox), which keeps a captured CUDA graph valid."""

    def __init__(s, E, H, I, nm_gu=0, nm_dn=0, Bmax=4, topk=8, G=4, dev="cuda", mod=None, ksplit=None, share=1.0):
        """ksplit: optional (gate|up, down) k-slices per strip to size the workspaces for, when calls will override
        the per-token-count default through cfg_gu / cfg_dn.  share: fraction of the experts resident on this GPU (1 / ranks
        under expert parallelism); it only steers the default k-split."""
        s.M = mod or _ext
        s.E, s.H, s.I, s.nm_gu, s.nm_dn, s.G, s.Bmax, s.topk = E, H, I, nm_gu, nm_dn, G, Bmax, topk
        s.table = torch.zeros(E, TBL_W, dtype=torch.int64, device=dev)
        s.out = torch.zeros(Bmax, H, dtype=torch.float32, device=dev)
        s.hits_ptr = 0      # set to a (host-mapped) int32 [E] pointer to export routing hits
        s.cfg_gu = s.cfg_dn = None     # [k-slices per strip]; None = chosen from the token count of each call
        # workspaces sized for the deepest k-split any call shape can ask for
        s.share = share
        ws = [s.M.moe_workspace(b, topk, H, I, *s.M.default_ksplit(b, H, I, share)) for b in range(1, Bmax + 1)]
        if ksplit is not None:
            ws.append(s.M.moe_workspace(Bmax, topk, H, I, *ksplit))
        n = {k: max(w[k] for w in ws) for k in ws[0]}
        f32, f16, i32 = torch.float32, torch.float16, torch.int32
        s.acc_gu = torch.zeros(n["acc_gu_floats"], dtype=f32, device=dev)
        s.h = torch.zeros(n["h_halves"], dtype=f16, device=dev)
        s.acc_d = torch.zeros(n["acc_d_floats"], dtype=f32, device=dev)
        s.cnt_gu = torch.zeros(n["cnt_gu_ints"], dtype=i32, device=dev)
        s.cnt_d = torch.zeros(n["cnt_d_ints"], dtype=i32, device=dev)
        s.wq = torch.zeros(n["wq_ints"], dtype=i32, device=dev)
        s.zd = torch.zeros(n["zd_floats"], dtype=f32, device=dev)
        s.cnt_h = torch.zeros(n["cnt_h_ints"], dtype=i32, device=dev)

    def set(s, e, ex, level):
        w = had_dn(ex)
        assert w in (128, 512) and s.I % w == 0, f"in_had_down {w} must be 128 or 512 and divide I={s.I}"
        if getattr(ex, "lr", None) is not None:
            assert ex.rg <= 4 and ex.rd <= 4 and ex.lr.dtype == torch.float16
        bks = (base_code(ex.gu), base_code(ex.dn))
        if bks != (0, 0):
            bkm = s.M.bk_codes()
            assert bkm[0] >> bks[0] & 1 and bkm[1] >> bks[1] & 1, f"base K code gu {bks[0]} / dn {bks[1]} not compiled (bk_codes {bkm})"
            if level == 4:      # base code 1 is built with the residual codes it ships with
                for p, name in ((ex.gu, "gu"), (ex.dn, "dn")):
                    assert base_code(p) == 0 or p.rk in (3, 9), f"{name}: base K code {base_code(p)} is built with residual codes 3 and 9, not {p.rk}"
        if level == 4:
            rkm = s.M.rk_codes()
            assert rkm[0] >> ex.gu.rk & 1 and rkm[1] >> ex.dn.rk & 1, f"residual K code gu {ex.gu.rk} / dn {ex.dn.rk} not compiled (rk_codes {rkm})"
        s.table[e].copy_(entry(ex, level).to(s.table.device), non_blocking=False)


    def __call__(s, x, sel, rw, out=None, force_level=0, which=3, cfg_gu=None, cfg_dn=None, table=None, ep=None):
        """x fp16 [B,H], sel int64 [B,topk], rw fp16 [B,topk] -> fp32 [B,H] (s.out[:B] unless `out` is given).
        table: optional [E,20] override of s.table.  ep: see ext.moe_forward.  Enqueued on the current stream; no host sync."""
        assert x.dtype == torch.float16 and rw.dtype == torch.float16 and sel.dtype == torch.int64, (x.dtype, rw.dtype, sel.dtype)
        B = x.shape[0]
        assert B <= s.Bmax and sel.shape[1] == s.topk, f"layer was built for up to {s.Bmax} tokens, top-{s.topk}"
        out = s.out[:B] if out is None else out
        ks = s.M.default_ksplit(B, s.H, s.I, s.share)
        s.M.moe_forward(x, sel, rw, s.table if table is None else table, out, s.acc_gu, s.h, s.acc_d, s.cnt_gu, s.cnt_d,
                        s.wq, s.I, s.nm_gu, s.nm_dn, cfg_gu or s.cfg_gu or [ks[0]], cfg_dn or s.cfg_dn or [ks[1]], s.G,
                        force_level, which, s.hits_ptr, s.zd, s.cnt_h, **({} if ep is None else {"ep": ep}))
        return out


    def status(s):
        """0, or 1 if a device-side wait of a decode-path call ran out (its outputs are then invalid).  Synchronises."""
        return int(s.cnt_h[0].item())

    def capture(s, B, with_mailbox=None, host_io=False, ep=None):
        """Capture one B-token layer call in a CUDA graph over static buffers and return the handle:
        .x [B,H] fp16, .sel [B,topk] int64, .rw [B,topk] fp16, .out [B,H] fp32 (device), .replay().
        with_mailbox: a Mailbox whose apply() is captured in front of the layer.  host_io=True adds pinned host mirrors
        (.x_host, .sel_host, .rw_host, .out_host) and captures the host->device / device->host copies too, so one replay
        is a complete call from host buffers.  ep: see ext.moe_forward (every rank of the group must capture and replay in step)."""
        dev = s.table.device
        g = _Captured()
        # the three inputs live in one buffer (sel | x | rw, each 16-byte aligned) so that a call from host memory is a
        # single host -> device copy
        up = lambda n: (n + 15) // 16 * 16
        o_sel, o_x = 0, up(B * s.topk * 8)
        o_rw = o_x + up(B * s.H * 2)
        nbytes = o_rw + up(B * s.topk * 2)
        g.inputs = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
        view = lambda buf, o, n, dt, shape: buf[o:o + n].view(dt).view(shape)
        g.sel = view(g.inputs, o_sel, B * s.topk * 8, torch.int64, (B, s.topk))
        g.x = view(g.inputs, o_x, B * s.H * 2, torch.float16, (B, s.H))
        g.rw = view(g.inputs, o_rw, B * s.topk * 2, torch.float16, (B, s.topk))
        g.out = torch.zeros(B, s.H, dtype=torch.float32, device=dev)
        if host_io:
            g.inputs_host = torch.zeros(nbytes, dtype=torch.uint8).pin_memory()
            g.sel_host = view(g.inputs_host, o_sel, B * s.topk * 8, torch.int64, (B, s.topk))
            g.x_host = view(g.inputs_host, o_x, B * s.H * 2, torch.float16, (B, s.H))
            g.rw_host = view(g.inputs_host, o_rw, B * s.topk * 2, torch.float16, (B, s.topk))
            g.out_host = g.out.cpu().pin_memory()

        def body():
            if host_io:
                g.inputs.copy_(g.inputs_host, non_blocking=True)
            if with_mailbox is not None:
                with_mailbox.apply()
            s(g.x, g.sel, g.rw, out=g.out, ep=ep)
            if host_io:
                g.out_host.copy_(g.out, non_blocking=True)

        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                body()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        g.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g.graph):
            body()
        return g

    def prefill(s, x, sel, rw, out=None, R=None, G=None, table=None, x_peers=None):
        """T > Bmax tokens: pairs (token, pick) sorted by expert, each routed expert decoded inside the grouped GEMM (tcgen05 /
        TMEM; dense weights never touch HBM), same math as __call__.  x fp16 [T,H], sel int64 [T,topk], rw fp16 [T,topk] ->
        fp32 [T,H].  Same call shape as the reference's prefill (sm120/moe.py:282-327).
        R: pairs per scratch chunk (default 65536 = an 8192-token window of top-8 picks; the scratch, ~45 KB per pair at
        the GLM shape, is allocated once per R and kept).  The expert-sorted pair list is processed chunk by chunk and each
        token's picks are added chunk after chunk in pick order, so the result is bitwise repeatable for a given R.
        G (experts decoded per group in the reference) is accepted and ignored: nothing is decoded ahead of the GEMM.
        Picks whose expert id is outside [0, E) (e.g. -1 padding) are ignored, as on the decode path.
        x_peers = (device addresses of every rank's input buffer, tokens per rank): expert parallelism - x is ignored (pass
        any fp16 [*, H] tensor on the device), token t of sel / rw is read from buffer t // tokens_per_rank by the first pass
        itself (see nq_pf_pre_ep).
        Nothing here synchronises with the host; a device-side time-out inside the GEMM raises a flag that
        prefill_status() reads."""
        assert x.dtype == torch.float16 and rw.dtype == torch.float16 and sel.dtype == torch.int64, (x.dtype, rw.dtype, sel.dtype)
        T, k = sel.shape
        H, I, E, M, dev = s.H, s.I, s.E, s.M, sel.device
        tb = s.table if table is None else table
        P = T * k
        R = max(1, min(R or 65536, P))
        out = torch.empty(T, H, dtype=torch.float32, device=dev) if out is None else out
        if P == 0:
            return out
        sc = s._prefill_scratch(R, dev)
        # pairs sorted by expert on the device: pe / pt of each sorted pair, pos of each pick, first pair of each expert.  Picks
        # that contribute nothing (no valid expert id, expert not resident here, zero weight) sort behind every real pair.
        sel, rw = sel.contiguous(), rw.contiguous()
        perm = s._prefill_perm(P, dev)
        pe, pt, pos = perm["pe"][:P], perm["pt"][:P], perm["pos"][:P]
        hit = None
        if s.hits_ptr:
            hit = perm["hit"].zero_()
        M.pf_sort(sel, rw, tb, pe, pt, pos, perm["start"], hit, perm["scratch"])
        if s.hits_ptr:
            M.pf_hits(hit, s.hits_ptr)
        for c0 in range(0, P, R):
            n = min(R, P - c0)
            M.pf_plan_window(perm["start"], tb, sc["plan"], c0, n)       # pass list of this chunk, built on the device
            xg, xu, y = sc["xg"][:n], sc["xu"][:n], sc["y"][:n]
            if x_peers is None:
                M.pf_pre(x, pt[c0:c0 + n], pe[c0:c0 + n], tb, xg, xu, sc["zg"], I, kperm=True)
            else:
                M.pf_pre_ep(x_peers[0], x_peers[1], H, pt[c0:c0 + n], pe[c0:c0 + n], tb, xg, xu, sc["zg"], I, kperm=True)
            M.pf_gemm(tb, sc["plan"], xg, xu, sc["acc_g"], sc["acc_u"], H, I, s.nm_gu, s.nm_dn, False, sc["status"])
            M.pf_mid(sc["acc_g"], sc["acc_u"], sc["zg"], pe[c0:c0 + n], tb, sc["h"], sc["zd"], H, I, kperm=True)
            M.pf_gemm(tb, sc["plan"], sc["h"][:n], None, y, None, H, I, s.nm_gu, s.nm_dn, True, sc["status"])     # y overwrites xg | xu
            M.pf_combine(y, sc["zd"], pos, sel, rw, tb, out, I, pair0=c0, npairs=n, accumulate=c0 > 0)
        return out

    def _prefill_scratch(s, R, dev):
        """scratch of the prefill path for chunks of R pairs, kept between calls (the reference's pf_scratch,
        sm120/moe.py:263-275, without its dense weight buffers): xg | xu fp16 [R,H] each, aliased by y fp32 [R,H];
        acc_g, acc_u fp32 [R,I]; h fp16 [R,I]; zg, zd fp32 [R,4]; the pass list; the status word"""
        owner = getattr(s, "_pf_owner", None)
        if owner is not None:
            return owner._prefill_scratch(R, dev)
        sc = getattr(s, "_pf_sc", None)
        if sc is not None and sc["R"] == R and sc["y"].device == dev:
            return sc
        H, I, E = s.H, s.I, s.E
        f16, f32, i32 = torch.float16, torch.float32, torch.int32
        y = torch.empty(R, H, dtype=f32, device=dev)
        halves = y.view(-1).view(f16)
        status = sc["status"] if sc is not None and sc["status"].device == dev else torch.zeros(1, dtype=i32, device=dev)
        s._pf_sc = dict(R=R, y=y, xg=halves[:R * H].view(R, H), xu=halves[R * H:].view(R, H),
                        acc_g=torch.empty(R, I, dtype=f32, device=dev), acc_u=torch.empty(R, I, dtype=f32, device=dev),
                        h=torch.empty(R, I, dtype=f16, device=dev), zg=torch.zeros(R, 4, dtype=f32, device=dev),
                        zd=torch.zeros(R, 4, dtype=f32, device=dev),
                        plan=torch.empty(s.M.pf_plan_ints(E, R), dtype=i32, device=dev), status=status)
        return s._pf_sc

    def _prefill_perm(s, P, dev):
        """index arrays of the pair sort for windows of up to P pairs, kept between calls"""
        owner = getattr(s, "_pf_owner", None)
        if owner is not None:
            return owner._prefill_perm(P, dev)
        pm = getattr(s, "_pf_perm", None)
        if pm is not None and pm["P"] >= P and pm["pe"].device == dev:
            return pm
        i32 = torch.int32
        mk = lambda n: torch.empty(n, dtype=i32, device=dev)
        s._pf_perm = dict(P=P, pe=mk(P), pt=mk(P), pos=mk(P), start=mk(s.E + 2), hit=mk(s.E), scratch=mk(max(1, s.M.pf_sort_scratch_ints(P, s.E))))
        return s._pf_perm

    def share_prefill_scratch(s, other):
        """use the prefill scratch (and status word) of another layer of the same shape: the layers of a stack run one after
        the other on one stream, so one set of buffers serves them all"""
        assert (other.H, other.I, other.E) == (s.H, s.I, s.E)
        s._pf_owner = other

    def prefill_status(s):
        """0, or 1 if a device-side wait inside the prefill GEMM has run out since the layer was built (results of that call are
        invalid).  Synchronises with the device."""
        owner = getattr(s, "_pf_owner", None)
        if owner is not None:
            return owner.prefill_status()
        sc = getattr(s, "_pf_sc", None)
        return 0 if sc is None else int(sc["status"].item())


class _Captured:
    """static buffers + CUDA graph of one captured layer call (MoELayer.capture)"""

    def replay(s):
        s.graph.replay()
        return s.out


class Mailbox:
    """Graph-safe table updates: call .apply() inside the captured graph before the layer; stage rows from a side stream.
    Same protocol and attribute names as the reference's Mailbox (sm120/moe.py:329-342): stage / seq / applied /
    applied_host are the objects its executor writes and polls."""

    def __init__(s, layer):
        E, dev = layer.E, layer.table.device
        s.L = layer
        s.stage = torch.zeros(E, TBL_W, dtype=torch.int64, device=dev)
        s.seq = torch.zeros(E, dtype=torch.int32, device=dev)
        s.applied = torch.zeros(E, dtype=torch.int32, device=dev)
        s.applied_host = torch.zeros(E, dtype=torch.int32).pin_memory()
        s.hseq = [0] * E
        s.pins = []

    def apply(s):
        s.L.M.mailbox(s.L.table, s.stage, s.seq, s.applied, s.applied_host.data_ptr())

    def post(s, e, row, stream):
        """enqueue on `stream` (after any plane copy already enqueued there): stage[e] = row; seq[e] += 1"""
        assert s.done(e), "one outstanding op per expert"
        s.hseq[e] += 1
        r = row.pin_memory()
        q = torch.tensor([s.hseq[e]], dtype=torch.int32).pin_memory()
        s.pins += [r, q]
        with torch.cuda.stream(stream):
            s.stage[e].copy_(r, non_blocking=True)
            s.seq[e:e + 1].copy_(q, non_blocking=True)

    def done(s, e):
        return int(s.applied_host[e]) == s.hseq[e]
