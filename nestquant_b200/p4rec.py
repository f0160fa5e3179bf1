"""Residual-plane records and the slot pool they are promoted into.

A record holds what an expert needs on top of its resident base to run at level 4: segments
gu.p4 | gu.d4 | dn.p4 | dn.d4 | lr4, each 256-byte aligned, the whole record rounded up to 4 KiB - the byte contract of the
reference's streaming/p4rec.py:13-37 (`layout`, `pack`, `row`), so records written by its repack tool land in these
slots unchanged.  `SlotPool` is the device side: nslot x rec_bytes bytes plus the promote / demote calls that put a
record and its table row in flight on a side stream (streaming/nqstream.cu:183-191, streaming/executor.py:62-93 keep
the policy; this is only the data movement).
"""
import torch

from . import capi
from .capi import check, lib

SEG_ALIGN, ALIGN, RMAX = 256, 4096, 4
SEGS = ("gu.p4", "gu.d4", "dn.p4", "dn.d4", "lr4")


def _up(n, a):
    return (n + a - 1) // a * a


def layout(ex, H, I):
    """segment (offset, bytes) table and record size for the experts of a layer (sizes depend only on shapes and codes).
    A byte contract with the reference's record files: segment order, the 256-byte segment alignment and the 4 KiB record
    alignment are those of streaming/p4rec.py:13-26, so this function walks the segments in the schema's order."""
    n = {"gu.p4": ex.gu.p4.numel() * 4, "gu.d4": ex.gu.d4.numel() * 4, "dn.p4": ex.dn.p4.numel() * 4,
         "dn.d4": ex.dn.d4.numel() * 4, "lr4": RMAX * (2 * I + H) * 2}
    seg, o = {}, 0
    for k in SEGS:
        seg[k] = (o, n[k])
        o = _up(o + n[k], SEG_ALIGN)
    return dict(seg=seg, rec_bytes=_up(o, ALIGN))


def _tensors(ex):
    lr4 = ex.lr4 if getattr(ex, "lr4", None) is not None else torch.zeros(0, dtype=torch.float16)
    return {"gu.p4": ex.gu.p4, "gu.d4": ex.gu.d4, "dn.p4": ex.dn.p4, "dn.d4": ex.dn.d4, "lr4": lr4}


def pack(ex, lay, pin=True):
    """record of one expert as a (pinned) uint8 host tensor of lay['rec_bytes']"""
    rec = torch.zeros(lay["rec_bytes"], dtype=torch.uint8)
    for k, t in _tensors(ex).items():
        o, n = lay["seg"][k]
        raw = t.detach().contiguous().cpu().view(torch.uint8).reshape(-1)
        assert raw.numel() <= n, (k, raw.numel(), n)
        rec[o:o + raw.numel()] = raw
    return rec.pin_memory() if pin else rec


def row(ex, lay, slot_ptr, entry):
    """level-4 table row whose residual pointers point into a slot holding the expert's record; the resident planes
    (base, signs, scales, low-rank base part) stay where they are.  entry = nestquant_b200.moe.entry.  Which table fields are
    patched, and with which segment, is the reference's schema (streaming/p4rec.py:29-37)."""
    r = entry(ex, 4)
    s = lay["seg"]
    r[2], r[3], r[6], r[7] = (slot_ptr + s[k][0] for k in ("gu.p4", "gu.d4", "dn.p4", "dn.d4"))
    if getattr(ex, "rg", 0) + getattr(ex, "rd", 0):
        r[15] = slot_ptr + s["lr4"][0]
    if hasattr(ex, "sc"):
        r[9] = ex.sc[4].data_ptr()       # level-4 scale vectors of a loaded resident file (nestquant_b200/resident.py)
    return r


class SlotPool:
    """nslot slots of rec_bytes on the device; promotions copy a pinned record into a free slot and stage the row."""

    def __init__(s, nslot, rec_bytes, dev="cuda"):
        s.nslot, s.rec_bytes = nslot, rec_bytes
        s.buf = torch.zeros(nslot, rec_bytes, dtype=torch.uint8, device=dev)
        s.free = list(range(nslot))
        s.slot_of = {}
        s._keep = []          # pinned rows / sequence numbers in flight

    def slot_ptr(s, i):
        return s.buf[i].data_ptr()

    def promote(s, mailbox, e, ex, lay, record, entry, stream):
        """enqueue on `stream`: record -> free slot, level-4 row -> stage[e], seq[e] += 1.  Returns the slot index."""
        assert mailbox.done(e), "one outstanding op per expert"
        assert e not in s.slot_of and s.free, "expert already promoted or no free slot"
        assert record.is_pinned() and record.numel() == s.rec_bytes
        i = s.free.pop()
        s.slot_of[e] = i
        s._post(mailbox, e, row(ex, lay, s.slot_ptr(i), entry), stream, s.buf[i], record)
        return i

    def demote(s, mailbox, e, ex, entry, stream):
        """enqueue the level-2 row; the slot may be reused once mailbox.done(e) (the row switch has been applied)"""
        assert mailbox.done(e), "one outstanding op per expert"
        s._post(mailbox, e, entry(ex, 2), stream, None, None)

    def release(s, e):
        """after a demotion has been applied: return the expert's slot to the free list"""
        s.free.append(s.slot_of.pop(e))

    def _post(s, mailbox, e, r, stream, slot, record):
        mailbox.hseq[e] += 1
        hrow = r.to(torch.int64).pin_memory()
        hseq = torch.tensor([mailbox.hseq[e]], dtype=torch.int32).pin_memory()
        s._keep = s._keep[-64:] + [hrow, hseq, record]
        check(lib().nq_promote(None if slot is None else slot.data_ptr(), None if record is None else record.data_ptr(),
                               0 if record is None else record.numel(), mailbox.stage[e].data_ptr(), hrow.data_ptr(),
                               mailbox.seq[e:e + 1].data_ptr(), hseq.data_ptr(), stream.cuda_stream), "promote")
