"""Promotion engine: reads fixed-size expert records from the rank's record file and puts them, their table rows and
sequence numbers in flight on a side stream.

Python face of the C-ABI engine in csrc/nq_engine.cu, with the call shape of the reference's torch-extension class
(streaming/nqstream.cu:8-25, used by streaming/executor.py):

    e = Engine(path, rec_bytes, n_host, qd, device, alt_path="", qd_alt=0)
    e.upgrade(tag, rec_index, slot_ptr, stage_ptr, row, seq_ptr, seq)     # queued, returns at once
    e.post(tag, stage_ptr, row, seq_ptr, seq)                             # demotion / row-only operation
    e.poll() -> [(tag, hit, t_read_s, t_e2e_s)]
    e.cancel(tag); e.tier_load(recs) -> n; e.tier_drop(); e.stats() -> dict; e.close()

device < 0 runs against host memory (pointers are then host addresses), which is how the CPU tests drive it.
`write_records` makes a record file from packed records (nestquant_b200.p4rec.pack).
"""
import ctypes as C

from . import capi
from .capi import check, lib


def _row20(row):
    vals = [int(v) for v in (row.tolist() if hasattr(row, "tolist") else row)]
    assert len(vals) == capi.TABLE_WIDTH, "row: 20 int64 values"
    return (C.c_int64 * capi.TABLE_WIDTH)(*vals)


class Engine:
    def __init__(s, path, rec_bytes, n_host, qd, device, alt_path="", qd_alt=0):
        h = C.c_void_p()
        check(lib().nq_engine_open(str(path).encode(), (alt_path or "").encode(), int(rec_bytes), int(n_host), int(qd), int(qd_alt),
                                   int(device), C.byref(h)), "engine open")
        s._h, s.rec_bytes = h, int(rec_bytes)

    def upgrade(s, tag, rec, slot_ptr, stage_ptr, row, seq_ptr, seq):
        check(lib().nq_engine_upgrade(s._h, int(tag), int(rec), C.c_void_p(int(slot_ptr)), C.c_void_p(int(stage_ptr)), _row20(row),
                                      C.c_void_p(int(seq_ptr)), int(seq)), "engine upgrade")

    def post(s, tag, stage_ptr, row, seq_ptr, seq):
        check(lib().nq_engine_post(s._h, int(tag), C.c_void_p(int(stage_ptr)), _row20(row), C.c_void_p(int(seq_ptr)), int(seq)), "engine post")

    def cancel(s, tag):
        check(lib().nq_engine_cancel(s._h, int(tag)), "engine cancel")

    def poll(s, max_ops=256):
        buf = (capi.NqEngineDone * max_ops)()
        n = lib().nq_engine_poll(s._h, buf, max_ops)
        if n < 0:
            check(n, "engine poll")
        return [(int(d.tag), bool(d.hit), float(d.t_read_s), float(d.t_done_s)) for d in buf[:n]]

    def tier_load(s, recs):
        recs = [int(r) for r in recs]
        arr = (C.c_int64 * max(1, len(recs)))(*recs)
        n = lib().nq_engine_tier_load(s._h, arr, len(recs))
        if n < 0:
            check(n, "engine tier_load")
        return n

    def tier_drop(s):
        check(lib().nq_engine_tier_drop(s._h), "engine tier_drop")

    def stats(s):
        st = capi.NqEngineStats()
        check(lib().nq_engine_stats(s._h, C.byref(st)), "engine stats")
        d = {}
        for name, _ in capi.NqEngineStats._fields_:
            v = getattr(st, name)
            d[name] = list(v) if hasattr(v, "__len__") else v
        nd = int(st.drives)
        for k in ("drive_reads", "drive_bytes", "drive_inflight", "drive_qd", "drive_read_s"):
            d[k] = d[k][:nd]
        d["now"] = d.pop("now_s")
        return d

    def close(s):
        if s._h is not None:
            lib().nq_engine_close(s._h)
            s._h = None

    def __del__(s):
        try:
            s.close()
        except Exception:
            pass


def write_records(path, records):
    """record file = the packed records back to back (record i at byte i * rec_bytes)"""
    with open(path, "wb") as f:
        for r in records:
            f.write(bytes(r.cpu().numpy().tobytes()) if hasattr(r, "cpu") else bytes(r))
