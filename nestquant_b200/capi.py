"""ctypes binding of the C ABI declared in include/nestquant_b200.h.

The library is built in-tree by `python -m nestquant_b200.build`.  There is no fallback: if the shared object is
missing or fails to load, importing a symbol from here raises, and every compute entry point needs a CUDA device.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libnestquant_b200.so")

NQ_OK, NQ_ERR_ARG, NQ_ERR_CUDA, NQ_ERR_UNSUPPORTED = 0, -1, -2, -3
TABLE_WIDTH = 20
MAX_TOKENS = 32
MAX_PICKS = 256

_p, _i, _i64, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_size_t



class NqMoeWorkspace(C.Structure):
    _fields_ = [(n, _sz) for n in ("acc_gu_floats", "h_halves", "acc_d_floats", "cnt_gu_ints", "cnt_d_ints", "wq_ints",
                                   "zd_floats", "cnt_h_ints")]


class NqMoeForward(C.Structure):
    _fields_ = ([(n, _p) for n in ("x", "sel", "rw", "table", "out", "acc_gu", "h", "acc_d", "cnt_gu", "cnt_d", "wq", "zd",
                                   "cnt_h", "hits")] +
                [(n, _sz) for n in ("out_floats", "acc_gu_floats", "h_halves", "acc_d_floats", "cnt_gu_ints", "cnt_d_ints",
                                    "wq_ints", "zd_floats", "cnt_h_ints")] +
                [(n, _i) for n in ("B", "topk", "E", "H", "I", "nm_gu", "nm_dn", "ks_gu", "ks_dn", "G", "force_level",
                                   "which")])


class NqMoeEp(C.Structure):
    _fields_ = [("world", _i), ("rank", _i), ("peer_recv", C.POINTER(_p)), ("peer_counters", C.POINTER(_p)), ("epoch", _p)]


class NqEngineDone(C.Structure):
    _fields_ = [("tag", _i64), ("hit", C.c_int32), ("t_read_s", C.c_double), ("t_done_s", C.c_double)]


class NqEngineStats(C.Structure):
    _fields_ = ([(n, _i64) for n in ("upgrades", "posts", "host_hits", "bytes_read", "fault_injected", "cancelled",
                                     "device_errors", "queued", "waiting", "reading", "copying")] +
                [(n, _i64 * 2) for n in ("drive_reads", "drive_bytes", "drive_inflight", "drive_qd")] +
                [("drive_read_s", C.c_double * 2)] +
                [(n, _i64) for n in ("drives", "n_host", "tier_state", "tier_recs", "tier_hits", "tier_bytes")] +
                [("now_s", C.c_double)])


# name -> (restype, argtypes); mirrors include/nestquant_b200.h one to one
SIGNATURES = {
    "nq_last_error": (C.c_char_p, []),
    "nq_build_arch": (_i, []),
    "nq_rk_codes": (_i, [C.POINTER(_i64)]),
    "nq_bk_codes": (_i, [C.POINTER(_i64)]),
    "nq_plane_bytes": (_sz, [_sz, _i]),
    "nq_pf_decode": (_i, [_p, _p, _i, _p, _p, _i, _i, _i, _i, _i, _p]),
    "nq_mailbox": (_i, [_p, _p, _p, _p, _p, _i, _p]),
    "nq_promote": (_i, [_p, _p, _sz, _p, _p, _p, _p, _p]),
    "nq_pf_pre": (_i, [_p, _p, _p, _i, _p, _i, _p, _p, _p, _i, _i, _i, _p]),
    "nq_pf_pre_ep": (_i, [C.POINTER(_p), _i, _i, _p, _p, _i, _p, _i, _p, _p, _p, _i, _i, _i, _p]),
    "nq_pf_mid": (_i, [_p, _p, _p, _p, _i, _p, _i, _p, _p, _i, _i, _i, _p]),
    "nq_pf_post": (_i, [_p, _p, _p, _p, _p, _i, _p, _i, _p, _i, _i, _p]),
    "nq_pf_combine": (_i, [_p, _p, _p, _p, _p, _i, _i, _p, _i, _p, _i, _i, _i, _i, _i, _p]),
    "nq_pf_hits": (_i, [_p, _p, _i, _p]),
    "nq_pf_sort_scratch_ints": (_i, [_i, _i]),
    "nq_pf_sort": (_i, [_p, _p, _p, _i, _i, _i, _p, _p, _p, _p, _p, _p, _i, _p]),
    "nq_pf_plan_window": (_i, [_p, _p, _i, _i, _i, _p, _i, _p]),
    "nq_pf_plan_ints": (_i, [_i, _i]),
    "nq_pf_plan": (_i, [_p, _p, _i, _i, _p, _i, _p]),
    "nq_pf_gemm": (_i, [_p, _p, _p, _p, _i, _p, _p, _i, _i, _i, _i, _i, _p, _p]),
    "nq_moe_workspace": (_i, [_i, _i, _i, _i, _i, _i, C.POINTER(NqMoeWorkspace)]),
    "nq_moe_forward": (_i, [C.POINTER(NqMoeForward), _p]),
    "nq_moe_forward_ep": (_i, [C.POINTER(NqMoeForward), C.POINTER(NqMoeEp), _p]),
    "nq_moe_ep_recv_floats": (_sz, [_i, _i]),
    "nq_moe_ep_counter_ints": (_sz, []),
    "nq_moe_static_scratch_bytes": (_sz, []),
    "nq_moe_forward_static": (_i, [_p, _p, _p, _p, _p] + [_i] * 9 + [_p, _p]),
    "nq_salience": (_i, [_p, _i, _i64, _p, _p, _i, _i, _i, _i, C.c_float, _p, _p, _p]),
    "nq_ep_barrier": (_i, [C.POINTER(_p), _i, _i, _p, _p, C.c_longlong, _p]),
    "nq_ep_picks": (_i, [C.POINTER(_p), C.POINTER(_p), _i, _i, _i, _i, _i, _p, _p, _p]),
    "nq_ep_gather": (_i, [_p, C.POINTER(_p), _p, _p, _i, _i, _i, _i, _i, _i, _p]),
    "nq_ep_combine": (_i, [_p, C.POINTER(_p), _p, _i, _i, _i, _p]),
    "nq_engine_open": (_i, [C.c_char_p, C.c_char_p, _sz, _i, _i, _i, _i, C.POINTER(_p)]),
    "nq_engine_upgrade": (_i, [_p, _i64, _i64, _p, _p, C.POINTER(_i64), _p, C.c_int32]),
    "nq_engine_post": (_i, [_p, _i64, _p, C.POINTER(_i64), _p, C.c_int32]),
    "nq_engine_cancel": (_i, [_p, _i64]),
    "nq_engine_poll": (_i, [_p, C.POINTER(NqEngineDone), _i]),
    "nq_engine_tier_load": (_i, [_p, C.POINTER(_i64), _i]),
    "nq_engine_tier_drop": (_i, [_p]),
    "nq_engine_stats": (_i, [_p, C.POINTER(NqEngineStats)]),
    "nq_engine_close": (_i, [_p]),
}

_lib = None


class NestQuantError(RuntimeError):
    pass


def lib():
    """The loaded shared library (loads on first use; raises if it has not been built)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise NestQuantError(f"{LIB_PATH} is missing: run `python -m nestquant_b200.build` (needs nvcc); "
                                 "there is no CPU or PyTorch fallback for this path")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            f = getattr(L, name)        # AttributeError here = header and library out of sync
            f.restype, f.argtypes = res, args
        _lib = L
    return _lib


def check(rc, what=""):
    if rc != NQ_OK:
        msg = lib().nq_last_error()
        raise NestQuantError(f"{what or 'nestquant_b200'} failed ({rc}): {msg.decode() if msg else ''}")


def ptr(t):
    """data pointer of a torch tensor (or None / int passthrough)"""
    if t is None:
        return None
    if isinstance(t, int):
        return t or None
    return t.data_ptr()


def current_stream():
    import torch
    return torch.cuda.current_stream().cuda_stream
