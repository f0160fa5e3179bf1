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
