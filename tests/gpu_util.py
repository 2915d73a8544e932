"""Helpers shared by the GPU parity tests: device buffers via torch, calls via the C ABI."""
import ctypes as C

import numpy as np
import torch

from lightseq_b200 import _lib as L

_ctx = None


def ctx():
    global _ctx
    if _ctx is None:
        _ctx = L.Context(0)
    return _ctx


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).to("cuda:0")


def empty(shape, dtype) -> torch.Tensor:
    return torch.empty(shape, dtype=dtype, device="cuda:0")


def ptr(t):
    return None if t is None else t.data_ptr()


def sync_check():
    torch.cuda.synchronize()
    assert ctx().poll_error() == 0, "device-side bounded wait reported a timeout"


def gemm(a_q, w_q, *, s_acc, out_kind, s_outq=0.0, bias=None, act=L.ACT_NONE, resid=None, s_req=0.0, w_off=None,
         out_dtype=None, ln=None, in_place=False, table=False):
    """a_q [M,K] int8 device, w_q [N,K] int8 device -> device tensor. table: tabulate bias / activation /
    requantisation first (ls100_gemm_i8_build_table) and pass the table."""
    m, k = a_q.shape
    n = w_q.shape[0]
    dt = {L.OUT_OUTQ_I8: torch.int8, L.OUT_F32: torch.float32, L.OUT_REQ_S8: torch.int8, L.OUT_REQ_U8: torch.int8,
          L.OUT_F16: torch.float16, L.OUT_I32: torch.int32}[out_kind]
    out = resid if in_place else torch.full((m, n), 0, dtype=dt, device="cuda:0")  # in_place: the residual buffer is the output
    args = L.GemmI8Args(a=ptr(a_q), lda=a_q.stride(0), w=ptr(w_q), ldw=w_q.stride(0), m=m, n=n, k=k, s_acc=s_acc,
                        w_off=ptr(w_off), s_outq=s_outq, bias=ptr(bias), act=act, resid=ptr(resid),
                        ldr=(resid.stride(0) if resid is not None else 0), out_kind=out_kind, s_req=s_req,
                        out=ptr(out), ldo=n)
    if table:
        tab = torch.empty(L.lib.ls100_gemm_i8_table_bytes(n), dtype=torch.uint8, device="cuda:0")
        L.check(L.lib.ls100_gemm_i8_build_table(ctx().handle, L.C.byref(args), L.C.c_void_p(ptr(tab)), None),
                "ls100_gemm_i8_build_table")
        args.req_table = ptr(tab)
    if ln is not None:  # (gamma, beta, amax): fused LayerNorm + quantise, returns (out, ln_out)
        ln_out = torch.full((m, n), 0, dtype=torch.int8, device="cuda:0")
        args.ln_gamma, args.ln_beta, args.ln_amax, args.ln_out, args.ln_ldq = ptr(ln[0]), ptr(ln[1]), ln[2], ptr(ln_out), n
        L.call("ls100_gemm_i8", ctx(), args)
        return out, ln_out
    L.call("ls100_gemm_i8", ctx(), args)
    return out
