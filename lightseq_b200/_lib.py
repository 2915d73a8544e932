"""ctypes binding of ``libls100.so`` (the C ABI declared in ``include/ls100.h``).

The library is required: importing this module raises if it has not been built
(``python -m lightseq_b200.build``); there is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libls100.so"

if not LIB_PATH.exists():
    raise ImportError(
        f"{LIB_PATH} is missing: build the CUDA library first with `python -m lightseq_b200.build` "
        "(lightseq_b200 has no fallback path)"
    )

lib = C.CDLL(str(LIB_PATH), mode=C.RTLD_GLOBAL)

OK = 0
ERR_BAD_ARG, ERR_ALIGN, ERR_UNSUPPORTED, ERR_CUDA, ERR_TIMEOUT, ERR_NO_DRIVER = -1, -2, -3, -4, -5, -6

OUT_OUTQ_I8, OUT_F32, OUT_REQ_S8, OUT_REQ_U8, OUT_F16, OUT_I32 = range(6)
ACT_NONE, ACT_RELU, ACT_GELU = range(3)


class Ls100Error(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        msg = lib.ls100_strerror(code)
        super().__init__(f"{where}: {msg.decode() if msg else code} ({code})")


def check(code: int, where: str) -> None:
    if code != 0:
        raise Ls100Error(code, where)


class GemmI8Args(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("lda", C.c_int64),
        ("w", C.c_void_p), ("ldw", C.c_int64),
        ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
        ("s_acc", C.c_float),
        ("w_off", C.c_void_p),
        ("s_outq", C.c_float),
        ("bias", C.c_void_p),
        ("act", C.c_int32),
        ("resid", C.c_void_p), ("ldr", C.c_int64),
        ("out_kind", C.c_int32),
        ("s_req", C.c_float),
        ("out", C.c_void_p), ("ldo", C.c_int64),
        ("ln_gamma", C.c_void_p), ("ln_beta", C.c_void_p), ("ln_amax", C.c_float), ("ln_out", C.c_void_p),
        ("ln_ldq", C.c_int64),
        ("stat_max", C.c_void_p), ("stat_sum", C.c_void_p),
        ("req_table", C.c_void_p),
    ]



class EmbedArgs(C.Structure):
    _fields_ = [("ids", C.c_void_p), ("ld_ids", C.c_int64), ("batch", C.c_int32), ("seq", C.c_int32),
                ("hidden", C.c_int32), ("step_ptr", C.c_void_p), ("table_q", C.c_void_p), ("s_emb", C.c_float),
                ("sqrt_h", C.c_float), ("pos", C.c_void_p), ("n_pos", C.c_int32), ("pad_id", C.c_int32),
                ("vocab", C.c_int32), ("out", C.c_void_p), ("pad_mask", C.c_void_p), ("pos_mode", C.c_int32)]


class LnQuantArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("ldx", C.c_int64), ("gamma", C.c_void_p), ("beta", C.c_void_p),
                ("rows", C.c_int32), ("hidden", C.c_int32), ("amax", C.c_float),
                ("out_q", C.c_void_p), ("ldq", C.c_int64), ("out_f", C.c_void_p), ("ldf", C.c_int64),
                ("emb", EmbedArgs)]  # optional: rows looked up instead of read (decode-step form)


class PatchEmbedArgs(C.Structure):
    _fields_ = [("pixels", C.c_void_p), ("conv_wt", C.c_void_p), ("conv_bias", C.c_void_p), ("pos", C.c_void_p),
                ("cls", C.c_void_p), ("batch", C.c_int32), ("channels", C.c_int32), ("image", C.c_int32),
                ("patch", C.c_int32), ("hidden", C.c_int32), ("out", C.c_void_p)]


class AttnSelfArgs(C.Structure):
    _fields_ = [("qkv", C.c_void_p), ("ld_qkv", C.c_int64), ("s_qkv", C.c_float), ("bias", C.c_void_p),
                ("pad_mask", C.c_void_p), ("batch", C.c_int32), ("seq", C.c_int32), ("heads", C.c_int32),
                ("causal", C.c_int32), ("amax_out", C.c_float), ("out", C.c_void_p), ("ld_out", C.c_int64),
                ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("max_step", C.c_int32)]


class AttnDecArgs(C.Structure):
    _fields_ = [("qkv", C.c_void_p), ("ld_qkv", C.c_int64), ("s_kv", C.c_float), ("k_cache", C.c_void_p),
                ("v_cache", C.c_void_p), ("anc", C.c_void_p), ("step_ptr", C.c_void_p), ("rows", C.c_int32),
                ("heads", C.c_int32), ("max_step", C.c_int32), ("amax_out", C.c_float), ("out", C.c_void_p),
                ("ld_out", C.c_int64), ("history_static", C.c_int32)]


class AttnCrossArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("ld_q", C.c_int64), ("s_q", C.c_float), ("bias", C.c_void_p),
                ("k", C.c_void_p), ("v", C.c_void_p), ("ld_kv", C.c_int64), ("pad_mask", C.c_void_p),
                ("batch", C.c_int32), ("beam", C.c_int32), ("src_len", C.c_int32), ("heads", C.c_int32),
                ("amax_out", C.c_float), ("out", C.c_void_p), ("ld_out", C.c_int64), ("kv_static", C.c_int32),
                ("kv_head_major", C.c_int32)]


class ProjF32Args(C.Structure):
    _fields_ = [("x", C.c_void_p), ("ldx", C.c_int64), ("w", C.c_void_p), ("ldw", C.c_int64), ("s_w", C.c_float),
                ("bias", C.c_void_p), ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("out", C.c_void_p),
                ("ldo", C.c_int64), ("split_seq", C.c_int32)]


class BeamTopkArgs(C.Structure):
    _fields_ = [("logits", C.c_void_p), ("ld_logits", C.c_int64), ("s_logits", C.c_float), ("batch", C.c_int32),
                ("beam", C.c_int32), ("vocab", C.c_int32), ("max_step", C.c_int32), ("end_id", C.c_int32),
                ("step_ptr", C.c_void_p), ("length_norm", C.c_void_p), ("alive", C.c_void_p),
                ("seq_probs", C.c_void_p), ("seq_score", C.c_void_p), ("cand_score", C.c_void_p),
                ("cand_token", C.c_void_p), ("diverse_lambda", C.c_float)]


class BeamSelectArgs(C.Structure):
    _fields_ = [("topk", BeamTopkArgs), ("stat_max", C.c_void_p), ("stat_sum", C.c_void_p), ("n_groups", C.c_int32)]


class BeamUpdateArgs(C.Structure):
    _fields_ = [("cand_score", C.c_void_p), ("cand_token", C.c_void_p), ("batch", C.c_int32), ("beam", C.c_int32),
                ("max_step", C.c_int32), ("end_id", C.c_int32), ("step_ptr", C.c_void_p),
                ("length_norm", C.c_void_p), ("alive", C.c_void_p), ("anc", C.c_void_p), ("seq_probs", C.c_void_p),
                ("seq_score", C.c_void_p), ("fin_count", C.c_void_p), ("ticket", C.c_void_p),
                ("stop_step", C.c_void_p), ("stop_host", C.c_void_p), ("diverse_lambda", C.c_float)]


class SampleTopkArgs(C.Structure):
    _fields_ = [("logits", C.c_void_p), ("ld_logits", C.c_int64), ("s_logits", C.c_float), ("rows", C.c_int32),
                ("vocab", C.c_int32), ("k", C.c_int32), ("max_step", C.c_int32), ("end_id", C.c_int32),
                ("seed_lo", C.c_uint32), ("seed_hi", C.c_uint32), ("seq", C.c_void_p), ("cur", C.c_void_p),
                ("ticket", C.c_void_p), ("n_ended", C.c_void_p), ("stop", C.c_void_p), ("stop_host", C.c_void_p)]


class ProjTcArgs(C.Structure):
    _fields_ = [("x3", C.c_void_p), ("w_bf16", C.c_void_p), ("s_w", C.c_float), ("bias", C.c_void_p), ("m", C.c_int32),
                ("n", C.c_int32), ("k", C.c_int32), ("out", C.c_void_p), ("ldo", C.c_int64), ("split_seq", C.c_int32)]


class BeamResultArgs(C.Structure):
    _fields_ = [("alive", C.c_void_p), ("seq_score", C.c_void_p), ("batch", C.c_int32), ("beam", C.c_int32),
                ("max_step", C.c_int32), ("end_id", C.c_int32), ("n_out", C.c_int32), ("mode", C.c_int32),
                ("out_tokens", C.c_void_p), ("out_scores", C.c_void_p)]


class SampleToppArgs(C.Structure):
    _fields_ = [("logits", C.c_void_p), ("ld_logits", C.c_int64), ("s_logits", C.c_float), ("p", C.c_float),
                ("rows", C.c_int32), ("vocab", C.c_int32), ("max_step", C.c_int32), ("end_id", C.c_int32),
                ("seed_lo", C.c_uint32), ("seed_hi", C.c_uint32), ("seq", C.c_void_p), ("cur", C.c_void_p),
                ("ticket", C.c_void_p), ("n_ended", C.c_void_p), ("stop", C.c_void_p), ("stop_host", C.c_void_p)]


lib.ls100_strerror.restype = C.c_char_p
lib.ls100_strerror.argtypes = [C.c_int]
lib.ls100_ctx_create.restype = C.c_int
lib.ls100_ctx_create.argtypes = [C.POINTER(C.c_void_p), C.c_int]
lib.ls100_ctx_destroy.restype = None
lib.ls100_ctx_destroy.argtypes = [C.c_void_p]
lib.ls100_ctx_poll_error.restype = C.c_int
lib.ls100_ctx_poll_error.argtypes = [C.c_void_p, C.c_void_p]
lib.ls100_sm_count.restype = C.c_int
lib.ls100_sm_count.argtypes = [C.c_void_p]
lib.ls100_gemm_i8.restype = C.c_int
lib.ls100_gemm_i8.argtypes = [C.c_void_p, C.POINTER(GemmI8Args), C.c_void_p]
lib.ls100_gemm_i8_table_bytes.restype = C.c_size_t
lib.ls100_gemm_i8_table_bytes.argtypes = [C.c_int64]
lib.ls100_gemm_i8_build_table.restype = C.c_int
lib.ls100_gemm_i8_build_table.argtypes = [C.c_void_p, C.POINTER(GemmI8Args), C.c_void_p, C.c_void_p]


for _name, _cls in (("ls100_ln_quant", LnQuantArgs), ("ls100_embed", EmbedArgs), ("ls100_attn_self", AttnSelfArgs),
                    ("ls100_attn_dec", AttnDecArgs), ("ls100_attn_cross", AttnCrossArgs),
                    ("ls100_proj_f32", ProjF32Args), ("ls100_beam_topk", BeamTopkArgs),
                    ("ls100_beam_update", BeamUpdateArgs), ("ls100_beam_update_noalloc", BeamUpdateArgs), ("ls100_sample_topk", SampleTopkArgs),
                    ("ls100_sample_topp", SampleToppArgs),
                    ("ls100_proj_tc", ProjTcArgs), ("ls100_patch_embed", PatchEmbedArgs),
                    ("ls100_beam_write_result", BeamResultArgs), ("ls100_beam_select", BeamSelectArgs)):
    _fn = getattr(lib, _name)
    _fn.restype = C.c_int
    _fn.argtypes = [C.c_void_p, C.POINTER(_cls), C.c_void_p]
lib.ls100_split_bf16x3.restype = C.c_int
lib.ls100_split_bf16x3.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
lib.ls100_i8_to_bf16.restype = C.c_int
lib.ls100_i8_to_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
lib.ls100_quantize_weight.restype = C.c_int
lib.ls100_quantize_weight.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_float, C.c_void_p,
                                      C.c_void_p, C.c_void_p]
lib.ls100_measure_i8_mma_peak.restype = C.c_int
lib.ls100_measure_i8_mma_peak.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_float)]
lib.ls100_measure_phase_floor.restype = C.c_int
lib.ls100_measure_phase_floor.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.POINTER(C.c_float)]
lib.ls100_debug_expire_wait.restype = C.c_int
lib.ls100_debug_expire_wait.argtypes = [C.c_void_p, C.c_void_p]


def call(name: str, ctx: "Context", args, stream: int = 0) -> None:
    """Launches ``name`` and raises on a non-zero status."""
    check(getattr(lib, name)(ctx.handle, C.byref(args), C.c_void_p(stream)), name)


class Context:
    """Owns one ``ls100_ctx`` for a device."""

    def __init__(self, device: int = 0):
        h = C.c_void_p()
        check(lib.ls100_ctx_create(C.byref(h), device), "ls100_ctx_create")
        self.handle = h
        self.device = device

    def poll_error(self, stream: int = 0) -> int:
        return lib.ls100_ctx_poll_error(self.handle, C.c_void_p(stream))

    def close(self):
        if self.handle:
            lib.ls100_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
