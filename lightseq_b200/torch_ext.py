"""Torch-tensor entry points with the signatures of the reference's training-side extension
(lightseq/csrc/pybind/pybind_layer.cpp:421-476, 553-560), forward only, on the B200 kernels:

    create_quant_linear_layer_fp32 / _fp16(layer_id, in_features, out_features, max_batch_tokens) -> 0
    quant_linear_layer_fw_fp32 / _fp16(layer_id, inputs[B,S,K], weight[N,K], clip_max[3], quant_mode) -> Tensor[B,S,N]

``quant_mode=True`` is QuantLinearLayer<T>::Forward's int8 branch (lightseq/csrc/layers/quant_linear_layer.cpp:
25-52): quantise the input with clip_max[0], the weight with clip_max[1], int8 GEMM, requantise the accumulators
with clip_max[2], dequantise. Here that is two launches of the weight/activation quantiser and ONE GEMM whose
epilogue does the requantise + dequantise; the arithmetic is the exact-integer form of
QuantLinear.forward (lightseq/training/ops/pytorch/quantization.py:50-61) without bias, as in the reference
layer. ``quant_mode=False`` is the reference's unquantised cuBLAS branch, which is not part of the int8 path:
it is passed to torch.nn.functional.linear.

Layers live in a module-level table keyed by ``layer_id`` (static unordered_map in the reference); the stream is
torch's current stream; inputs must be CUDA and contiguous (CHECK_INPUT in the reference). Reading the three
clip-max values costs one device-to-host copy whenever the clip_max tensor has changed since the last call.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict

import torch

from . import _lib as L

_contexts: Dict[int, "L.Context"] = {}
_layers: Dict[int, "_QuantLinearLayer"] = {}


def _ctx(device: int) -> "L.Context":
    c = _contexts.get(device)
    if c is None:
        with torch.cuda.device(device):
            c = L.Context(device)
        _contexts[device] = c
    return c


def _check_input(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


class _QuantLinearLayer:
    def __init__(self, layer_id: int, in_features: int, out_features: int, max_batch_tokens: int, dtype: torch.dtype):
        if in_features % 16 or out_features <= 0 or max_batch_tokens <= 0:
            raise RuntimeError("in_features must be a multiple of 16 (int8 rows are 16-byte aligned for TMA)")
        self.layer_id, self.k, self.n, self.max_tokens, self.dtype = layer_id, in_features, out_features, max_batch_tokens, dtype
        self.buffers = {}  # device index -> (x_q, w_q)
        self.cmax_key = None
        self.cmax = None

    def _bufs(self, device: torch.device):
        b = self.buffers.get(device.index)
        if b is None:
            b = (torch.empty(self.max_tokens, self.k, dtype=torch.int8, device=device),
                 torch.empty(self.n, self.k, dtype=torch.int8, device=device))
            self.buffers[device.index] = b
        return b

    def _clip_max(self, clip_max: torch.Tensor):
        # The host copy is reused only for the SAME tensor object at the same version. An address is not an identity:
        # a fresh tensor built per call usually gets the previous one's address back from the caching allocator, and
        # its new values must not be ignored. The cached object is kept alive so that `is` cannot be fooled either.
        if self.cmax_key is None or self.cmax_key[0] is not clip_max or self.cmax_key[1] != clip_max._version:
            v = [float(x) for x in clip_max.detach().float().cpu().tolist()]
            if len(v) != 3 or not all(x > 0 for x in v):
                raise RuntimeError("clip_max must hold three positive values: input, weight, output")
            self.cmax_key, self.cmax = (clip_max, clip_max._version), v
        return self.cmax

    def forward(self, inputs: torch.Tensor, weight: torch.Tensor, clip_max: torch.Tensor, quant_mode: bool) -> torch.Tensor:
        _check_input(inputs, "inputs")
        _check_input(weight, "weight")
        if inputs.dim() != 3 or inputs.size(2) != self.k or tuple(weight.shape) != (self.n, self.k):
            raise RuntimeError("expected inputs [batch, seq, in_features] and weight [out_features, in_features]")
        if inputs.dtype != self.dtype or weight.dtype != self.dtype:
            raise RuntimeError(f"layer {self.layer_id} was created for {self.dtype}")
        bsz, seq = inputs.size(0), inputs.size(1)
        tokens = bsz * seq
        if tokens > self.max_tokens:
            raise RuntimeError("batch_size * seq_len exceeds max_batch_tokens")
        if not quant_mode:
            return torch.nn.functional.linear(inputs, weight)
        a_in, a_w, a_out = self._clip_max(clip_max)
        dev = inputs.device
        ctx = _ctx(dev.index)
        st = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        x32 = inputs.reshape(tokens, self.k).float()  # no copy for fp32 inputs
        w32 = weight.float()
        x_q, w_q = self._bufs(dev)
        with torch.cuda.device(dev):
            L.check(L.lib.ls100_quantize_weight(ctx.handle, C.c_void_p(x32.data_ptr()), tokens, self.k, a_in,
                                                C.c_void_p(x_q.data_ptr()), None, st), "quantize inputs")
            L.check(L.lib.ls100_quantize_weight(ctx.handle, C.c_void_p(w32.data_ptr()), self.n, self.k, a_w,
                                                C.c_void_p(w_q.data_ptr()), None, st), "quantize weight")
            out = torch.empty(tokens, self.n, dtype=torch.float32, device=dev)
            f32 = torch.tensor([a_in / 127.0, a_w / 127.0, a_out / 127.0], dtype=torch.float32)  # fp32 scale arithmetic
            args = L.GemmI8Args(a=x_q.data_ptr(), lda=self.k, w=w_q.data_ptr(), ldw=self.k, m=tokens, n=self.n, k=self.k,
                                s_acc=float(f32[0] * f32[1]), s_outq=float(f32[2]), out_kind=L.OUT_F32,
                                out=out.data_ptr(), ldo=self.n)
            L.check(L.lib.ls100_gemm_i8(ctx.handle, C.byref(args), st), "ls100_gemm_i8")
        out = out.reshape(bsz, seq, self.n)
        return out if self.dtype == torch.float32 else out.to(self.dtype)


def _create(layer_id: int, in_features: int, out_features: int, max_batch_tokens: int, dtype: torch.dtype) -> int:
    _layers[layer_id] = _QuantLinearLayer(layer_id, in_features, out_features, max_batch_tokens, dtype)
    return 0


def _forward(layer_id: int, inputs, weight, clip_max, quant_mode, dtype) -> torch.Tensor:
    layer = _layers.get(layer_id)
    if layer is None:
        raise RuntimeError(f"quant linear layer {layer_id} has not been created")
    if layer.dtype != dtype:
        raise RuntimeError(f"quant linear layer {layer_id} was created for {layer.dtype}")
    return layer.forward(inputs, weight, clip_max, bool(quant_mode))


def create_quant_linear_layer_fp32(layer_id: int, in_features: int, out_features: int, max_batch_tokens: int) -> int:
    return _create(layer_id, in_features, out_features, max_batch_tokens, torch.float32)


def create_quant_linear_layer_fp16(layer_id: int, in_features: int, out_features: int, max_batch_tokens: int) -> int:
    return _create(layer_id, in_features, out_features, max_batch_tokens, torch.float16)


def quant_linear_layer_fw_fp32(layer_id: int, inputs: torch.Tensor, weight: torch.Tensor, clip_max: torch.Tensor,
                               quant_mode: bool) -> torch.Tensor:
    return _forward(layer_id, inputs, weight, clip_max, quant_mode, torch.float32)


def quant_linear_layer_fw_fp16(layer_id: int, inputs: torch.Tensor, weight: torch.Tensor, clip_max: torch.Tensor,
                               quant_mode: bool) -> torch.Tensor:
    return _forward(layer_id, inputs, weight, clip_max, quant_mode, torch.float16)


# ------------------------------------------------------------------------------------------------------------------
# transformer_encoder_layer_fw: the quantised forward of LSTransformerEncoderLayer.eval()
# (lightseq/training/ops/pytorch/transformer_encoder_layer.py:119-172 for the parameter layout,
# lightseq/csrc/pybind/pybind_layer.cpp:28-73 for the entry points). The layer's single flat parameter tensor holds
#   qkv weight [3H,H], qkv bias [3H], out weight [H,H], out bias [H], attention LayerNorm g/b [H],
#   fc1 weight [F,H], fc1 bias [F], fc2 weight [H,F], fc2 bias [H], FFN LayerNorm g/b [H], clip_max [12]
# with clip_max = (input, weight, output) for each of qkv, out, fc1, fc2. Numerics are those of the torch fake-quant
# TransformerEncoderLayer (lightseq/training/ops/pytorch/torch_transformer_layers.py) on exact integer accumulators.
_encoder_layers: Dict[int, "_EncoderLayer"] = {}


def _gen_offset(hs: int, ims: int):
    sizes = [hs * hs * 3, hs * 3, hs * hs, hs, hs, hs, hs * ims, ims, hs * ims, hs, hs, hs, 12]
    off = [0]
    for s in sizes:
        off.append(off[-1] + s)
    return off


class _EncoderLayer:
    def __init__(self, layer_id, max_batch_tokens, max_seq_len, hidden, heads, ffn, pre_ln, activation_fn, mask_future, dtype):
        if hidden != heads * 64:
            raise RuntimeError("the B200 attention kernels need head_dim 64")
        if activation_fn not in ("relu", "gelu"):
            raise RuntimeError("activation_fn must be relu or gelu")
        self.layer_id, self.max_tokens, self.max_seq = layer_id, max_batch_tokens, max_seq_len
        self.H, self.heads, self.F, self.pre_ln, self.act, self.causal = hidden, heads, ffn, bool(pre_ln), activation_fn, bool(mask_future)
        self.dtype = dtype
        self.offset = _gen_offset(hidden, ffn)
        self.para = None
        self.key = None
        self.state = None  # per-version: int8 weights, offsets, fp32 vectors, clip-max

    def assign(self, weight: torch.Tensor):
        if weight.numel() != self.offset[-1]:
            raise RuntimeError(f"parameter tensor has {weight.numel()} elements, the layer needs {self.offset[-1]}")
        if weight is not self.para:
            self.key = None  # a new tensor may sit at the old one's address: never reuse the prepared state for it
        self.para = weight

    def _prepare(self, ctx, st):
        p = self.para
        key = (p.data_ptr(), p._version, p.device.index)
        if key == self.key:
            return self.state
        H, F, o = self.H, self.F, self.offset
        f = p.detach().float().contiguous()
        seg = [f[o[i]:o[i + 1]] for i in range(13)]
        cm = [float(v) for v in seg[12].cpu().tolist()]
        if not all(v > 0 for v in cm):
            raise RuntimeError("clip_max values must be positive")
        dev = p.device
        shapes = {"qkv": (3 * H, H), "out": (H, H), "fc1": (F, H), "fc2": (H, F)}
        s = {"cm": cm, "vec": seg}
        for i, (name, wi) in enumerate((("qkv", 0), ("out", 2), ("fc1", 6), ("fc2", 8))):
            n, k = shapes[name]
            wq = torch.empty(n, k, dtype=torch.int8, device=dev)
            off = torch.empty(n, dtype=torch.int32, device=dev)
            L.check(L.lib.ls100_quantize_weight(ctx.handle, C.c_void_p(seg[wi].data_ptr()), n, k, cm[3 * i + 1],
                                                C.c_void_p(wq.data_ptr()), C.c_void_p(off.data_ptr()), st), "quantize " + name)
            s[name] = (wq, off)
        self.key, self.state = key, s
        return s

    def forward(self, inp: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        _check_input(inp, "input")
        _check_input(mask, "input_mask")
        if self.para is None:
            raise RuntimeError(f"encoder layer {self.layer_id}: assign_layer_weight_grad has not been called")
        if inp.dim() != 3 or inp.size(2) != self.H or inp.dtype != self.dtype:
            raise RuntimeError("expected input [batch, seq, hidden] of the layer's dtype")
        B, S = inp.size(0), inp.size(1)
        rows = B * S
        if rows > self.max_tokens or S > self.max_seq:
            raise RuntimeError("batch tokens exceed max_batch_tokens or seq_len exceeds max_seq_len")
        if tuple(mask.shape) != (B, S):
            raise RuntimeError("input_mask must be [batch, seq] with 1 at padding positions")
        dev = inp.device
        ctx = _ctx(dev.index)
        st = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        H, F = self.H, self.F
        with torch.cuda.device(dev):
            s = self._prepare(ctx, st)
            cm, v = s["cm"], s["vec"]
            f32 = lambda a: float(torch.tensor(a, dtype=torch.float32))  # noqa: E731
            sc = lambda a, unsigned=False: f32(f32(a) / (254.0 if unsigned else 127.0))  # noqa: E731
            mul = lambda a, b: float(torch.tensor(a, dtype=torch.float32) * torch.tensor(b, dtype=torch.float32))  # noqa: E731
            relu = self.act == "relu"
            x = inp.reshape(rows, H).float().clone()  # residual stream, updated in place
            pad = (mask.reshape(B, S) != 0).to(torch.uint8).contiguous()
            a_q = torch.empty(rows, H, dtype=torch.int8, device=dev)
            qkv_q = torch.empty(rows, 3 * H, dtype=torch.int8, device=dev)
            attn_q = torch.empty(rows, H, dtype=torch.int8, device=dev)
            h_q = torch.empty(rows, F, dtype=torch.int8, device=dev)
            p = lambda t: None if t is None else t.data_ptr()  # noqa: E731

            def ln(g, b, amax, write_f=False, write_q=True):
                a = L.LnQuantArgs(x=p(x), ldx=H, gamma=p(g), beta=p(b), rows=rows, hidden=H, amax=amax,
                                  out_q=p(a_q) if write_q else None, ldq=H, out_f=p(x) if write_f else None, ldf=H)
                L.check(L.lib.ls100_ln_quant(ctx.handle, C.byref(a), st), "ls100_ln_quant")

            def gemm(a_in, name, idx, n, k, out, out_kind, bias, act=L.ACT_NONE, resid=None, s_req=0.0, unsigned_in=False):
                wq, off = s[name]
                a = L.GemmI8Args(a=p(a_in), lda=k, w=p(wq), ldw=k, m=rows, n=n, k=k,
                                 s_acc=mul(sc(cm[3 * idx], unsigned_in), sc(cm[3 * idx + 1])),
                                 w_off=p(off) if unsigned_in else None, s_outq=sc(cm[3 * idx + 2]), bias=p(bias), act=act,
                                 resid=p(resid) if resid is not None else None, ldr=n, out_kind=out_kind, s_req=s_req,
                                 out=p(out), ldo=n)
                L.check(L.lib.ls100_gemm_i8(ctx.handle, C.byref(a), st), "ls100_gemm_i8 " + name)

            if self.pre_ln:
                ln(v[4], v[5], cm[0])
            else:  # post-LN: the block input itself is quantised
                L.check(L.lib.ls100_quantize_weight(ctx.handle, C.c_void_p(p(x)), rows, H, cm[0], C.c_void_p(p(a_q)), None, st),
                        "quantize input")
            gemm(a_q, "qkv", 0, 3 * H, H, qkv_q, L.OUT_OUTQ_I8, None)
            at = L.AttnSelfArgs(qkv=p(qkv_q), ld_qkv=3 * H, s_qkv=sc(cm[2]), bias=p(v[1]), pad_mask=p(pad), batch=B, seq=S,
                                heads=self.heads, causal=int(self.causal), amax_out=cm[3], out=p(attn_q), ld_out=H)
            L.check(L.lib.ls100_attn_self(ctx.handle, C.byref(at), st), "ls100_attn_self")
            gemm(attn_q, "out", 1, H, H, x, L.OUT_F32, v[3], resid=x)
            if self.pre_ln:
                ln(v[10], v[11], cm[6])
            else:
                ln(v[4], v[5], cm[6], write_f=True)
            gemm(a_q, "fc1", 2, F, H, h_q, L.OUT_REQ_U8 if relu else L.OUT_REQ_S8, v[7], act=L.ACT_RELU if relu else L.ACT_GELU,
                 s_req=sc(cm[9], relu))
            gemm(h_q, "fc2", 3, H, F, x, L.OUT_F32, v[9], resid=x, unsigned_in=relu)
            if not self.pre_ln:
                ln(v[10], v[11], 1.0, write_f=True, write_q=False)
        out = x.reshape(B, S, H)
        return out if self.dtype == torch.float32 else out.to(self.dtype)


def _create_encoder(dtype, layer_id, max_batch_tokens, max_seq_len, hidden_dim, num_heads, intermediate_size,
                    attn_prob_dropout_ratio, activation_dropout_ratio, hidden_dropout_ratio, is_pre_ln, activation_fn,
                    mask_future_tokens) -> int:
    del attn_prob_dropout_ratio, activation_dropout_ratio, hidden_dropout_ratio  # inference: dropout is the identity
    _encoder_layers[layer_id] = _EncoderLayer(layer_id, max_batch_tokens, max_seq_len, hidden_dim, num_heads, intermediate_size,
                                              is_pre_ln, activation_fn, mask_future_tokens, dtype)
    return 0


def create_transformer_encoder_layer_fp32(*args) -> int:
    return _create_encoder(torch.float32, *args)


def create_transformer_encoder_layer_fp16(*args) -> int:
    return _create_encoder(torch.float16, *args)


def assign_layer_weight_grad(layer_id: int, weight: torch.Tensor, grad, layer_name: str) -> None:
    """Binds the layer's flat parameter tensor (pybind_layer.cpp:300-337); gradients are not used in inference."""
    del grad
    if layer_name != "TransformerEncoderLayer":
        raise RuntimeError(f"{layer_name}: only TransformerEncoderLayer has a B200 quantised forward")
    layer = _encoder_layers.get(layer_id)
    if layer is None:
        raise RuntimeError(f"encoder layer {layer_id} has not been created")
    _check_input(weight, "weight")
    layer.assign(weight)


def _encoder_fw(dtype, layer_id, inp, input_mask, training_mode, prelayernorm, quant_mode):
    layer = _encoder_layers.get(layer_id)
    if layer is None:
        raise RuntimeError(f"encoder layer {layer_id} has not been created")
    if layer.dtype != dtype:
        raise RuntimeError(f"encoder layer {layer_id} was created for {layer.dtype}")
    if training_mode:
        raise RuntimeError("the B200 layer is forward-only (training_mode must be False)")
    if not quant_mode:
        raise RuntimeError("the B200 layer implements the quantised forward only (quant_mode must be True)")
    if bool(prelayernorm) != layer.pre_ln:
        raise RuntimeError("prelayernorm differs from the layer's configuration")
    return [layer.forward(inp, input_mask)]


def transformer_encoder_layer_fw_fp32(layer_id, inp, input_mask, training_mode, prelayernorm, quant_mode):
    return _encoder_fw(torch.float32, layer_id, inp, input_mask, training_mode, prelayernorm, quant_mode)


def transformer_encoder_layer_fw_fp16(layer_id, inp, input_mask, training_mode, prelayernorm, quant_mode):
    return _encoder_fw(torch.float16, layer_id, inp, input_mask, training_mode, prelayernorm, quant_mode)
