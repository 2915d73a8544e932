"""Reader and writer for the reference's ``QuantTransformer`` protobuf weight files
(lightseq/inference/proto/quant_transformer.proto:10-165) and, further down, its ``QuantBert``, ``QuantGpt`` and
``QuantVit`` files (quant_bert.proto, quant_gpt.proto, quant_vit.proto), without protoc or the protobuf package: a
proto3 wire-format codec (varint / 32-bit / length-delimited fields, packed and unpacked repeated floats) plus the
field tables of the messages.

Conventions of the files, taken from the exporter that writes them
(examples/inference/python/export/fairseq/ls_torch_fs_quant_transformer_export.py:20-290,
lightseq/training/ops/pytorch/export_quant.py:12-19) and the loader that reads them
(lightseq/inference/proto/quant_transformer_weight.cc:95-510):

* every ``*_kernel*`` and ``token_embedding`` field is ``bytes`` of uint8 ``u = q + 127`` with
  ``q = floor(clip(x * 127 / clip_max, -127, 127) + 0.5)``; the loader dequantises ``(u - 127) * clip_max / 127``;
* linear kernels are stored transposed, ``[in, out]`` (torch keeps ``[out, in]``); the target token embedding is
  stored transposed, ``[hidden, vocab]``; ``encode_output_project_kernel_kv`` is the transpose of
  ``concat(k_0, v_0, k_1, v_1, ...)``, i.e. ``[hidden, n_dec * 2 * hidden]``, its bias ``[n_dec, 2, hidden]``, and it
  carries ONE clip-max per decoder layer (that of k_proj) for both matrices;
* sizes are not stored: hidden = len(norm_scale), max_step = len(position_embedding) / hidden,
  vocab = len(token_embedding) / hidden, ffn = len(ffn_first_bias).

``read_quant_transformer`` returns the engine's (conf, amax, tensors) triple (fp32 tensors in torch layout, as
``lightseq_b200.weights.save`` takes them); ``write_quant_transformer`` is its inverse. No file written by the
reference's own exporter is available offline, so the pair is checked by round trip and against the schema only.
"""
from __future__ import annotations

import struct
from typing import Dict, List, Tuple

import numpy as np

F32 = np.float32


# ------------------------------------------------------------------------------------------------ wire format
def _varint(n: int) -> bytes:
    if n < 0:
        n += 1 << 64  # int32 / int64 negatives are sign-extended to 64 bits
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        out.append(b | (0x80 if n else 0))
        if not n:
            return bytes(out)


def _tag(field: int, wt: int) -> bytes:
    return _varint((field << 3) | wt)


def _read_varint(buf: memoryview, pos: int) -> Tuple[int, int]:
    n = shift = 0
    while True:
        b = buf[pos]
        pos += 1
        n |= (b & 0x7F) << shift
        shift += 7
        if not b & 0x80:
            return n, pos
        if shift > 70:
            raise ValueError("malformed varint")


def parse_message(buf) -> Dict[int, List[Tuple[int, object]]]:
    """field number -> list of (wire type, value) in file order; length-delimited values stay memoryviews."""
    buf = memoryview(buf)
    out: Dict[int, List[Tuple[int, object]]] = {}
    pos, end = 0, len(buf)
    while pos < end:
        key, pos = _read_varint(buf, pos)
        field, wt = key >> 3, key & 7
        if wt == 0:
            val, pos = _read_varint(buf, pos)
        elif wt == 1:
            val, pos = bytes(buf[pos:pos + 8]), pos + 8
        elif wt == 2:
            n, pos = _read_varint(buf, pos)
            if pos + n > end:
                raise ValueError("length-delimited field runs past the end of the message")
            val, pos = buf[pos:pos + n], pos + n
        elif wt == 5:
            val, pos = bytes(buf[pos:pos + 4]), pos + 4
        else:
            raise ValueError(f"unsupported wire type {wt}")
        out.setdefault(field, []).append((wt, val))
    return out


def _floats(msg, field: int) -> np.ndarray:
    parts = []
    for wt, v in msg.get(field, []):
        if wt == 2:  # packed
            parts.append(np.frombuffer(v, dtype="<f4"))
        elif wt == 5:
            parts.append(np.frombuffer(v, dtype="<f4"))
        else:
            raise ValueError(f"field {field}: not a float field")
    return np.concatenate(parts).astype(F32) if parts else np.zeros(0, F32)


def _float(msg, field: int, default: float = 0.0) -> float:
    v = msg.get(field)
    return float(struct.unpack("<f", v[-1][1])[0]) if v else default


def _int(msg, field: int, default: int = 0) -> int:
    v = msg.get(field)
    if not v:
        return default
    n = int(v[-1][1])
    return n - (1 << 64) if n >= 1 << 63 else n


def _bytes(msg, field: int) -> np.ndarray:
    v = msg.get(field)
    return np.frombuffer(v[-1][1], dtype=np.uint8) if v else np.zeros(0, np.uint8)


def _str(msg, field: int, default: str = "") -> str:
    v = msg.get(field)
    return bytes(v[-1][1]).decode() if v else default


def _enc_floats(field: int, a) -> bytes:
    a = np.ascontiguousarray(a, dtype="<f4").reshape(-1)
    return _tag(field, 2) + _varint(a.nbytes) + a.tobytes() if a.size else b""


def _enc_float(field: int, v: float) -> bytes:
    return _tag(field, 5) + struct.pack("<f", float(v)) if float(v) != 0.0 else b""


def _enc_int(field: int, v: int) -> bytes:
    return _tag(field, 0) + _varint(int(v)) if int(v) != 0 else b""


def _enc_bytes(field: int, b: bytes) -> bytes:
    return _tag(field, 2) + _varint(len(b)) + b if len(b) else b""


# ------------------------------------------------------------------------------------------------ quantised tensors
def _quant_u8(x: np.ndarray, clip_max: float) -> np.ndarray:
    """export_quant.py:12-19."""
    x = np.asarray(x, dtype=F32)
    return np.floor(np.clip(x * F32(127) / F32(clip_max), -127, 127) + 127 + 0.5).astype(np.uint8)


def _dequant(u: np.ndarray, clip_max: float) -> np.ndarray:
    """quant_transformer_weight.cc: dequantize(ele, quant_range, clip_max) = (ele - 127) * clip_max / 127."""
    return ((u.astype(F32) - F32(127)) * F32(clip_max) / F32(127)).astype(F32)


def _quant_engine(x: np.ndarray, clip_max: float) -> np.ndarray:
    """uint8 = q + 127 with the engine's own rounding, q = floor(x / (clip_max / 127) + 0.5) in fp32: the same integers
    as export_quant.quantize except where fp32 rounding of x * 127 / clip_max and x / (clip_max / 127) differs at an
    exact half, so that a file written here and read back gives the engine bit-identical int8 weights."""
    x = np.clip(np.asarray(x, dtype=F32), -F32(clip_max), F32(clip_max))
    s = F32(clip_max) / F32(127)
    q = np.clip(np.floor(x / s + F32(0.5)), -127, 127)
    return (q + 127).astype(np.uint8)


# (proto field, engine suffix) tables. Kernels are (bytes field, clip-max field, engine weight name).
_ENC_VEC = [(1, "ln1.g"), (2, "ln1.b"), (4, "qkv.b"), (6, "out.b"), (7, "ln2.g"), (8, "ln2.b"), (10, "fc1.b"), (12, "fc2.b")]
_ENC_KER = [(3, 13, "qkv.w"), (5, 14, "out.w"), (9, 15, "fc1.w"), (11, 16, "fc2.w")]
_ENC_CLIP = [(17, "qkv.in"), (18, "out.in"), (19, "fc1.in"), (20, "fc2.in"), (21, "qkv.out"), (22, "out.out"),
             (23, "fc1.out"), (24, "fc2.out")]
_DEC_VEC = [(1, "ln1.g"), (2, "ln1.b"), (4, "qkv.b"), (6, "out.b"), (7, "ln2.g"), (8, "ln2.b"), (10, "xq.b"), (12, "xout.b"),
            (13, "ln3.g"), (14, "ln3.b"), (16, "fc1.b"), (18, "fc2.b")]
_DEC_KER = [(3, 19, "qkv.w"), (5, 20, "out.w"), (9, 21, "xq.w"), (11, 22, "xout.w"), (15, 23, "fc1.w"), (17, 24, "fc2.w")]
_DEC_CLIP = [(25, "qkv.in"), (26, "out.in"), (27, "xq.in"), (28, "xout.in"), (29, "fc1.in"), (30, "fc2.in"),
             (31, "qkv.out"), (32, "out.out"), (33, "xq.out"), (34, "xout.out"), (35, "fc1.out"), (36, "fc2.out"), (37, "kv")]


def _read_layer(msg, prefix, vec, ker, clip, amax, tensors, dims):
    for f, name in vec:
        tensors[f"{prefix}.{name}"] = _floats(msg, f)
    for f, name in clip:
        amax[f"{prefix}.{name}"] = _float(msg, f)
    for fb, fc, name in ker:
        c = _float(msg, fc)
        u = _bytes(msg, fb)
        n_out = tensors[f"{prefix}.{name[:-2]}.b"].size  # bias length = output features
        if c <= 0 or u.size == 0 or u.size % n_out:
            raise ValueError(f"{prefix}.{name}: missing kernel or clip-max")
        amax[f"{prefix}.{name}"] = c
        tensors[f"{prefix}.{name}"] = np.ascontiguousarray(_dequant(u, c).reshape(u.size // n_out, n_out).T)  # [in,out] -> [out,in]
    dims.setdefault("ffn", tensors[f"{prefix}.fc1.b"].size)


def read_quant_transformer(path: str):
    """Reference QuantTransformer protobuf file -> (conf, amax, tensors) of the engine."""
    root = parse_message(open(path, "rb").read())
    for f in (1, 3, 5):
        if f not in root:
            raise ValueError("not a QuantTransformer file: src_embedding, trg_embedding and model_conf are required")
    src, trg, mc = parse_message(root[1][-1][1]), parse_message(root[3][-1][1]), parse_message(root[5][-1][1])
    amax: Dict[str, float] = {}
    t: Dict[str, np.ndarray] = {}
    H = _floats(src, 3).size
    if H == 0:
        raise ValueError("src_embedding.norm_scale is empty")
    pos = _floats(src, 2)
    max_step = pos.size // H
    emb_u = _bytes(src, 1)
    V = emb_u.size // H
    c_emb = _float(src, 9)
    t["emb"] = _dequant(emb_u, c_emb).reshape(V, H)
    amax["emb"] = c_emb
    trg_u = _bytes(trg, 1)
    if trg_u.size != emb_u.size or not np.array_equal(trg_u.reshape(H, V).T, emb_u.reshape(V, H)) or _float(trg, 9) != c_emb:
        raise ValueError("source and target embeddings differ: the engine shares one table (share-all-embeddings models)")
    t["pos"] = pos.reshape(max_step, H)
    t["enc.ln.g"], t["enc.ln.b"] = _floats(src, 3), _floats(src, 4)
    t["dec.ln.g"], t["dec.ln.b"] = _floats(trg, 3), _floats(trg, 4)
    amax["logits.in"], amax["logits.out"] = _float(trg, 11), _float(trg, 12)
    dims: Dict[str, int] = {}
    enc_layers, dec_layers = root.get(2, []), root.get(4, [])
    for i, (_, m) in enumerate(enc_layers):
        _read_layer(parse_message(m), f"enc.{i}", _ENC_VEC, _ENC_KER, _ENC_CLIP, amax, t, dims)
    for i, (_, m) in enumerate(dec_layers):
        _read_layer(parse_message(m), f"dec.{i}", _DEC_VEC, _DEC_KER, _DEC_CLIP, amax, t, dims)
    n_dec = len(dec_layers)
    kv_u = _bytes(trg, 5)
    kv_b = _floats(trg, 6)
    kv_c = _floats(trg, 10)
    if kv_u.size != H * 2 * n_dec * H or kv_b.size != 2 * n_dec * H or kv_c.size != n_dec:
        raise ValueError("encode_output_project_kernel_kv / bias / clip_max have the wrong size")
    kv_u = kv_u.reshape(H, n_dec, 2, H)  # [in, layer, k|v, out]
    kv_b = kv_b.reshape(n_dec, 2, H)
    for i in range(n_dec):
        for j, nm in enumerate(("xk", "xv")):
            t[f"dec.{i}.{nm}.w"] = np.ascontiguousarray(_dequant(kv_u[:, i, j, :], float(kv_c[i])).T)
            t[f"dec.{i}.{nm}.b"] = kv_b[i, j].copy()
            amax[f"dec.{i}.{nm}.w"] = float(kv_c[i])
    if _int(mc, 15) != 0:
        raise ValueError("multilingual models are not supported by the engine")
    # fields that change the reference's output and that the engine does not implement are refused, not dropped
    bias = _floats(trg, 7)
    if bias.size and np.any(bias != 0):
        raise ValueError("a non-zero shared_bias (logit bias) is not supported by the engine")
    if _floats(src, 8).size or _floats(trg, 8).size:
        raise ValueError("language embeddings (lang_emb) are not supported by the engine")
    trg_pos = _floats(trg, 2)
    if trg_pos.size and (trg_pos.size != t["pos"].size or not np.array_equal(trg_pos, t["pos"].reshape(-1))):
        raise ValueError("the target position table differs from the source one: the engine holds a single table")
    method = _str(mc, 8, "beam_search")
    methods = ("beam_search", "topk", "topp", "topk_greedy")
    if method not in methods:
        raise ValueError(f"unknown sampling_method {method!r}")
    # QuantTransformer of the reference returns every beam (its decoder is built with output_topk = true,
    # lightseq/inference/pywrapper/quant_transformer.cc:60-62): files in its format keep that behaviour
    conf = dict(hidden=H, heads=_int(mc, 1), ffn=dims.get("ffn", 0), n_enc=len(enc_layers), n_dec=n_dec, vocab=V,
                act_gelu=float(_int(mc, 14)), pre_ln=float(not _int(mc, 12)), beam=_int(mc, 2), length_penalty=_float(mc, 4),
                extra_decode_length=_int(mc, 3), max_step=max_step, pad_id=_int(mc, 5), start_id=_int(mc, 6), end_id=_int(mc, 11),
                sampling_method=float(methods.index(method)), topk=float(max(_int(mc, 10), 1)), topp=_float(mc, 9),
                output_topk=1.0, no_scale_embedding=float(_int(mc, 13)), diverse_lambda=_float(mc, 7))
    return conf, amax, t


def _write_layer(prefix, vec, ker, clip, amax, t) -> bytes:
    out = bytearray()
    fields = []
    for f, name in vec:
        fields.append((f, _enc_floats(f, t[f"{prefix}.{name}"])))
    for fb, fc, name in ker:
        c = amax[f"{prefix}.{name}"]
        w = t[f"{prefix}.{name}"]  # [out, in] -> stored [in, out]
        fields.append((fb, _enc_bytes(fb, _quant_engine(w, c).T.tobytes())))
        fields.append((fc, _enc_float(fc, c)))
    for f, name in clip:
        fields.append((f, _enc_float(f, amax[f"{prefix}.{name}"])))
    for _, b in sorted(fields, key=lambda x: x[0]):
        out += b
    return bytes(out)


def write_quant_transformer(path: str, conf, amax, t) -> None:
    """(conf, amax, tensors) of the engine -> reference QuantTransformer protobuf file. The format holds one clip-max
    per decoder layer for both cross-attention projections: dec.i.xk.w and dec.i.xv.w must share theirs."""
    H, V = int(conf["hidden"]), int(conf["vocab"])
    n_enc, n_dec = int(conf["n_enc"]), int(conf["n_dec"])
    emb_u = _quant_engine(t["emb"], amax["emb"])  # [V, H]
    pos = np.asarray(t["pos"], F32)
    src = (_enc_bytes(1, emb_u.tobytes()) + _enc_floats(2, pos) + _enc_floats(3, t["enc.ln.g"]) + _enc_floats(4, t["enc.ln.b"]) +
           _enc_float(9, amax["emb"]))
    kv_u = np.zeros((H, n_dec, 2, H), np.uint8)
    kv_b = np.zeros((n_dec, 2, H), F32)
    kv_c = np.zeros(n_dec, F32)
    for i in range(n_dec):
        ck, cv = amax[f"dec.{i}.xk.w"], amax[f"dec.{i}.xv.w"]
        if F32(ck) != F32(cv):
            raise ValueError(f"dec.{i}: xk.w and xv.w have different clip-max values ({ck} vs {cv}); the file format holds one")
        kv_c[i] = ck
        for j, nm in enumerate(("xk", "xv")):
            kv_u[:, i, j, :] = _quant_engine(t[f"dec.{i}.{nm}.w"], ck).T
            kv_b[i, j] = t[f"dec.{i}.{nm}.b"]
    trg = (_enc_bytes(1, np.ascontiguousarray(emb_u.T).tobytes()) + _enc_floats(2, pos) + _enc_floats(3, t["dec.ln.g"]) +
           _enc_floats(4, t["dec.ln.b"]) + _enc_bytes(5, kv_u.tobytes()) + _enc_floats(6, kv_b) +
           _tag(7, 2) + _varint(4 * V) + np.zeros(V, "<f4").tobytes() +  # shared_bias: zeros, as the reference exporter writes
           _enc_float(9, amax["emb"]) + _enc_floats(10, kv_c) + _enc_float(11, amax["logits.in"]) + _enc_float(12, amax["logits.out"]))
    method = ("beam_search", "topk", "topp", "topk_greedy")[int(conf.get("sampling_method", 0))].encode()
    mc = (_enc_int(1, conf["heads"]) + _enc_int(2, conf["beam"]) + _enc_int(3, conf["extra_decode_length"]) +
          _enc_float(4, conf["length_penalty"]) + _enc_int(5, conf["pad_id"]) + _enc_int(6, conf["start_id"]) +
          _enc_float(7, conf.get("diverse_lambda", 0.0)) + _tag(8, 2) + _varint(len(method)) + method + _enc_float(9, conf.get("topp", 0.0)) + _enc_int(10, int(conf.get("topk", 1))) +
          _enc_int(11, conf["end_id"]) + _enc_int(12, 0 if int(conf.get("pre_ln", 1)) else 1) + _enc_int(13, 1 if conf.get("no_scale_embedding") else 0) +
          _enc_int(14, 1 if conf.get("act_gelu") else 0))
    out = bytearray()
    out += _tag(1, 2) + _varint(len(src)) + src
    for i in range(n_enc):
        m = _write_layer(f"enc.{i}", _ENC_VEC, _ENC_KER, _ENC_CLIP, amax, t)
        out += _tag(2, 2) + _varint(len(m)) + m
    out += _tag(3, 2) + _varint(len(trg)) + trg
    for i in range(n_dec):
        m = _write_layer(f"dec.{i}", _DEC_VEC, _DEC_KER, _DEC_CLIP, amax, t)
        out += _tag(4, 2) + _varint(len(m)) + m
    out += _tag(5, 2) + _varint(len(mc)) + mc
    with open(path, "wb") as f:
        f.write(out)


# ------------------------------------------------------------------------------------------------ QuantBert / QuantGpt / QuantVit
# Their layer message is the encoder layer of QuantTransformer without ffn_second_output_clip_max (the reference's
# encoder-only engines dequantise the second FFN GEMM straight from int32); QuantGpt adds self_qkv_bias_out_clip_max
# as field 24. A clip-max the file does not hold is stored as 0 = "this output is not quantised".
_ENC_CLIP_23 = _ENC_CLIP[:-1]


def _read_stack(root, prefix: str, amax, t, dims, kv_field: int = 0) -> int:
    layers = root.get(2, [])
    for i, (_, m) in enumerate(layers):
        msg = parse_message(m)
        _read_layer(msg, f"{prefix}.{i}", _ENC_VEC, _ENC_KER, _ENC_CLIP_23, amax, t, dims)
        amax[f"{prefix}.{i}.fc2.out"] = 0.0
        if kv_field:
            amax[f"{prefix}.{i}.kv"] = _float(msg, kv_field)
    return len(layers)


def _write_stack(prefix: str, n: int, amax, t, kv_field: int = 0) -> bytes:
    out = bytearray()
    for i in range(n):
        if float(amax.get(f"{prefix}.{i}.fc2.out", 0.0)) != 0.0:
            raise ValueError(f"{prefix}.{i}.fc2.out: this file format has no clip-max for the second FFN output (store 0)")
        m = _write_layer(f"{prefix}.{i}", _ENC_VEC, _ENC_KER, _ENC_CLIP_23, amax, t)
        if kv_field:
            m += _enc_float(kv_field, amax[f"{prefix}.{i}.kv"])
        out += _tag(2, 2) + _varint(len(m)) + m
    return bytes(out)


def _parts(path: str, what: str):
    root = parse_message(open(path, "rb").read())
    if 1 not in root or 3 not in root:
        raise ValueError(f"not a {what} file: src_embedding and model_conf are required")
    return root, parse_message(root[1][-1][1]), parse_message(root[3][-1][1])


def read_quant_bert(path: str):
    """Reference QuantBert protobuf file (lightseq/inference/proto/quant_bert.proto) -> (conf, amax, tensors). The file
    holds ONE token table (word + token-type 0 already summed by the exporter): it becomes ``emb`` with a zero
    ``type_emb``."""
    root, src, mc = _parts(path, "QuantBert")
    H = _floats(src, 3).size
    if H == 0:
        raise ValueError("src_embedding.norm_scale is empty")
    amax: Dict[str, float] = {}
    t: Dict[str, np.ndarray] = {}
    emb_u = _bytes(src, 1)
    V = emb_u.size // H
    amax["emb"] = _float(src, 5)
    t["emb"] = _dequant(emb_u, amax["emb"]).reshape(V, H)
    t["type_emb"] = np.zeros((2, H), F32)
    pos = _floats(src, 2)
    t["pos"] = pos.reshape(pos.size // H, H)
    t["emb.ln.g"], t["emb.ln.b"] = _floats(src, 3), _floats(src, 4)
    dims: Dict[str, int] = {}
    n = _read_stack(root, "enc", amax, t, dims)
    if _int(mc, 3) == 0:
        raise ValueError("pre-LN BERT models are not supported by the engine")
    if _int(mc, 5) != 0:
        raise ValueError("multilingual models are not supported by the engine")
    conf = dict(hidden=H, heads=_int(mc, 1), ffn=dims.get("ffn", 0), n_enc=n, vocab=V, act_gelu=float(_int(mc, 4)), pre_ln=0.0,
                max_step=pos.size // H, pad_id=_int(mc, 2))
    return conf, amax, t


def write_quant_bert(path: str, conf, amax, t) -> None:
    if np.any(np.asarray(t["type_emb"])[0] != 0):
        raise ValueError("the file format holds one token table: fold type_emb[0] into emb first")
    src = (_enc_bytes(1, _quant_engine(t["emb"], amax["emb"]).tobytes()) + _enc_floats(2, t["pos"]) + _enc_floats(3, t["emb.ln.g"]) +
           _enc_floats(4, t["emb.ln.b"]) + _enc_float(5, amax["emb"]))
    mc = _enc_int(1, conf["heads"]) + _enc_int(2, conf["pad_id"]) + _enc_int(3, 1) + _enc_int(4, 1 if conf.get("act_gelu") else 0)
    out = _tag(1, 2) + _varint(len(src)) + src + _write_stack("enc", int(conf["n_enc"]), amax, t) + _tag(3, 2) + _varint(len(mc)) + mc
    with open(path, "wb") as f:
        f.write(out)


def read_quant_gpt(path: str):
    """Reference QuantGpt protobuf file (lightseq/inference/proto/quant_gpt.proto) -> (conf, amax, tensors)."""
    root, src, mc = _parts(path, "QuantGpt")
    H = _floats(src, 3).size
    if H == 0:
        raise ValueError("src_embedding.norm_scale is empty")
    amax: Dict[str, float] = {}
    t: Dict[str, np.ndarray] = {}
    emb_u = _bytes(src, 1)
    V = emb_u.size // H
    amax["emb"] = _float(src, 5)
    t["emb"] = _dequant(emb_u, amax["emb"]).reshape(V, H)
    pos = _floats(src, 2)
    t["pos"] = pos.reshape(pos.size // H, H)
    t["dec.ln.g"], t["dec.ln.b"] = _floats(src, 3), _floats(src, 4)
    amax["logits.in"], amax["logits.out"] = _float(src, 6), _float(src, 7)
    dims: Dict[str, int] = {}
    n = _read_stack(root, "dec", amax, t, dims, kv_field=24)
    method = _str(mc, 3, "topk")
    if method not in ("topk", "topp"):
        raise ValueError(f"sampling_method {method!r}: the QuantGpt engine implements topk and topp")
    max_step = pos.size // H
    extra = _int(mc, 7)
    conf = dict(hidden=H, heads=_int(mc, 1), ffn=dims.get("ffn", 0), n_dec=n, vocab=V, act_gelu=1.0, pre_ln=1.0, max_step=max_step,
                end_id=_int(mc, 6), topk=_int(mc, 5, 1) if method == "topk" else 1, topp=_float(mc, 4) if method == "topp" else 0.0,
                pad_id=_int(mc, 2), max_new_tokens=extra if extra > 0 else max_step)
    return conf, amax, t


def write_quant_gpt(path: str, conf, amax, t) -> None:
    src = (_enc_bytes(1, _quant_engine(t["emb"], amax["emb"]).tobytes()) + _enc_floats(2, t["pos"]) + _enc_floats(3, t["dec.ln.g"]) +
           _enc_floats(4, t["dec.ln.b"]) + _enc_float(5, amax["emb"]) + _enc_float(6, amax["logits.in"]) + _enc_float(7, amax["logits.out"]))
    topp = float(conf.get("topp", 0.0))
    method = b"topp" if topp > 0 else b"topk"
    mc = (_enc_int(1, conf["heads"]) + _enc_int(2, conf.get("pad_id", 0)) + _tag(3, 2) + _varint(len(method)) + method + _enc_float(4, topp) +
          _enc_int(5, conf.get("topk", 1)) + _enc_int(6, conf["end_id"]) + _enc_int(7, conf.get("max_new_tokens", 0)))
    out = (_tag(1, 2) + _varint(len(src)) + src + _write_stack("dec", int(conf["n_dec"]), amax, t, kv_field=24) +
           _tag(3, 2) + _varint(len(mc)) + mc)
    with open(path, "wb") as f:
        f.write(out)


def read_quant_vit(path: str):
    """Reference QuantVit protobuf file (lightseq/inference/proto/quant_vit.proto) -> (conf, amax, tensors)."""
    root, src, mc = _parts(path, "QuantVit")
    H = _floats(src, 2).size
    if H == 0:
        raise ValueError("src_embedding.conv_bias is empty")
    patch, image = _int(mc, 4), _int(mc, 3)
    if patch < 1 or image < patch or image % patch:
        raise ValueError(f"image_size {image} / patch_size {patch}")
    amax: Dict[str, float] = {}
    t: Dict[str, np.ndarray] = {}
    cw = _floats(src, 1)
    if cw.size % (H * patch * patch):
        raise ValueError("conv_weight: size is not hidden * channels * patch * patch")
    channels = cw.size // (H * patch * patch)
    t["conv.w"] = cw.reshape(H, channels * patch * patch)
    t["conv.b"] = _floats(src, 2)
    n_tok = 1 + (image // patch) ** 2
    pos = _floats(src, 3)
    if pos.size < n_tok * H:
        raise ValueError("position_embedding is shorter than 1 + (image_size / patch_size)^2 rows")
    t["pos"] = pos.reshape(pos.size // H, H)[:n_tok].copy()
    t["cls"] = _floats(src, 4)
    t["enc.ln.g"], t["enc.ln.b"] = _floats(src, 5), _floats(src, 6)
    dims: Dict[str, int] = {}
    n = _read_stack(root, "enc", amax, t, dims)
    if _int(mc, 5) != 0:
        raise ValueError("post-LN ViT models are not supported by the engine")
    conf = dict(hidden=H, heads=_int(mc, 1), ffn=dims.get("ffn", 0), n_enc=n, act_gelu=float(_int(mc, 2)), pre_ln=1.0, max_step=n_tok,
                image_size=image, patch_size=patch, channels=channels)
    return conf, amax, t


def write_quant_vit(path: str, conf, amax, t) -> None:
    src = (_enc_floats(1, t["conv.w"]) + _enc_floats(2, t["conv.b"]) + _enc_floats(3, t["pos"]) + _enc_floats(4, t["cls"]) +
           _enc_floats(5, t["enc.ln.g"]) + _enc_floats(6, t["enc.ln.b"]))
    mc = (_enc_int(1, conf["heads"]) + _enc_int(2, 1 if conf.get("act_gelu") else 0) + _enc_int(3, conf["image_size"]) +
          _enc_int(4, conf["patch_size"]))
    out = _tag(1, 2) + _varint(len(src)) + src + _write_stack("enc", int(conf["n_enc"]), amax, t) + _tag(3, 2) + _varint(len(mc)) + mc
    with open(path, "wb") as f:
        f.write(out)


READERS = {"QuantTransformer": read_quant_transformer, "QuantBert": read_quant_bert, "QuantGpt": read_quant_gpt,
           "QuantVit": read_quant_vit}
WRITERS = {"QuantTransformer": write_quant_transformer, "QuantBert": write_quant_bert, "QuantGpt": write_quant_gpt,
           "QuantVit": write_quant_vit}


def convert(pb_path: str, ls100_path: str, model: str = "QuantTransformer") -> None:
    """Reference protobuf file of the named model class -> the engine's .ls100 container."""
    from . import weights

    if model not in READERS:
        raise ValueError(f"model {model!r}: one of {sorted(READERS)}")
    conf, amax, t = READERS[model](pb_path)
    weights.save(ls100_path, model, conf, amax, t)


if __name__ == "__main__":
    import sys

    if len(sys.argv) not in (3, 4):
        raise SystemExit("usage: python -m lightseq_b200.ls_proto <model.pb> <out.ls100> [QuantTransformer|QuantBert|QuantGpt|QuantVit]")
    convert(sys.argv[1], sys.argv[2], sys.argv[3] if len(sys.argv) == 4 else "QuantTransformer")
