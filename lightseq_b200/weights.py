"""Weight container of the B200 int8 engine (``.ls100`` files).

One flat little-endian file holding what the reference keeps in its
``QuantTransformer`` / ``QuantBert`` / ``QuantGpt`` protobuf or HDF5 files
(lightseq/inference/proto/quant_transformer.proto:10-165): the model
configuration (``QuantModelConf``), every clip-max, and the fp32 tensors. Like the
reference loader (lightseq/inference/proto/quant_transformer_weight.cc), the engine
quantises the matrices to int8 on the device when the file is loaded.

Layout::

    magic   8 bytes  b"LS100W\\x01\\x00"
    u32 n_conf   then n_conf   x (u16 len, name, f64 value)
    u32 n_str    then n_str    x (u16 len, name, u16 len, value)
    u32 n_amax   then n_amax   x (u16 len, name, f32 value)
    u32 n_tensor then n_tensor x (u16 len, name, u32 ndim, u64 dims[ndim], u64 offset, u64 nbytes)
    padding to a multiple of 64 bytes, then the fp32 data (each tensor 64-byte aligned;
    offsets are relative to the start of the data section)
"""
from __future__ import annotations

import struct
from typing import Dict, Tuple

import numpy as np

MAGIC = b"LS100W\x01\x00"


def _name(b: str) -> bytes:
    e = b.encode()
    return struct.pack("<H", len(e)) + e


def save(path: str, model: str, conf: Dict[str, float], amax: Dict[str, float], tensors: Dict[str, np.ndarray]):
    head = bytearray(MAGIC)
    head += struct.pack("<I", len(conf))
    for k, v in conf.items():
        head += _name(k) + struct.pack("<d", float(v))
    strs = {"model": model}
    head += struct.pack("<I", len(strs))
    for k, v in strs.items():
        head += _name(k) + _name(v)
    head += struct.pack("<I", len(amax))
    for k, v in amax.items():
        head += _name(k) + struct.pack("<f", float(v))
    head += struct.pack("<I", len(tensors))
    off = 0
    blobs = []
    for k, t in tensors.items():
        t = np.ascontiguousarray(t, dtype=np.float32)
        head += _name(k) + struct.pack("<I", t.ndim) + struct.pack("<%dQ" % t.ndim, *t.shape)
        head += struct.pack("<QQ", off, t.nbytes)
        blobs.append((off, t))
        off += (t.nbytes + 63) // 64 * 64
    pad = (-len(head)) % 64
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * pad)
        pos = 0
        for o, t in blobs:
            if o > pos:
                f.write(b"\0" * (o - pos))
                pos = o
            f.write(t.tobytes())
            pos += t.nbytes
        if off > pos:
            f.write(b"\0" * (off - pos))


def load(path: str) -> Tuple[str, Dict[str, float], Dict[str, float], Dict[str, np.ndarray]]:
    """Returns (model name, conf, amax, tensors)."""
    with open(path, "rb") as f:
        buf = f.read()
    if buf[:8] != MAGIC:
        raise ValueError(f"{path}: not an .ls100 weight file")
    p = 8

    def rd(fmt):
        nonlocal p
        v = struct.unpack_from(fmt, buf, p)
        p += struct.calcsize(fmt)
        return v

    def rd_name():
        nonlocal p
        (n,) = rd("<H")
        s = buf[p:p + n].decode()
        p += n
        return s

    conf, strs, amax, tens = {}, {}, {}, {}
    for _ in range(rd("<I")[0]):
        k = rd_name()
        conf[k] = rd("<d")[0]
    for _ in range(rd("<I")[0]):
        k = rd_name()
        strs[k] = rd_name()
    for _ in range(rd("<I")[0]):
        k = rd_name()
        amax[k] = rd("<f")[0]
    meta = []
    for _ in range(rd("<I")[0]):
        k = rd_name()
        (nd,) = rd("<I")
        dims = rd("<%dQ" % nd)
        off, nb = rd("<QQ")
        meta.append((k, dims, off, nb))
    data0 = (p + 63) // 64 * 64
    for k, dims, off, nb in meta:
        tens[k] = np.frombuffer(buf, dtype=np.float32, count=nb // 4, offset=data0 + off).reshape(dims).copy()
    return strs.get("model", ""), conf, amax, tens
