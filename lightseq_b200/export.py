"""Exporter: a Fairseq Transformer trained with the reference's torch fake-quant layers -> the reference's
``QuantTransformer`` protobuf file (and from there, through ``ls_proto.convert``, the engine's own container).

Restates the name mapping of examples/inference/python/export/fairseq/ls_torch_fs_quant_transformer_export.py:20-131
(which checkpoint tensor feeds which proto field) and the conventions of lightseq/training/ops/pytorch/export_quant.py:12-19
(uint8 = q + 127). Checkpoint keys are those of the modules in lightseq/training/ops/pytorch/torch_transformer_layers.py and
quantization.py:

    {encoder|decoder}.layers.<i>.<block>.<proj>.weight                      [out, in]
    {encoder|decoder}.layers.<i>.<block>.<proj>.bias                        [out]
    ....<proj>.weight_quant._amax                                           clip-max of the weight quantiser
    ....<proj>.input_quant.clip.clip_value_max                              learned clip-max of the input quantiser
    ....<proj>.output_quant._amax                                           clip-max of the output quantiser
    decoder.layers.<i>.self_attn.attention_quant._amax                      clip-max of the cached K/V (decoder)
    {encoder|decoder}.layers.<i>.{self_attn_layer_norm|encoder_attn_layer_norm|final_layer_norm}.{weight|bias}
    {encoder|decoder}.layer_norm.{weight|bias}                              final LayerNorm of each stack (pre-LN)
    {encoder|decoder}.embed_tokens.emb_lookup.weight                        [vocab, hidden]
    {encoder|decoder}.embed_tokens.emb_quant.clip.clip_value_max
    {encoder|decoder}.embed_tokens.embed_positions.weight                   optional; sinusoids otherwise
    decoder.output_projection.input_quant.clip.clip_value_max, decoder.output_projection.output_quant._amax

with <block>.<proj> in self_attn.{qkv_proj,out_proj}, encoder_attn.{q_proj,k_proj,v_proj,out_proj}, fc1, fc2.
Values may be numpy arrays, python floats or torch tensors. ``engine_to_state_dict`` is the inverse map (used by the
tests, and to hand an engine model back to the torch layers).
"""
from __future__ import annotations

import sys
from typing import Dict, Mapping, Tuple

import numpy as np

from . import ls_proto
from .synth import sinusoid_table

F32 = np.float32

# engine projection name -> checkpoint module path inside a layer
_ENC_PROJ = {"qkv": "self_attn.qkv_proj", "out": "self_attn.out_proj", "fc1": "fc1", "fc2": "fc2"}
_DEC_PROJ = {"qkv": "self_attn.qkv_proj", "out": "self_attn.out_proj", "xq": "encoder_attn.q_proj", "xout": "encoder_attn.out_proj",
             "fc1": "fc1", "fc2": "fc2"}
_ENC_LN = {"ln1": "self_attn_layer_norm", "ln2": "final_layer_norm"}
_DEC_LN = {"ln1": "self_attn_layer_norm", "ln2": "encoder_attn_layer_norm", "ln3": "final_layer_norm"}


def _np(v) -> np.ndarray:
    if hasattr(v, "detach"):
        v = v.detach().cpu().numpy()
    return np.asarray(v, dtype=F32)


def _scalar(state: Mapping[str, object], key: str) -> float:
    if key not in state:
        raise KeyError(f"checkpoint has no {key!r} (is this a model trained with the fake-quant layers?)")
    a = _np(state[key]).reshape(-1)
    if a.size != 1:
        raise ValueError(f"{key}: expected one value (per-tensor quantisation), got {a.size}")
    v = float(a[0])
    if not v > 0.0:
        raise ValueError(f"{key}: clip-max must be positive, got {v}")
    return v


def _tensor(state: Mapping[str, object], key: str, shape=None) -> np.ndarray:
    if key not in state:
        raise KeyError(f"checkpoint has no {key!r}")
    a = np.ascontiguousarray(_np(state[key]))
    if shape is not None and tuple(a.shape) != tuple(shape):
        raise ValueError(f"{key}: shape {tuple(a.shape)}, expected {tuple(shape)}")
    return a


def _count_layers(state: Mapping[str, object], side: str) -> int:
    ids = set()
    for k in state:
        p = k.split(".")
        if len(p) > 3 and p[0] == side and p[1] == "layers" and p[2].isdigit():
            ids.add(int(p[2]))
    if ids != set(range(len(ids))):
        raise ValueError(f"{side}.layers: indices {sorted(ids)} are not 0..n-1")
    return len(ids)


def _take_proj(state, base: str, eng: str, amax: Dict[str, float], t: Dict[str, np.ndarray], want_out: bool = True) -> None:
    t[f"{eng}.w"] = _tensor(state, f"{base}.weight")
    t[f"{eng}.b"] = _tensor(state, f"{base}.bias", (t[f"{eng}.w"].shape[0],))
    amax[f"{eng}.w"] = _scalar(state, f"{base}.weight_quant._amax")
    amax[f"{eng}.in"] = _scalar(state, f"{base}.input_quant.clip.clip_value_max")
    if want_out:
        amax[f"{eng}.out"] = _scalar(state, f"{base}.output_quant._amax")


def state_dict_to_engine(state: Mapping[str, object], *, heads: int, beam: int = 4, length_penalty: float = 0.6,
                         extra_decode_length: int = 50, max_step: int = 300, pad_id: int = 1, bos_id: int = 2, eos_id: int = 2,
                         activation: str = "relu") -> Tuple[dict, Dict[str, float], Dict[str, np.ndarray]]:
    """Checkpoint ``state`` (the ``"model"`` dict of a Fairseq checkpoint) -> the engine's (conf, amax, tensors). The
    defaults of the generation settings are the reference exporter's (max_step 300, bos = eos = 2, pad 1)."""
    amax: Dict[str, float] = {}
    t: Dict[str, np.ndarray] = {}
    emb = _tensor(state, "encoder.embed_tokens.emb_lookup.weight")
    V, H = emb.shape
    trg = _tensor(state, "decoder.embed_tokens.emb_lookup.weight", (V, H))
    c_src = _scalar(state, "encoder.embed_tokens.emb_quant.clip.clip_value_max")
    c_trg = _scalar(state, "decoder.embed_tokens.emb_quant.clip.clip_value_max")
    if not np.array_equal(emb, trg) or F32(c_src) != F32(c_trg):
        raise ValueError("source and target embeddings differ: the engine shares one table (train with --share-all-embeddings)")
    if H % heads or (H // heads) != 64:
        raise ValueError(f"hidden {H} / heads {heads}: the engine's attention kernels are built for a head size of 64")
    t["emb"], amax["emb"] = emb, c_src
    pos_key = "encoder.embed_tokens.embed_positions.weight"
    if pos_key in state:
        t["pos"] = _tensor(state, pos_key)
        if t["pos"].shape[1] != H:
            raise ValueError(f"{pos_key}: width {t['pos'].shape[1]}, expected {H}")
        max_step = t["pos"].shape[0]
    else:
        t["pos"] = sinusoid_table(max_step, H)
    t["enc.ln.g"], t["enc.ln.b"] = _tensor(state, "encoder.layer_norm.weight", (H,)), _tensor(state, "encoder.layer_norm.bias", (H,))
    t["dec.ln.g"], t["dec.ln.b"] = _tensor(state, "decoder.layer_norm.weight", (H,)), _tensor(state, "decoder.layer_norm.bias", (H,))
    amax["logits.in"] = _scalar(state, "decoder.output_projection.input_quant.clip.clip_value_max")
    amax["logits.out"] = _scalar(state, "decoder.output_projection.output_quant._amax")
    n_enc, n_dec = _count_layers(state, "encoder"), _count_layers(state, "decoder")
    ffn = None
    for i in range(n_enc):
        for ln, mod in _ENC_LN.items():
            t[f"enc.{i}.{ln}.g"] = _tensor(state, f"encoder.layers.{i}.{mod}.weight", (H,))
            t[f"enc.{i}.{ln}.b"] = _tensor(state, f"encoder.layers.{i}.{mod}.bias", (H,))
        for eng, mod in _ENC_PROJ.items():
            _take_proj(state, f"encoder.layers.{i}.{mod}", f"enc.{i}.{eng}", amax, t)
        ffn = t[f"enc.{i}.fc1.w"].shape[0] if ffn is None else ffn
    for i in range(n_dec):
        for ln, mod in _DEC_LN.items():
            t[f"dec.{i}.{ln}.g"] = _tensor(state, f"decoder.layers.{i}.{mod}.weight", (H,))
            t[f"dec.{i}.{ln}.b"] = _tensor(state, f"decoder.layers.{i}.{mod}.bias", (H,))
        for eng, mod in _DEC_PROJ.items():
            _take_proj(state, f"decoder.layers.{i}.{mod}", f"dec.{i}.{eng}", amax, t)
        amax[f"dec.{i}.kv"] = _scalar(state, f"decoder.layers.{i}.self_attn.attention_quant._amax")
        # cross-attention K and V read the encoder output unquantised (weight-only fake-quant); the file keeps ONE
        # clip-max per layer for both matrices, the k_proj one (exporter: _get_encode_output_mapping_dict)
        ck = _scalar(state, f"decoder.layers.{i}.encoder_attn.k_proj.weight_quant._amax")
        for eng, mod in (("xk", "k_proj"), ("xv", "v_proj")):
            t[f"dec.{i}.{eng}.w"] = _tensor(state, f"decoder.layers.{i}.encoder_attn.{mod}.weight", (H, H))
            t[f"dec.{i}.{eng}.b"] = _tensor(state, f"decoder.layers.{i}.encoder_attn.{mod}.bias", (H,))
            amax[f"dec.{i}.{eng}.w"] = ck
        ffn = t[f"dec.{i}.fc1.w"].shape[0] if ffn is None else ffn
    if activation not in ("relu", "gelu"):
        raise ValueError(f"activation {activation!r}: relu or gelu")
    conf = dict(hidden=H, heads=int(heads), ffn=int(ffn or 0), n_enc=n_enc, n_dec=n_dec, vocab=V,
                act_gelu=1.0 if activation == "gelu" else 0.0, pre_ln=1.0, beam=int(beam), length_penalty=float(length_penalty),
                extra_decode_length=int(extra_decode_length), max_step=int(max_step), pad_id=int(pad_id), start_id=int(bos_id),
                end_id=int(eos_id))
    return conf, amax, t


def engine_to_state_dict(conf, amax: Mapping[str, float], t: Mapping[str, np.ndarray]) -> Dict[str, np.ndarray]:
    """The inverse map: the engine's tensors and clip-max values under the checkpoint's key names."""
    s: Dict[str, np.ndarray] = {}

    def one(v):
        return np.array([v], dtype=F32)

    def put_proj(base, eng, want_out=True):
        s[f"{base}.weight"], s[f"{base}.bias"] = np.asarray(t[f"{eng}.w"], F32), np.asarray(t[f"{eng}.b"], F32)
        s[f"{base}.weight_quant._amax"] = one(amax[f"{eng}.w"])
        if f"{eng}.in" in amax:
            s[f"{base}.input_quant.clip.clip_value_max"] = one(amax[f"{eng}.in"])
        if want_out and f"{eng}.out" in amax:
            s[f"{base}.output_quant._amax"] = one(amax[f"{eng}.out"])

    for side in ("encoder", "decoder"):
        s[f"{side}.embed_tokens.emb_lookup.weight"] = np.asarray(t["emb"], F32)
        s[f"{side}.embed_tokens.emb_quant.clip.clip_value_max"] = one(amax["emb"])
        s[f"{side}.embed_tokens.embed_positions.weight"] = np.asarray(t["pos"], F32)
    s["encoder.layer_norm.weight"], s["encoder.layer_norm.bias"] = t["enc.ln.g"], t["enc.ln.b"]
    s["decoder.layer_norm.weight"], s["decoder.layer_norm.bias"] = t["dec.ln.g"], t["dec.ln.b"]
    s["decoder.output_projection.input_quant.clip.clip_value_max"] = one(amax["logits.in"])
    s["decoder.output_projection.output_quant._amax"] = one(amax["logits.out"])
    for i in range(int(conf["n_enc"])):
        for ln, mod in _ENC_LN.items():
            s[f"encoder.layers.{i}.{mod}.weight"], s[f"encoder.layers.{i}.{mod}.bias"] = t[f"enc.{i}.{ln}.g"], t[f"enc.{i}.{ln}.b"]
        for eng, mod in _ENC_PROJ.items():
            put_proj(f"encoder.layers.{i}.{mod}", f"enc.{i}.{eng}")
    for i in range(int(conf["n_dec"])):
        for ln, mod in _DEC_LN.items():
            s[f"decoder.layers.{i}.{mod}.weight"], s[f"decoder.layers.{i}.{mod}.bias"] = t[f"dec.{i}.{ln}.g"], t[f"dec.{i}.{ln}.b"]
        for eng, mod in _DEC_PROJ.items():
            put_proj(f"decoder.layers.{i}.{mod}", f"dec.{i}.{eng}")
        s[f"decoder.layers.{i}.self_attn.attention_quant._amax"] = one(amax[f"dec.{i}.kv"])
        for eng, mod in (("xk", "k_proj"), ("xv", "v_proj")):
            put_proj(f"decoder.layers.{i}.encoder_attn.{mod}", f"dec.{i}.{eng}", want_out=False)
    return s


def export_quant_transformer(state: Mapping[str, object], pb_path: str, **generation) -> dict:
    """Writes the QuantTransformer protobuf file for ``state``; returns the model configuration that went into it."""
    conf, amax, t = state_dict_to_engine(state, **generation)
    ls_proto.write_quant_transformer(pb_path, conf, amax, t)
    return conf


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(description="Fairseq checkpoint (fake-quant torch layers) -> QuantTransformer protobuf file")
    ap.add_argument("checkpoint", help="checkpoint_best.pt: a dict with 'model' (state dict) and 'args'")
    ap.add_argument("output", help="path of the .pb file to write")
    ap.add_argument("--beam", type=int, default=4)
    ap.add_argument("--length-penalty", type=float, default=0.6)
    ap.add_argument("--extra-decode-length", type=int, default=50)
    ap.add_argument("--max-step", type=int, default=300)
    ap.add_argument("--bos-id", type=int, default=2)
    ap.add_argument("--eos-id", type=int, default=2)
    ap.add_argument("--pad-id", type=int, default=1)
    a = ap.parse_args(argv)
    import torch

    # a Fairseq checkpoint pickles its argparse Namespace beside the tensors, hence the full unpickler: only load files you trust
    ck = torch.load(a.checkpoint, map_location="cpu", weights_only=False)
    args = ck.get("args")
    heads = int(getattr(args, "encoder_attention_heads"))
    act = str(getattr(args, "activation_fn", "relu"))
    conf = export_quant_transformer(ck["model"], a.output, heads=heads, beam=a.beam, length_penalty=a.length_penalty,
                                    extra_decode_length=a.extra_decode_length, max_step=a.max_step, pad_id=a.pad_id,
                                    bos_id=a.bos_id, eos_id=a.eos_id, activation=act)
    print("wrote", a.output, conf)
    return 0


if __name__ == "__main__":
    sys.exit(main())
