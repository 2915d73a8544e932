"""The reader / writer of the reference's QuantTransformer protobuf files: wire-format primitives against hand-encoded
bytes, a write -> read round trip that preserves every int8 weight, clip-max, fp32 vector and configuration value,
unpacked repeated floats, and the errors for what the engine cannot run."""
import numpy as np
import pytest

from lightseq_b200 import ls_proto as lp
from lightseq_b200 import synth, weights

F32 = np.float32


def test_wire_format_primitives():
    # field 1 varint 150 (the protobuf documentation's example), field 2 string "testing", field 4 float 1.5
    raw = bytes([0x08, 0x96, 0x01]) + bytes([0x12, 0x07]) + b"testing" + bytes([0x25]) + np.float32(1.5).tobytes()
    m = lp.parse_message(raw)
    assert lp._int(m, 1) == 150 and lp._str(m, 2) == "testing" and lp._float(m, 4) == 1.5
    assert lp._enc_int(1, 150) == raw[:3]
    assert lp._int(lp.parse_message(lp._enc_int(3, -2)), 3) == -2  # negatives: ten-byte sign-extended varint
    assert len(lp._enc_int(3, -2)) == 11
    assert lp._enc_int(5, 0) == b"" and lp._enc_float(5, 0.0) == b""  # proto3 omits defaults
    packed = lp._enc_floats(7, [1.0, -2.5, 3.25])
    assert np.array_equal(lp._floats(lp.parse_message(packed), 7), np.array([1.0, -2.5, 3.25], F32))
    unpacked = b"".join(lp._tag(7, 5) + np.float32(v).tobytes() for v in (1.0, -2.5, 3.25))
    assert np.array_equal(lp._floats(lp.parse_message(unpacked), 7), np.array([1.0, -2.5, 3.25], F32))
    with pytest.raises(ValueError):
        lp.parse_message(bytes([0x12, 0x7F, 0x00]))  # length runs past the end


def test_quantisation_conventions():
    x = np.array([-2.0, -1.0, -0.004, 0.0, 0.0039, 0.5, 1.0, 3.0], F32)
    u = lp._quant_u8(x, 1.0)  # export_quant.quantize
    assert u.tolist() == [0, 0, 126, 127, 127, 191, 254, 254]
    assert np.array_equal(lp._quant_engine(x, 1.0), u)
    back = lp._dequant(u, 1.0)
    assert np.array_equal(lp._quant_engine(back, 1.0), u)  # dequantise -> requantise is the identity on the integers


def _model(tmp_path):
    conf, amax, w = synth.make_transformer(None, hidden=64, heads=1, ffn=128, n_enc=2, n_dec=2, vocab=40, max_step=16, seed=3)
    for i in range(2):
        amax[f"dec.{i}.xv.w"] = amax[f"dec.{i}.xk.w"]  # the file format holds one clip-max for both
    return conf, amax, w


def test_round_trip_preserves_int8_weights_and_everything_else(tmp_path):
    conf, amax, w = _model(tmp_path)
    pb = str(tmp_path / "m.pb")
    lp.write_quant_transformer(pb, conf, amax, w)
    conf2, amax2, w2 = lp.read_quant_transformer(pb)
    for k in conf:
        if k in ("output_topk", "rng_seed"):  # not in the file: the reference's model always returns every beam
            continue
        assert float(conf2[k]) == pytest.approx(float(conf[k]), rel=1e-6), k
    assert conf2["output_topk"] == 1.0
    assert set(amax2) == set(amax)
    for k in amax:
        assert F32(amax2[k]) == F32(amax[k]), k
    assert set(w2) == set(w)
    for k, t in w.items():
        assert w2[k].shape == t.shape, k
        if k.endswith(".w") or k == "emb":  # matrices come back dequantised: the same integers under the same clip-max
            assert np.array_equal(lp._quant_engine(w2[k], amax[k]), lp._quant_engine(t, amax[k])), k
        else:
            assert np.array_equal(w2[k], t.astype(F32)), k
    # a second write of what was read is byte-identical (the reader and the writer agree on every layout)
    pb2 = str(tmp_path / "m2.pb")
    lp.write_quant_transformer(pb2, conf2, amax2, w2)
    assert open(pb, "rb").read() == open(pb2, "rb").read()
    # and the converter produces a container the engine's loader accepts
    out = str(tmp_path / "m.ls100")
    lp.convert(pb, out)
    name, conf3, amax3, w3 = weights.load(out)
    assert name == "QuantTransformer" and int(conf3["n_dec"]) == 2 and w3["dec.1.xv.w"].shape == (64, 64)


def test_layouts_follow_the_reference_exporter(tmp_path):
    """Kernels are stored [in, out]; the target embedding [hidden, vocab]; the cross K/V kernel
    [hidden, n_dec, 2, hidden]."""
    conf, amax, w = _model(tmp_path)
    pb = str(tmp_path / "m.pb")
    lp.write_quant_transformer(pb, conf, amax, w)
    root = lp.parse_message(open(pb, "rb").read())
    enc0 = lp.parse_message(root[2][0][1])
    qkv = lp._bytes(enc0, 3).reshape(64, 192)
    assert np.array_equal(qkv, lp._quant_engine(w["enc.0.qkv.w"], amax["enc.0.qkv.w"]).T)
    trg = lp.parse_message(root[3][0][1])
    assert np.array_equal(lp._bytes(trg, 1).reshape(64, 40), lp._quant_engine(w["emb"], amax["emb"]).T)
    kv = lp._bytes(trg, 5).reshape(64, 2, 2, 64)
    assert np.array_equal(kv[:, 1, 0, :], lp._quant_engine(w["dec.1.xk.w"], amax["dec.1.xk.w"]).T)
    assert lp._floats(trg, 7).size == 40 and not lp._floats(trg, 7).any()
    mc = lp.parse_message(root[5][0][1])
    assert lp._str(mc, 8) == "beam_search" and lp._int(mc, 2) == 4 and lp._int(mc, 11) == 2


def test_rejects_what_the_engine_cannot_run(tmp_path):
    conf, amax, w = _model(tmp_path)
    bad = dict(amax)
    bad["dec.0.xv.w"] = amax["dec.0.xk.w"] * 2
    with pytest.raises(ValueError, match="different clip-max"):
        lp.write_quant_transformer(str(tmp_path / "x.pb"), conf, bad, w)
    with pytest.raises(ValueError, match="not a QuantTransformer"):
        p = tmp_path / "junk.pb"
        p.write_bytes(lp._enc_int(1, 5))
        lp.read_quant_transformer(str(p))


def _no_fc2_out(amax):
    """The encoder-only file formats hold no clip-max for the second FFN output: 0 = not quantised."""
    return {k: (0.0 if k.endswith(".fc2.out") else v) for k, v in amax.items()}


def _same_model(a, b, skip_conf=()):
    (conf, amax, w), (conf2, amax2, w2) = a, b
    for k in conf:
        if k not in skip_conf:
            assert float(conf2[k]) == pytest.approx(float(conf[k]), rel=1e-6), k
    assert set(amax2) == set(amax)
    for k in amax:
        assert F32(amax2[k]) == F32(amax[k]), k
    assert set(w2) == set(w)
    for k, t in w.items():
        assert w2[k].shape == tuple(np.shape(t)), k
        if (k.endswith(".w") and k != "conv.w") or k == "emb":
            assert np.array_equal(lp._quant_engine(w2[k], amax[k]), lp._quant_engine(t, amax[k])), k
        else:
            assert np.array_equal(w2[k], np.asarray(t, F32)), k


def test_quant_bert_file_round_trip(tmp_path):
    conf, amax, w = synth.make_bert(None, hidden=64, heads=1, ffn=128, n_layer=2, vocab=50, max_step=24, seed=2)
    w["emb"] = (w["emb"] + w["type_emb"][0]).astype(F32)  # the file holds one table
    w["type_emb"] = np.zeros_like(w["type_emb"])
    amax = _no_fc2_out(amax)
    pb = str(tmp_path / "bert.pb")
    lp.write_quant_bert(pb, conf, amax, w)
    _same_model((conf, amax, w), lp.read_quant_bert(pb))
    with pytest.raises(ValueError, match="second FFN"):
        lp.write_quant_bert(pb, conf, dict(amax, **{"enc.0.fc2.out": 1.0}), w)


def test_quant_gpt_file_round_trip(tmp_path):
    conf, amax, w = synth.make_gpt(None, hidden=64, heads=1, ffn=128, n_layer=2, vocab=60, max_step=32, max_new_tokens=9, topk=4)
    amax = _no_fc2_out(amax)
    pb = str(tmp_path / "gpt.pb")
    lp.write_quant_gpt(pb, conf, amax, w)
    got = lp.read_quant_gpt(pb)
    _same_model((conf, amax, w), got, skip_conf=("rng_seed",))  # the seed is not part of the file
    assert int(got[0]["topk"]) == 4 and float(got[0]["topp"]) == 0.0 and int(got[0]["max_new_tokens"]) == 9
    conf_p = dict(conf, topp=0.75)
    lp.write_quant_gpt(pb, conf_p, amax, w)
    c = lp.read_quant_gpt(pb)[0]
    assert float(c["topp"]) == pytest.approx(0.75) and int(c["topk"]) == 1


def test_quant_vit_file_round_trip(tmp_path):
    conf, amax, w = synth.make_vit(None, hidden=64, heads=1, ffn=128, n_layer=2, image=16, patch=4, seed=4)
    amax = _no_fc2_out(amax)
    pb = str(tmp_path / "vit.pb")
    lp.write_quant_vit(pb, conf, amax, w)
    _same_model((conf, amax, w), lp.read_quant_vit(pb))


def test_convert_names_the_model_class(tmp_path):
    conf, amax, w = synth.make_vit(None, hidden=64, heads=1, ffn=128, n_layer=1, image=8, patch=4, seed=4)
    pb, out = str(tmp_path / "vit.pb"), str(tmp_path / "vit.ls100")
    lp.write_quant_vit(pb, conf, _no_fc2_out(amax), w)
    lp.convert(pb, out, "QuantVit")
    model, conf2, amax2, _ = weights.load(out)
    assert model == "QuantVit" and int(conf2["patch_size"]) == 4 and amax2["enc.0.fc2.out"] == 0.0
    with pytest.raises(ValueError, match="one of"):
        lp.convert(pb, out, "QuantLlama")
