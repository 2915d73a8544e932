"""The exporter from a Fairseq checkpoint of the reference's fake-quant torch layers to the QuantTransformer
protobuf file: key mapping both ways, the file it writes read back into the engine's tensors, and its errors."""
import numpy as np
import pytest

from lightseq_b200 import export as ex
from lightseq_b200 import ls_proto as lp
from lightseq_b200 import synth

F32 = np.float32


def _model():
    conf, amax, w = synth.make_transformer(None, hidden=64, heads=1, ffn=128, n_enc=2, n_dec=3, vocab=40, max_step=16, seed=5)
    for i in range(3):
        amax[f"dec.{i}.xv.w"] = amax[f"dec.{i}.xk.w"]  # the checkpoint format keeps k_proj's clip-max for both
    return conf, amax, w


def _gen(conf):
    return dict(heads=int(conf["heads"]), beam=int(conf["beam"]), length_penalty=float(conf["length_penalty"]),
                extra_decode_length=int(conf["extra_decode_length"]), max_step=int(conf["max_step"]), pad_id=int(conf["pad_id"]),
                bos_id=int(conf["start_id"]), eos_id=int(conf["end_id"]))


def test_key_names_follow_the_torch_layers():
    conf, amax, w = _model()
    s = ex.engine_to_state_dict(conf, amax, w)
    for k in ("encoder.layers.1.self_attn.qkv_proj.weight", "encoder.layers.0.self_attn.qkv_proj.weight_quant._amax",
              "encoder.layers.0.fc2.input_quant.clip.clip_value_max", "encoder.layers.0.fc1.output_quant._amax",
              "decoder.layers.2.encoder_attn.q_proj.bias", "decoder.layers.0.encoder_attn.k_proj.weight_quant._amax",
              "decoder.layers.1.self_attn.attention_quant._amax", "decoder.layers.0.encoder_attn_layer_norm.weight",
              "decoder.layers.0.final_layer_norm.bias", "encoder.embed_tokens.emb_lookup.weight",
              "decoder.embed_tokens.emb_quant.clip.clip_value_max", "decoder.output_projection.output_quant._amax",
              "encoder.layer_norm.weight"):
        assert k in s, k
    assert s["encoder.layers.0.self_attn.qkv_proj.weight"].shape == (192, 64)  # torch layout [out, in]
    assert "decoder.layers.0.encoder_attn.k_proj.output_quant._amax" not in s  # weight-only fake-quant


def test_state_dict_round_trip_is_exact():
    conf, amax, w = _model()
    s = ex.engine_to_state_dict(conf, amax, w)
    conf2, amax2, w2 = ex.state_dict_to_engine(s, **_gen(conf))
    assert {k: float(v) for k, v in conf2.items()} == {k: float(conf[k]) for k in conf2}
    assert set(amax2) == set(amax) and all(F32(amax2[k]) == F32(amax[k]) for k in amax)
    assert set(w2) == set(w) and all(np.array_equal(w2[k], w[k]) for k in w)


def test_exported_file_reads_back_as_the_same_int8_model(tmp_path):
    conf, amax, w = _model()
    s = ex.engine_to_state_dict(conf, amax, w)
    pb = str(tmp_path / "m.pb")
    ex.export_quant_transformer(s, pb, **_gen(conf))
    conf2, amax2, w2 = lp.read_quant_transformer(pb)
    assert int(conf2["n_enc"]) == 2 and int(conf2["n_dec"]) == 3 and int(conf2["vocab"]) == 40 and int(conf2["ffn"]) == 128
    for k in amax:
        assert F32(amax2[k]) == F32(amax[k]), k
    for k, t in w.items():
        if k.endswith(".w") or k == "emb":
            assert np.array_equal(lp._quant_engine(w2[k], amax[k]), lp._quant_engine(t, amax[k])), k
        else:
            assert np.array_equal(w2[k], np.asarray(t, F32)), k


def test_sinusoids_when_the_checkpoint_has_no_position_table():
    conf, amax, w = _model()
    s = ex.engine_to_state_dict(conf, amax, w)
    del s["encoder.embed_tokens.embed_positions.weight"], s["decoder.embed_tokens.embed_positions.weight"]
    g = _gen(conf)
    g["max_step"] = 24
    conf2, _, w2 = ex.state_dict_to_engine(s, **g)
    assert int(conf2["max_step"]) == 24 and np.array_equal(w2["pos"], synth.sinusoid_table(24, 64))


def test_torch_tensors_are_accepted():
    torch = pytest.importorskip("torch")
    conf, amax, w = _model()
    s = {k: torch.from_numpy(np.ascontiguousarray(np.asarray(v, F32))) for k, v in ex.engine_to_state_dict(conf, amax, w).items()}
    _, amax2, w2 = ex.state_dict_to_engine(s, **_gen(conf))
    assert np.array_equal(w2["dec.1.fc2.w"], w["dec.1.fc2.w"]) and F32(amax2["dec.1.kv"]) == F32(amax["dec.1.kv"])


def test_errors():
    conf, amax, w = _model()
    s = ex.engine_to_state_dict(conf, amax, w)
    g = _gen(conf)
    bad = dict(s)
    del bad["encoder.layers.0.fc1.weight_quant._amax"]
    with pytest.raises(KeyError, match="fake-quant"):
        ex.state_dict_to_engine(bad, **g)
    bad = dict(s)
    bad["decoder.embed_tokens.emb_lookup.weight"] = s["decoder.embed_tokens.emb_lookup.weight"] + 1
    with pytest.raises(ValueError, match="share"):
        ex.state_dict_to_engine(bad, **g)
    bad = dict(s)
    bad["encoder.layers.0.fc1.output_quant._amax"] = np.array([0.5, 0.5], F32)
    with pytest.raises(ValueError, match="per-tensor"):
        ex.state_dict_to_engine(bad, **g)
    bad = {k: v for k, v in s.items() if not k.startswith("encoder.layers.0.")}
    with pytest.raises(ValueError, match="0..n-1"):
        ex.state_dict_to_engine(bad, **g)
    g2 = dict(g)
    g2["heads"] = 2
    with pytest.raises(ValueError, match="head size"):
        ex.state_dict_to_engine(s, **g2)


def test_checkpoint_with_the_reference_layers_own_keys():
    """A checkpoint assembled from the key names and shapes of the reference's torch layers themselves
    (tests/golden/torch_layer_state_keys.json, written by tests/golden/gen_state_keys.py from the real modules) under
    the Fairseq wrapper's prefixes: every tensor the exporter wants is found, the extra buffers are ignored."""
    import json
    import pathlib

    keys = json.loads((pathlib.Path(__file__).parent / "golden" / "torch_layer_state_keys.json").read_text())
    r = np.random.default_rng(11)

    def val(name, shape):
        if name.endswith("_amax") or name.endswith("clip_value_max"):
            return np.asarray(r.uniform(0.5, 4.0), F32).reshape(shape)
        return r.standard_normal(shape).astype(F32) * F32(0.05)

    s = {}
    for i in range(2):
        for k, shp in keys["encoder_layer"].items():
            s[f"encoder.layers.{i}.{k}"] = val(k, shp)
        for k, shp in keys["decoder_layer"].items():
            s[f"decoder.layers.{i}.{k}"] = val(k, shp)
    for k, shp in keys["embedding"].items():
        s[f"encoder.embed_tokens.{k}"] = val(k, shp)
        s[f"decoder.embed_tokens.{k}"] = s[f"encoder.embed_tokens.{k}"]  # shared embeddings
    for side in ("encoder", "decoder"):
        s[f"{side}.layer_norm.weight"], s[f"{side}.layer_norm.bias"] = np.ones(64, F32), np.zeros(64, F32)
    s["decoder.output_projection.input_quant.clip.clip_value_max"] = np.asarray(2.0, F32)
    s["decoder.output_projection.output_quant._amax"] = np.asarray(9.0, F32)
    conf, amax, t = ex.state_dict_to_engine(s, heads=1)
    assert (int(conf["hidden"]), int(conf["ffn"]), int(conf["vocab"]), int(conf["n_enc"]), int(conf["n_dec"])) == (64, 128, 40, 2, 2)
    assert int(conf["max_step"]) == 300 and int(conf["start_id"]) == 2 and int(conf["end_id"]) == 2 and int(conf["pad_id"]) == 1
    assert t["enc.1.qkv.w"].shape == (192, 64) and t["dec.0.xk.w"].shape == (64, 64) and t["pos"].shape == (300, 64)
    assert F32(amax["dec.1.kv"]) == s["decoder.layers.1.self_attn.attention_quant._amax"].reshape(-1)[0]
    assert F32(amax["dec.0.xv.w"]) == s["decoder.layers.0.encoder_attn.k_proj.weight_quant._amax"].reshape(-1)[0]
    assert F32(amax["enc.0.fc2.out"]) == s["encoder.layers.0.fc2.output_quant._amax"].reshape(-1)[0]
    wanted = {k for k in ex.engine_to_state_dict(conf, amax, t) if "embed_positions" not in k}
    assert wanted <= set(s), sorted(wanted - set(s))[:5]
