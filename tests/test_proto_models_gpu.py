"""Models in the reference's QuantBert / QuantGpt / QuantVit protobuf file formats, converted and run: the engine on the
converted file against the numpy oracle on the tensors read back from the same file. These formats hold no clip-max
for the second FFN output, so that output stays unquantised in both (a clip-max of 0)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from lightseq_b200 import ls_proto as lp  # noqa: E402
from lightseq_b200 import synth  # noqa: E402
from oracle import model as om  # noqa: E402

F32 = np.float32


def _no_fc2_out(amax):
    return {k: (0.0 if k.endswith(".fc2.out") else v) for k, v in amax.items()}


def test_quant_bert_protobuf_file(tmp_path):
    import lightseq_b200.inference as lsi

    conf, amax, w = synth.make_bert(None, hidden=128, heads=2, ffn=256, n_layer=2, vocab=400, max_step=32, seed=21)
    w["emb"] = (w["emb"] + w["type_emb"][0]).astype(F32)
    w["type_emb"] = np.zeros_like(w["type_emb"])
    pb, path = str(tmp_path / "bert.pb"), str(tmp_path / "bert.ls100")
    lp.write_quant_bert(pb, conf, _no_fc2_out(amax), w)
    lp.convert(pb, path, "QuantBert")
    conf2, amax2, w2 = lp.read_quant_bert(pb)
    cfg = om.Config(hidden=128, heads=2, ffn=256, n_enc=2, n_dec=0, vocab=400, act="gelu", pre_ln=False, pad_id=int(conf2["pad_id"]))
    ids = synth.bert_inputs(batch=4, seq=21, vocab=400, pad_id=int(conf2["pad_id"]), seed=6)
    ref = om.Bert(cfg, om.State(w=w2, amax=amax2)).forward(ids)
    out = lsi.QuantBert(path, 4).infer(ids)
    d = np.abs(out - ref)[ids != int(conf2["pad_id"])]
    print("bert (protobuf file) max abs", d.max(), "mean abs", d.mean())
    assert d.max() < 6e-2 and d.mean() < 5e-3


def test_quant_vit_protobuf_file(tmp_path):
    import lightseq_b200.inference as lsi

    conf, amax, w = synth.make_vit(None, hidden=128, heads=2, ffn=256, n_layer=2, image=32, patch=8, seed=22)
    pb, path = str(tmp_path / "vit.pb"), str(tmp_path / "vit.ls100")
    lp.write_quant_vit(pb, conf, _no_fc2_out(amax), w)
    lp.convert(pb, path, "QuantVit")
    conf2, amax2, w2 = lp.read_quant_vit(pb)
    cfg = om.Config(hidden=128, heads=2, ffn=256, n_enc=2, n_dec=0, act="gelu", pre_ln=True)
    px = synth.vit_inputs(batch=3, image=32, seed=8)
    ref = om.Vit(cfg, om.State(w=w2, amax=amax2), 8).forward(px)
    out = lsi.QuantVit(path, 3).infer(px)
    d = np.abs(out - ref)
    print("vit (protobuf file) max abs", d.max(), "mean abs", d.mean())
    assert d.max() < 6e-2 and d.mean() < 5e-3


def test_quant_gpt_protobuf_file(tmp_path):
    import lightseq_b200.inference as lsi

    conf, amax, w = synth.make_gpt(None, hidden=128, heads=2, ffn=256, n_layer=2, vocab=300, max_step=40, end_id=299, topk=8,
                                   max_new_tokens=20, seed=23, rng_seed=2024)
    pb, path = str(tmp_path / "gpt.pb"), str(tmp_path / "gpt.ls100")
    lp.write_quant_gpt(pb, conf, _no_fc2_out(amax), w)
    lp.convert(pb, path, "QuantGpt")
    conf2, amax2, w2 = lp.read_quant_gpt(pb)
    cfg = om.Config(hidden=128, heads=2, ffn=256, n_enc=0, n_dec=2, vocab=300, act="gelu", pre_ln=True, max_step=40, end_id=299)
    ids = synth.gpt_inputs(batch=5, prompt=7, vocab=300, seed=2)
    ref = om.Gpt(cfg, om.State(w=w2, amax=amax2)).generate(ids, 20, 8, 2024, 0)  # the engine's default seed: none is in the file
    out = lsi.QuantGpt(path, 8).sample(ids)
    assert out.shape == ref.shape, (out.shape, ref.shape)
    same = (out == ref).all(axis=1)
    print("gpt (protobuf file) identical sequences", int(same.sum()), "of", len(same))
    assert same.all()
