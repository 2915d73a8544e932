"""QuantGpt engine (pybind surface) vs the numpy oracle: GPT-2 layout, int8 KV cache, top-k sampling with the
seeded per-sequence Philox stream. Small model: every sampled sequence identical. GPT-2-medium width: the engine's
sequences are replayed through the oracle token by token (teacher forcing with the ENGINE's tokens) and every
sampled token must be the one the oracle draws from its own logits for that history; a mismatch is allowed only
on a small fraction of tokens (an int8 logit flip moving a cumulative-probability boundary across u)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from lightseq_b200 import synth  # noqa: E402
from oracle import beam as ob  # noqa: E402
from oracle import model as om  # noqa: E402


def _cfg(conf):
    return om.Config(hidden=int(conf["hidden"]), heads=int(conf["heads"]), ffn=int(conf["ffn"]), n_enc=0,
                     n_dec=int(conf["n_dec"]), vocab=int(conf["vocab"]), act="gelu", pre_ln=True,
                     max_step=int(conf["max_step"]), end_id=int(conf["end_id"]))


@pytest.mark.parametrize("prompt", [7, 19])  # 19: the prompt pass takes the tensor-core attention kernel
def test_small_gpt_sampled_sequences_match_oracle(tmp_path, prompt):
    import lightseq_b200.inference as lsi

    path = str(tmp_path / "gpt.ls100")
    conf, amax, w = synth.make_gpt(path, hidden=128, heads=2, ffn=256, n_layer=2, vocab=300, max_step=40, end_id=299,
                                   topk=8, max_new_tokens=20, seed=5, rng_seed=77)
    cfg = _cfg(conf)
    ids = synth.gpt_inputs(batch=5, prompt=prompt, vocab=300, seed=2)
    ref = om.Gpt(cfg, om.State(w=w, amax=amax)).generate(ids, 20, 8, 77, 0)
    model = lsi.QuantGpt(path, 8)
    out = model.sample(ids)
    assert out.shape == ref.shape, (out.shape, ref.shape)
    assert np.array_equal(out[:, :prompt], ids)
    same = (out == ref).all(axis=1)
    print("identical sequences", int(same.sum()), "of", len(same))
    # the longer prompt has 5 x 19 x 128 x 2 attention outputs, each of which either attention kernel (tensor-core or
    # SIMT: both give 4 of 5 here) may round one int8 step away from the oracle with probability ~1e-5; one such flip
    # can move a sampled token across a cumulative-probability boundary and the sequence then continues differently
    assert same.all() if prompt == 7 else same.sum() >= len(same) - 1
    assert np.array_equal(out, model.sample(ids))  # same seed, same counters -> same draw
    with pytest.raises(RuntimeError, match="max_batch_size"):
        model.sample(np.zeros((9, 4), np.int32))


def test_gpt_medium_width_teacher_forced(tmp_path):
    import lightseq_b200.inference as lsi

    path = str(tmp_path / "gpt.ls100")
    conf, amax, w = synth.make_gpt(path, hidden=1024, heads=16, ffn=4096, n_layer=3, vocab=5000, max_step=48, end_id=4999,
                                   topk=8, max_new_tokens=16, seed=11, rng_seed=2024)
    cfg = _cfg(conf)
    ids = synth.gpt_inputs(batch=6, prompt=12, vocab=5000, seed=3)
    model = lsi.QuantGpt(path, 6)
    out = model.sample(ids)
    B, P = ids.shape
    assert out.shape == (B, P + 16) and np.array_equal(out[:, :P], ids)
    m = om.Gpt(cfg, om.State(w=w, amax=amax))
    caches = [dict() for _ in range(cfg.n_dec)]
    h = m.forward(ids, 0, caches)[:, -1]
    total = match = 0
    for pos in range(P, out.shape[1]):
        lq, s_l = m.logits(h)
        for b in range(B):
            want = cfg.end_id if out[b, pos - 1] == cfg.end_id else ob.sample_topk_row(lq[b], s_l, 8, pos, b, 2024, 0)
            total += 1
            match += int(want == out[b, pos])
        if pos + 1 < out.shape[1]:
            h = m.forward(out[:, pos:pos + 1].astype(np.int64), pos, caches)[:, 0]
    print("teacher-forced token agreement", match, "of", total)
    assert match / total >= 0.95


def test_small_gpt_nucleus_sampling_matches_oracle(tmp_path):
    """topp > 0 in the weight file selects nucleus sampling (sampling_method "topp" of the reference)."""
    import lightseq_b200.inference as lsi

    path = str(tmp_path / "gpt.ls100")
    conf, amax, w = synth.make_gpt(path, hidden=128, heads=2, ffn=256, n_layer=2, vocab=300, max_step=40, end_id=299,
                                   topk=1, topp=0.6, max_new_tokens=20, seed=5, rng_seed=78)
    cfg = _cfg(conf)
    ids = synth.gpt_inputs(batch=5, prompt=7, vocab=300, seed=2)
    ref = om.Gpt(cfg, om.State(w=w, amax=amax)).generate(ids, 20, 1, 78, 0, topp=0.6)
    out = lsi.QuantGpt(path, 8).sample(ids)
    assert out.shape == ref.shape, (out.shape, ref.shape)
    same = (out == ref).all(axis=1)
    print("identical sequences", int(same.sum()), "of", len(same))
    assert same.all()
    assert len(set(out[:, 7:].ravel().tolist())) > 20  # a nucleus of 60 % of a flat distribution is wide


def test_gpt_ppl_matches_oracle(tmp_path):
    """QuantGpt.ppl: mean next-token negative log-likelihood per sequence from the int8 logits of every position;
    right-padded sequences count only their own tokens. fp32 device sums vs the float64 oracle: 1e-5 relative."""
    import lightseq_b200.inference as lsi

    path = str(tmp_path / "gpt.ls100")
    pad = 298
    conf, amax, w = synth.make_gpt(path, hidden=128, heads=2, ffn=256, n_layer=2, vocab=300, max_step=40, end_id=299,
                                   pad_id=pad, topk=4, max_new_tokens=8, seed=5)
    cfg = _cfg(conf)
    r = np.random.default_rng(4)
    ids = r.integers(0, 298, size=(6, 23)).astype(np.int32)
    lens = [23, 2, 1, 10, 17, 22]
    for b, n in enumerate(lens):
        ids[b, n:] = pad
    ref = om.Gpt(cfg, om.State(w=w, amax=amax)).ppl(ids, pad)
    model = lsi.QuantGpt(path, 8)
    out = model.ppl(ids)
    assert out.shape == (6,) and out.dtype == np.float32
    print("ppl", out, "ref", ref)
    assert out[2] == 0.0
    np.testing.assert_allclose(out, ref, rtol=2e-5, atol=1e-6)
    assert 4.0 < out[0] < 7.0  # about log(300) for an untrained model
    np.testing.assert_array_equal(out, model.ppl(ids))  # fixed summation order
    with pytest.raises(RuntimeError, match="max_step"):
        model.ppl(np.zeros((2, 41), np.int32))
