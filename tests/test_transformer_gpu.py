"""End-to-end parity of the QuantTransformer engine (through the pybind surface and the
model-level C ABI) against the numpy oracle's beam search on the same seeded weights and
inputs. Tolerances: encoder output 2e-2 max abs / 1e-3 mean abs (fp32 here, tighter than the
fp16 bound); generated token sequences identical on >= 99% of sentences for the large case
and on every sentence for the small ones unless a score near-tie is shown."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from lightseq_b200 import _lib as L  # noqa: E402
from lightseq_b200 import synth  # noqa: E402
from oracle import model as om  # noqa: E402


def _build(tmp_path, **kw):
    path = str(tmp_path / "model.ls100")
    conf, amax, w = synth.make_transformer(path, **kw)
    cfg = om.Config(hidden=int(conf["hidden"]), heads=int(conf["heads"]), ffn=int(conf["ffn"]), n_enc=int(conf["n_enc"]),
                    n_dec=int(conf["n_dec"]), vocab=int(conf["vocab"]), max_step=int(conf["max_step"]),
                    beam=int(conf["beam"]), length_penalty=float(conf["length_penalty"]),
                    extra_decode_length=int(conf["extra_decode_length"]), pad_id=int(conf["pad_id"]),
                    start_id=int(conf["start_id"]), end_id=int(conf["end_id"]),
                    sampling_method=synth.SAMPLING_METHODS[int(conf["sampling_method"])], topk=int(conf["topk"]),
                    topp=float(conf["topp"]), output_topk=bool(conf["output_topk"]),
                    no_scale_embedding=bool(conf["no_scale_embedding"]), seed_lo=int(conf["rng_seed"]),
                    pre_ln=bool(conf["pre_ln"]), diverse_lambda=float(conf["diverse_lambda"]))
    return path, cfg, om.State(w=w, amax=amax)


def _encoder_tap(model):
    L.lib.ls100_debug_encoder_output.restype = C.c_void_p
    L.lib.ls100_debug_encoder_output.argtypes = [C.c_void_p]
    return L.lib.ls100_debug_encoder_output(C.c_void_p(model._handle))


def _from_device(ptr, shape, dtype):
    n = int(np.prod(shape))
    t = torch.empty(n, dtype=dtype, device="cuda:0")
    ct = C.CDLL("libcudart.so.12", mode=C.RTLD_GLOBAL) if not hasattr(_from_device, "rt") else _from_device.rt
    _from_device.rt = ct
    rc = ct.cudaMemcpy(C.c_void_p(t.data_ptr()), C.c_void_p(ptr), C.c_size_t(n * t.element_size()), C.c_int(3))
    assert rc == 0
    return t.cpu().numpy().reshape(shape)


@pytest.mark.parametrize("eos_bias", [False, True])
def test_small_model_tokens_match_oracle(tmp_path, eos_bias):
    import lightseq_b200.inference as lsi

    kw = dict(hidden=128, heads=2, ffn=256, n_enc=2, n_dec=2, vocab=500, max_step=40, beam=4, extra_decode_length=12,
              seed=7)
    path, cfg, st = _build(tmp_path, **kw)
    if eos_bias:
        # make EOS competitive so that beams finish at different steps: a shared direction u in the
        # final LayerNorm bias and in the EOS embedding row adds ~0.8 to the EOS logit
        from lightseq_b200 import weights

        u = np.sign(np.random.default_rng(0).standard_normal(cfg.hidden)).astype(np.float32)
        st.w["dec.ln.b"] = (0.3 * u).astype(np.float32)
        st.w["emb"][cfg.end_id] = (0.02 * u).astype(np.float32)
        _, conf, amax, _ = weights.load(path)
        weights.save(path, "QuantTransformer", conf, amax, st.w)
    src = synth.transformer_inputs(batch=6, min_len=3, max_len=14, vocab=cfg.vocab, pad_id=cfg.pad_id, seed=3)
    ref_tok, ref_score, n_ref = om.Seq2Seq(cfg, st).generate(src)
    model = lsi.QuantTransformer(path, 8)
    tok, score = model.infer(src)
    assert tok.shape == (6, 1, n_ref), (tok.shape, n_ref)
    same = (tok[:, 0, :] == ref_tok).all(axis=1)
    print("identical sequences", same.sum(), "of", len(same), "steps", n_ref)
    assert same.all()
    np.testing.assert_allclose(score[:, 0], ref_score, rtol=1e-4, atol=1e-4)
    # encoder output tap
    enc_ref, pad = om.Seq2Seq(cfg, st).encode(src)
    enc = _from_device(_encoder_tap(model), enc_ref.shape, torch.float32)
    d = np.abs(enc - enc_ref)[~pad]
    print("encoder out max abs", d.max(), "mean abs", d.mean())
    assert d.max() < 2e-2 and d.mean() < 1e-3
    # a second call on the same object (graph replay, state re-initialisation) gives the same answer
    tok2, score2 = model.infer(src)
    assert np.array_equal(tok, tok2) and np.array_equal(score, score2)


def test_model_rejects_oversized_input(tmp_path):
    import lightseq_b200.inference as lsi

    path, cfg, st = _build(tmp_path, hidden=128, heads=2, ffn=256, n_enc=1, n_dec=1, vocab=100, max_step=16, seed=1)
    model = lsi.QuantTransformer(path, 2)
    with pytest.raises(RuntimeError, match="max_batch_size"):
        model.infer(np.full((3, 4), 5, np.int32))
    with pytest.raises(RuntimeError, match="max_step"):
        model.infer(np.full((1, 17), 5, np.int32))
    with pytest.raises(RuntimeError):
        lsi.QuantTransformer(str(tmp_path / "missing.ls100"), 2)


def _beam_state(model, rows):
    lib = L.lib
    lib.ls100_debug_beam_state.argtypes = [C.c_void_p] + [C.POINTER(C.c_void_p)] * 4 + [C.POINTER(C.c_int)] * 2
    pa, pn, pp, ps = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p()
    ms, beam = C.c_int(), C.c_int()
    assert lib.ls100_debug_beam_state(C.c_void_p(model._handle), C.byref(pa), C.byref(pn), C.byref(pp), C.byref(ps),
                                      C.byref(ms), C.byref(beam)) == 0
    alive = _from_device(pa.value, (rows, ms.value), torch.int32)
    anc = _from_device(pn.value, (rows, ms.value), torch.int32)
    probs = _from_device(pp.value, (rows,), torch.float32)
    score = _from_device(ps.value, (rows,), torch.float32)
    return alive, anc, probs, score


def guided_replay(model, cfg, st, src, n_steps):
    """Runs the engine for 1..n_steps decode steps (debug step limit) and replays the oracle along the
    ENGINE's beam choices: at every step the oracle, holding exactly the engine's histories, scores the
    engine's chosen (parent, token) pairs. Returns per-(sentence, step) statistics:
      exact  — engine's ordered choice equals the oracle's own top-beam list
      tie    — it differs, but every engine choice scores within `tol` of the oracle's k-th best, where tol is
               the largest engine-vs-oracle int8 logit difference of that sentence at that step (+ half a step)
      bad    — an engine choice scores worse than that (an unexplained divergence).
    Int8 logits differ at all because attention (fp32 softmax, different summation order) can flip an int8
    activation by one step, and every later quantiser can turn that perturbation into further one-step flips."""
    from oracle import beam as ob

    lib = L.lib
    lib.ls100_debug_set_step_limit.argtypes = [C.c_void_p, C.c_int]
    B, S = src.shape
    K = cfg.beam
    m = om.Seq2Seq(cfg, st)
    enc_out, pad = m.encode(src)
    ks, vs = m.cross_kv(enc_out)
    caches = [dict() for _ in range(cfg.n_dec)]
    alive = np.full((B, K, cfg.max_step), cfg.end_id, np.int32)
    alive[:, :, 0] = cfg.start_id
    probs = np.full((B, K), -1000.0, np.float32)
    probs[:, 0] = 0
    score = np.zeros((B, K), np.float32)
    stats = dict(exact=0, tie=0, bad=0, max_score_diff=0.0, logit_flips=0, logit_total=0)
    for s in range(n_steps):
        lib.ls100_debug_set_step_limit(C.c_void_p(model._handle), s + 1)
        model.infer(src)
        e_alive, e_anc, e_probs, e_score = _beam_state(model, B * K)
        e_alive = e_alive.reshape(B, K, -1)
        lq, s_l = m.decode_step(alive[:, :, s].reshape(-1), s, caches, ks, vs, pad)
        lq = lq.reshape(B, K, -1)
        ld = C.c_int()
        lib.ls100_debug_last_logits.restype = C.c_void_p
        lib.ls100_debug_last_logits.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
        lp = lib.ls100_debug_last_logits(C.c_void_p(model._handle), C.byref(ld))
        e_lq = _from_device(lp, (B * K, ld.value), torch.int8)[:, :cfg.vocab].reshape(B, K, -1)
        dl = np.abs(e_lq.astype(np.int32) - lq.astype(np.int32))
        stats["logit_flips"] += int((dl > 0).sum())
        stats["logit_total"] += dl.size
        stats["max_logit_diff"] = max(stats.get("max_logit_diff", 0), int(dl.max()))
        ln = ob.length_norm(s + 1, cfg.length_penalty)
        o_alive, o_probs, o_score, o_parent, _ = ob.beam_step(lq, s_l, alive, probs, score, s, ln, cfg.end_id)
        new_probs, new_score = probs.copy(), score.copy()
        parent = np.zeros((B, K), np.int64)
        for b in range(B):
            # tolerance: the largest int8 logit difference seen for this sentence at this step (+ half a step)
            tol = (float(dl[b].max()) + 0.5) * float(s_l) * float(ln) + 1e-4
            kth = float(o_score[b, K - 1])
            same = True
            worst = 0.0
            for j in range(K):
                par = int(e_anc[b * K + j, s]) - b * K
                tok = int(e_alive[b, j, s + 1])
                assert 0 <= par < K
                parent[b, j] = par
                assert np.array_equal(e_alive[b, j, :s + 1], alive[b, par, :s + 1]), "engine history is not its parent's"
                finished = s != 0 and alive[b, par, s] == cfg.end_id
                if finished:
                    assert tok == cfg.end_id
                    sc = float(score[b, par])
                else:
                    sc = float(ob.candidate_score(lq[b, par], s_l, probs[b, par], ln, tok))
                stats["max_score_diff"] = max(stats["max_score_diff"], abs(sc - float(e_score[b * K + j])))
                worst = max(worst, kth - sc)
                same &= (par == int(o_parent[b, j]) and tok == int(o_alive[b, j, s + 1]))
                new_score[b, j] = sc
                if tok != cfg.end_id:
                    new_probs[b, j] = np.float32(np.float32(sc) / ln)
                else:
                    new_probs[b, j] = probs[b, j]
            if not same and worst > tol:
                print(f"step {s} sentence {b}: worst gap {worst:.4f} tol {tol:.4f} logit diff max {dl[b].max()} "
                      f"rate {(dl[b] > 0).mean():.4f}")
            if same:
                stats["exact"] += 1
            elif worst <= tol:
                stats["tie"] += 1
            else:
                stats["bad"] += 1
        # continue from the engine's choice
        flat = (parent + np.arange(B)[:, None] * K).reshape(-1)
        for c in caches:
            c["k"], c["v"] = c["k"][flat], c["v"][flat]
        alive = e_alive.copy()
        probs, score = new_probs, new_score
    lib.ls100_debug_set_step_limit(C.c_void_p(model._handle), -1)
    return stats


def test_transformer_base_shape_guided_replay(tmp_path):
    """Transformer-base dimensions (6+6 layers, H 512, 8 heads, FFN 2048, vocab 32000, beam 4), 16 sentences,
    20 decode steps. A randomly initialised model has an almost flat output distribution, so free-running beam
    search is chaotic: a one-step int8 difference in a logit reorders near-tied candidates. The test therefore
    follows the engine's own beams and checks EVERY choice against the oracle's scores under identical histories:
    no choice may be worse than the oracle's k-th best by more than the int8 logit difference observed at that
    step, and scores must agree."""
    import lightseq_b200.inference as lsi

    path, cfg, st = _build(tmp_path, max_step=64, extra_decode_length=8, seed=1234)
    src = synth.transformer_inputs(batch=16, min_len=8, max_len=16, vocab=cfg.vocab, pad_id=cfg.pad_id, seed=4321)
    model = lsi.QuantTransformer(path, 16)
    stats = guided_replay(model, cfg, st, src, 20)
    total = stats["exact"] + stats["tie"] + stats["bad"]
    print("guided replay:", stats, "exact fraction", stats["exact"] / total)
    assert stats["bad"] == 0
    assert stats["exact"] / total >= 0.85
    assert stats["max_score_diff"] < 0.1
    assert stats["max_logit_diff"] <= 6
    # free-running comparison, reported (not asserted beyond a loose bound) for the record
    ref_tok, ref_score, n_ref = om.Seq2Seq(cfg, st).generate(src)
    tok, score = model.infer(src)
    assert tok.shape == (16, 1, n_ref)
    same = (tok[:, 0, :] == ref_tok).all(axis=1)
    print("free-running identical sequences", int(same.sum()), "of 16")


def test_reference_protobuf_file_runs_unchanged(tmp_path):
    """A model written in the reference's QuantTransformer protobuf format and converted back generates exactly what
    the same model does when loaded from the engine's own container (the int8 weights survive the trip)."""
    import lightseq_b200.inference as lsi
    from lightseq_b200 import ls_proto, weights

    conf, amax, w = synth.make_transformer(None, hidden=128, heads=2, ffn=256, n_enc=2, n_dec=2, vocab=120, max_step=40, seed=9)
    for i in range(2):
        amax[f"dec.{i}.xv.w"] = amax[f"dec.{i}.xk.w"]
    direct, pb, conv = str(tmp_path / "a.ls100"), str(tmp_path / "m.pb"), str(tmp_path / "b.ls100")
    weights.save(direct, "QuantTransformer", conf, amax, w)
    ls_proto.write_quant_transformer(pb, conf, amax, w)
    ls_proto.convert(pb, conv)
    src = synth.transformer_inputs(batch=6, min_len=5, max_len=14, vocab=120, pad_id=1, seed=4)
    t1, s1 = lsi.QuantTransformer(direct, 8).infer(src)
    t2, s2 = lsi.QuantTransformer(conv, 8).infer(src)
    # a file in the reference's format returns every beam, as the reference's QuantTransformer does; beam 0 is the answer
    assert t2.shape == (6, int(conf["beam"]), t1.shape[2]) and s2.shape == (6, int(conf["beam"]))
    assert np.array_equal(t1, t2[:, :1]) and np.array_equal(s1, s2[:, :1])


def test_exported_checkpoint_generates_the_same_tokens(tmp_path):
    """Checkpoint of the torch fake-quant layers (key names of the reference's modules) -> exporter -> protobuf file ->
    engine: the same tokens and scores as the model loaded from the engine's own container."""
    import lightseq_b200.inference as lsi
    from lightseq_b200 import export, ls_proto, weights

    conf, amax, w = synth.make_transformer(None, hidden=128, heads=2, ffn=256, n_enc=2, n_dec=2, vocab=120, max_step=40, seed=10)
    for i in range(2):
        amax[f"dec.{i}.xv.w"] = amax[f"dec.{i}.xk.w"]
    direct, pb, conv = str(tmp_path / "a.ls100"), str(tmp_path / "m.pb"), str(tmp_path / "b.ls100")
    weights.save(direct, "QuantTransformer", conf, amax, w)
    state = export.engine_to_state_dict(conf, amax, w)
    export.export_quant_transformer(state, pb, heads=2, beam=int(conf["beam"]), length_penalty=float(conf["length_penalty"]),
                                    extra_decode_length=int(conf["extra_decode_length"]), max_step=40, pad_id=int(conf["pad_id"]),
                                    bos_id=int(conf["start_id"]), eos_id=int(conf["end_id"]))
    ls_proto.convert(pb, conv)
    src = synth.transformer_inputs(batch=6, min_len=5, max_len=14, vocab=120, pad_id=int(conf["pad_id"]), seed=5)
    t1, s1 = lsi.QuantTransformer(direct, 8).infer(src)
    t2, s2 = lsi.QuantTransformer(conv, 8).infer(src)
    assert np.array_equal(t1, t2[:, :1]) and np.array_equal(s1, s2[:, :1])


def test_entry_point_smoke_runs():
    """The repository's smoke entry (one tcgen05 GEMM checked on its accumulators + a tiny generation checked token
    for token against the oracle) is part of the suite so that it cannot go stale."""
    import importlib

    importlib.import_module("__graft_entry__").smoke()


def test_device_timeout_surfaces_as_an_infer_error(tmp_path):
    """An expired device-side wait on the model's own context makes the next infer() raise (what the engine's
    drivers do with ls100_ctx_poll_error), and the model works again afterwards."""
    import lightseq_b200.inference as lsi

    path, cfg, st = _build(tmp_path, hidden=128, heads=2, ffn=256, n_enc=1, n_dec=1, vocab=100, max_step=16, seed=1)
    model = lsi.QuantTransformer(path, 2)
    src = np.full((2, 4), 5, np.int32)
    want, _ = model.infer(src)
    L.lib.ls100_debug_model_expire_wait.argtypes = [C.c_void_p]
    assert L.lib.ls100_debug_model_expire_wait(C.c_void_p(model._handle)) == 0
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        model.infer(src)
    got, _ = model.infer(src)
    assert np.array_equal(got, want)


def test_batch_split_over_two_gpus_is_bit_identical(tmp_path):
    """One request batch split over two GPUs (a replica, a host thread and a stream per GPU) gives, sentence for
    sentence, exactly the tokens and scores of the same batch on one GPU."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import lightseq_b200.inference as lsi
    from lightseq_b200 import sharding

    path, cfg, st = _build(tmp_path, hidden=128, heads=2, ffn=256, n_enc=2, n_dec=2, vocab=500, max_step=40, beam=4,
                           extra_decode_length=12, seed=7)
    src = synth.transformer_inputs(batch=11, min_len=3, max_len=14, vocab=cfg.vocab, pad_id=cfg.pad_id, seed=3)
    torch.cuda.set_device(0)
    tok1, sc1 = lsi.QuantTransformer(path, 11).infer(src)
    runner = sharding.ReplicaRunner(path, 11, [0, 1])
    tok2, sc2 = runner.infer(src, cfg.pad_id, cfg.end_id, trim=False)
    assert np.array_equal(tok1, tok2) and np.array_equal(sc1, sc2)
    tok3, sc3 = runner.infer(src, cfg.pad_id, cfg.end_id)  # trimmed shards: each decodes to its own length cap
    assert tok3.shape[0] == 11 and tok3.shape[2] <= tok1.shape[2]
    runner.close()


SMALL = dict(hidden=128, heads=2, ffn=256, n_enc=2, n_dec=2, vocab=500, max_step=24, beam=4, extra_decode_length=12, seed=7)


def _boost_eos(path, cfg, st, amount=0.3):
    """Makes EOS competitive (a shared direction in the final LayerNorm bias and the EOS embedding row), so that
    sequences end at different steps."""
    from lightseq_b200 import weights

    u = np.sign(np.random.default_rng(0).standard_normal(cfg.hidden)).astype(np.float32)
    st.w["dec.ln.b"] = (amount * u).astype(np.float32)
    st.w["emb"][cfg.end_id] = (0.02 * u).astype(np.float32)
    _, conf, amax, _ = weights.load(path)
    weights.save(path, "QuantTransformer", conf, amax, st.w)


@pytest.mark.parametrize("method,extra", [("topk", dict(topk=4)), ("topk", dict(topk=1)), ("topp", dict(topp=0.7)),
                                          ("topk_greedy", dict())])
def test_sampling_methods_match_oracle(tmp_path, method, extra):
    """sampling_method topk / topp (one sampled sequence per sentence, up to max_step tokens) and topk_greedy (a beam
    step, then every row takes its best token) of the reference's decoder: same tokens as the oracle, draw for draw
    (QuantDecoder::sample and topk_greedy_search, lightseq/inference/model/quant_decoder.cc.cu:951-985, 1101-1133)."""
    import lightseq_b200.inference as lsi

    path, cfg, st = _build(tmp_path, sampling_method=method, rng_seed=123, **extra, **SMALL)
    _boost_eos(path, cfg, st)
    src = synth.transformer_inputs(batch=5, min_len=3, max_len=10, vocab=cfg.vocab, pad_id=cfg.pad_id, seed=3)
    ref_tok, ref_score, n_ref = om.Seq2Seq(cfg, st).generate(src)
    tok, score = lsi.QuantTransformer(path, 5).infer(src)
    k = cfg.beam if method == "topk_greedy" else 1
    assert tok.shape == (5, k, n_ref) and score.shape == (5, k), (tok.shape, n_ref)
    same = (tok == ref_tok).all(axis=(1, 2))
    print(method, extra, "identical", int(same.sum()), "of 5, steps", n_ref, "distinct tokens", len(set(tok.ravel().tolist())))
    assert same.all()
    assert (tok[:, :, -1] == cfg.end_id).all()  # the last position is EOS whatever was generated there


def test_every_beam_is_returned_when_asked(tmp_path):
    """output_topk: tokens [batch, beam, len] and scores [batch, beam] (what the reference's QuantTransformer always
    returns, lightseq/inference/pywrapper/quant_transformer.cc:100-109); beam 0 is the single-beam answer."""
    import lightseq_b200.inference as lsi

    path, cfg, st = _build(tmp_path, output_topk=True, **SMALL)
    _boost_eos(path, cfg, st)
    src = synth.transformer_inputs(batch=6, min_len=3, max_len=10, vocab=cfg.vocab, pad_id=cfg.pad_id, seed=4)
    ref_tok, ref_score, n_ref = om.Seq2Seq(cfg, st).generate(src)
    tok, score = lsi.QuantTransformer(path, 6).infer(src)
    assert tok.shape == (6, cfg.beam, n_ref)
    assert np.array_equal(tok, ref_tok)
    np.testing.assert_allclose(score, ref_score, rtol=1e-4, atol=1e-4)
    assert (np.diff(score, axis=1) <= 1e-6).all()  # beams are ordered by score


def test_negative_length_penalty_picks_the_best_score_per_token(tmp_path):
    """length_penalty < 0: scores are normalised by 1/len during the search and the result is the beam with the best
    score per non-EOS token, not beam 0 (ker_write_trg_tokenid_neg_penalty,
    lightseq/inference/kernels/transformerKernels.cc.cu:1752-1784)."""
    import lightseq_b200.inference as lsi

    path, cfg, st = _build(tmp_path, length_penalty=-1.0, **SMALL)
    _boost_eos(path, cfg, st)
    src = synth.transformer_inputs(batch=8, min_len=3, max_len=10, vocab=cfg.vocab, pad_id=cfg.pad_id, seed=5)
    ref_tok, ref_score, n_ref = om.Seq2Seq(cfg, st).generate(src)
    tok, score = lsi.QuantTransformer(path, 8).infer(src)
    assert tok.shape == (8, 1, n_ref)
    assert np.array_equal(tok[:, 0], ref_tok)
    np.testing.assert_allclose(score[:, 0], ref_score, rtol=1e-4, atol=1e-4)


def test_unscaled_embeddings(tmp_path):
    """no_scale_embedding: the token embedding is not multiplied by sqrt(hidden) (quant_transformer.proto:148)."""
    import lightseq_b200.inference as lsi

    path, cfg, st = _build(tmp_path, no_scale_embedding=True, **SMALL)
    src = synth.transformer_inputs(batch=4, min_len=3, max_len=10, vocab=cfg.vocab, pad_id=cfg.pad_id, seed=6)
    ref_tok, ref_score, n_ref = om.Seq2Seq(cfg, st).generate(src)
    tok, score = lsi.QuantTransformer(path, 4).infer(src)
    assert tok.shape == (4, 1, n_ref) and np.array_equal(tok[:, 0], ref_tok)


def test_beam_result_writer_modes():
    """ls100_beam_write_result against a direct numpy statement of the three output forms."""
    B, K, ms, end_id, n = 3, 4, 12, 2, 7
    r = np.random.default_rng(9)
    alive = r.integers(3, 50, size=(B, K, ms)).astype(np.int32)
    alive[0, 1, 4:] = end_id
    alive[1, 2, 2:] = end_id
    score = -r.random((B, K)).astype(np.float32) * 5
    from tests.gpu_util import ctx, dev, empty, ptr, sync_check

    d_alive, d_score = dev(alive), dev(score)
    for mode in (0, 1, 2):
        rows = B * K if mode == 2 else B
        out_t, out_s = empty((rows, n), torch.int32), empty((rows,), torch.float32)
        a = L.BeamResultArgs(alive=ptr(d_alive), seq_score=ptr(d_score), batch=B, beam=K, max_step=ms, end_id=end_id, n_out=n,
                             mode=mode, out_tokens=ptr(out_t), out_scores=ptr(out_s))
        L.call("ls100_beam_write_result", ctx(), a)
        sync_check()
        t, s = out_t.cpu().numpy(), out_s.cpu().numpy()
        if mode == 0:
            assert np.array_equal(t, alive[:, 0, 1:n + 1]) and np.array_equal(s, score[:, 0])
        elif mode == 2:
            want = alive[:, :, 1:n + 1].reshape(B * K, n).copy()
            want[:, -1] = end_id
            assert np.array_equal(t, want) and np.array_equal(s, score.reshape(-1))
        else:
            for b in range(B):
                lens = (alive[b, :, 1:n + 1] != end_id).sum(1).astype(np.float32)
                per = score[b] / (lens + np.float32(1e-12))
                j = int(np.argmax(per))
                assert np.array_equal(t[b], alive[b, j, 1:n + 1]) and s[b] == per[j]


def test_post_ln_encoder_decoder_matches_oracle(tmp_path):
    """is_post_ln (quant_transformer.proto:147): LayerNorm after every residual sum, as the torch layers compute it with
    normalize_before false (torch_transformer_layers.py:630-679, 844-965); no final LayerNorms."""
    import lightseq_b200.inference as lsi

    path, cfg, st = _build(tmp_path, pre_ln=False, **SMALL)
    _boost_eos(path, cfg, st)
    src = synth.transformer_inputs(batch=6, min_len=3, max_len=10, vocab=cfg.vocab, pad_id=cfg.pad_id, seed=8)
    ref_tok, ref_score, n_ref = om.Seq2Seq(cfg, st).generate(src)
    model = lsi.QuantTransformer(path, 6)
    tok, score = model.infer(src)
    assert tok.shape == (6, 1, n_ref), (tok.shape, n_ref)
    same = (tok[:, 0] == ref_tok).all(axis=1)
    print("post-LN identical sequences", int(same.sum()), "of 6")
    assert same.all()
    np.testing.assert_allclose(score[:, 0], ref_score, rtol=1e-4, atol=1e-4)
    enc_ref, pad = om.Seq2Seq(cfg, st).encode(src)
    enc = _from_device(_encoder_tap(model), enc_ref.shape, torch.float32)
    d = np.abs(enc - enc_ref)[~pad]
    assert d.max() < 2e-2 and d.mean() < 1e-3


def test_diverse_beam_search_matches_oracle(tmp_path):
    """diverse_lambda: sibling candidates of one beam are penalised by their rank, which spreads the survivors over
    the beams (ker_diverse_beam_search, lightseq/inference/kernels/transformerKernels.cc.cu:312-333)."""
    import lightseq_b200.inference as lsi

    path, cfg, st = _build(tmp_path, diverse_lambda=0.4, output_topk=True, **SMALL)
    _boost_eos(path, cfg, st, 0.2)
    src = synth.transformer_inputs(batch=6, min_len=3, max_len=10, vocab=cfg.vocab, pad_id=cfg.pad_id, seed=11)
    ref_tok, ref_score, n_ref = om.Seq2Seq(cfg, st).generate(src)
    tok, score = lsi.QuantTransformer(path, 6).infer(src)
    assert tok.shape == (6, cfg.beam, n_ref)
    assert np.array_equal(tok, ref_tok)
    np.testing.assert_allclose(score, ref_score, rtol=1e-4, atol=1e-4)
    plain_path, plain_cfg, plain_st = _build(tmp_path, output_topk=True, **SMALL)
    _boost_eos(plain_path, plain_cfg, plain_st, 0.2)
    plain, _ = lsi.QuantTransformer(plain_path, 6).infer(src)
    assert plain.shape[2] != tok.shape[2] or not np.array_equal(plain, tok)  # the penalty changes what survives


def test_beam_selection_from_logit_statistics_gives_the_same_generation(tmp_path, monkeypatch):
    """LS100_FUSED_SELECT: the logits GEMM keeps per-group maxima and sums of exponentials and ls100_beam_select picks
    the candidates from them instead of ls100_beam_topk reading the logits again. Same tokens, scores to rounding."""
    import lightseq_b200.inference as lsi

    path, cfg, st = _build(tmp_path, **SMALL)
    _boost_eos(path, cfg, st)
    src = synth.transformer_inputs(batch=6, min_len=3, max_len=10, vocab=cfg.vocab, pad_id=cfg.pad_id, seed=3)
    tok0, score0 = lsi.QuantTransformer(path, 6).infer(src)
    monkeypatch.setenv("LS100_FUSED_SELECT", "1")
    tok1, score1 = lsi.QuantTransformer(path, 6).infer(src)
    assert np.array_equal(tok0, tok1)
    np.testing.assert_allclose(score1, score0, rtol=1e-5, atol=1e-5)
