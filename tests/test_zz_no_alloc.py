"""The allocation-free beam-update entry point (ls100_beam_update_noalloc) against ls100_beam_update.

Some callers of this library can never allocate device memory: a server that gave the whole GPU to its own
arena at start-up, or a real-time thread for which cudaMalloc's device-wide synchronisation is forbidden. For
them the two scratch arrays of the beam update (finished counters, CTA tickets) live inside the library. This
test drives both entry points through the C ABI from identical states, twice in a row (the second call sees
the scratch exactly as the first left it), and requires bit-identical results. It sits in its own file, named
to be collected last, and builds its own inputs, so it passes alone or after the rest of the suite."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from lightseq_b200 import _lib as L  # noqa: E402
from oracle import beam as ob  # noqa: E402
from tests.gpu_util import ctx, dev, empty, ptr, sync_check  # noqa: E402


def _state(B, K, ms, end_id):
    alive = np.full((B, K, ms), end_id, np.int32)
    alive[:, :, 0] = 3
    probs = np.full((B, K), -1000.0, np.float32)
    probs[:, 0] = 0
    return dict(alive=dev(alive), probs=dev(probs), score=dev(np.zeros((B, K), np.float32)),
                anc=dev(np.zeros((B * K, ms), np.int32)), step=dev(np.zeros(1, np.int32)),
                stop=dev(np.full(1, -1, np.int32)), fin=dev(np.zeros(ms, np.int32)), ticket=dev(np.zeros(ms, np.int32)))


def test_noalloc_beam_update_matches_the_allocating_entry_point_twice():
    B, K, ms, end_id, V = 5, 4, 32, 2, 777
    r = np.random.default_rng(12)
    ldv = (V + 15) // 16 * 16
    ln = dev(np.array([ob.length_norm(i + 1, 0.6) for i in range(ms)], np.float32))
    sa, sb = _state(B, K, ms, end_id), _state(B, K, ms, end_id)
    cs, ct = empty((B * K, K), torch.float32), empty((B * K, K), torch.int32)
    for call in range(2):
        lq = np.clip(np.rint(r.standard_normal((B * K, ldv)) * 30), -127, 127).astype(np.int8)
        if call == 1:
            lq[:, end_id] = 125  # second call: beams finish, so the finished counter is exercised
        d_l = dev(lq)
        for st, fn in ((sa, "ls100_beam_update"), (sb, "ls100_beam_update_noalloc")):
            a1 = L.BeamTopkArgs(logits=ptr(d_l), ld_logits=ldv, s_logits=0.05, batch=B, beam=K, vocab=V, max_step=ms,
                                end_id=end_id, step_ptr=ptr(st["step"]), length_norm=ptr(ln), alive=ptr(st["alive"]),
                                seq_probs=ptr(st["probs"]), seq_score=ptr(st["score"]), cand_score=ptr(cs),
                                cand_token=ptr(ct))
            L.call("ls100_beam_topk", ctx(), a1)
            a2 = L.BeamUpdateArgs(cand_score=ptr(cs), cand_token=ptr(ct), batch=B, beam=K, max_step=ms, end_id=end_id,
                                  step_ptr=ptr(st["step"]), length_norm=ptr(ln), alive=ptr(st["alive"]), anc=ptr(st["anc"]),
                                  seq_probs=ptr(st["probs"]), seq_score=ptr(st["score"]),
                                  fin_count=ptr(st["fin"]) if fn == "ls100_beam_update" else None,
                                  ticket=ptr(st["ticket"]) if fn == "ls100_beam_update" else None,
                                  stop_step=ptr(st["stop"]), stop_host=None)
            L.call(fn, ctx(), a2)
            sync_check()
        for key in ("alive", "anc", "probs", "score", "step", "stop"):
            assert torch.equal(sa[key], sb[key]), f"call {call}: {key} differs between the two entry points"
        assert int(sa["step"].cpu()[0]) == call + 1
    # a third step with every beam finished: both must report the stop step
    lq = np.full((B * K, ldv), -5, np.int8)
    lq[:, end_id] = 127
    d_l = dev(lq)
    for st, fn in ((sa, "ls100_beam_update"), (sb, "ls100_beam_update_noalloc")):
        a1 = L.BeamTopkArgs(logits=ptr(d_l), ld_logits=ldv, s_logits=0.05, batch=B, beam=K, vocab=V, max_step=ms, end_id=end_id,
                            step_ptr=ptr(st["step"]), length_norm=ptr(ln), alive=ptr(st["alive"]), seq_probs=ptr(st["probs"]),
                            seq_score=ptr(st["score"]), cand_score=ptr(cs), cand_token=ptr(ct))
        L.call("ls100_beam_topk", ctx(), a1)
        a2 = L.BeamUpdateArgs(cand_score=ptr(cs), cand_token=ptr(ct), batch=B, beam=K, max_step=ms, end_id=end_id,
                              step_ptr=ptr(st["step"]), length_norm=ptr(ln), alive=ptr(st["alive"]), anc=ptr(st["anc"]),
                              seq_probs=ptr(st["probs"]), seq_score=ptr(st["score"]),
                              fin_count=ptr(st["fin"]) if fn == "ls100_beam_update" else None,
                              ticket=ptr(st["ticket"]) if fn == "ls100_beam_update" else None,
                              stop_step=ptr(st["stop"]), stop_host=None)
        L.call(fn, ctx(), a2)
        sync_check()
    assert torch.equal(sa["stop"], sb["stop"]) and torch.equal(sa["alive"], sb["alive"])


def test_noalloc_beam_update_rejects_sizes_beyond_its_scratch():
    st = _state(1, 2, 8, 2)
    cs, ct = empty((2, 2), torch.float32), empty((2, 2), torch.int32)
    ln = dev(np.ones(8, np.float32))
    a2 = L.BeamUpdateArgs(cand_score=ptr(cs), cand_token=ptr(ct), batch=1, beam=2, max_step=4096, end_id=2,
                          step_ptr=ptr(st["step"]), length_norm=ptr(ln), alive=ptr(st["alive"]), anc=None,
                          seq_probs=ptr(st["probs"]), seq_score=ptr(st["score"]), fin_count=None, ticket=None,
                          stop_step=ptr(st["stop"]), stop_host=None)
    import ctypes as C

    assert L.lib.ls100_beam_update_noalloc(ctx().handle, C.byref(a2), None) == L.ERR_UNSUPPORTED


def test_noalloc_beam_update_rejected_call_enqueues_nothing():
    """A call that fails its argument checks (beam 9 > 8) must not clear the shared scratch: the counters a valid call
    left behind are still there afterwards, and the next valid call gives the same result as the allocating entry."""
    import ctypes as C

    B, K, ms, end_id, V = 3, 2, 16, 2, 64
    ldv = 64
    ln = dev(np.ones(ms, np.float32))
    lq = dev(np.clip(np.rint(np.random.default_rng(3).standard_normal((B * K, ldv)) * 30), -127, 127).astype(np.int8))
    sa, sb = _state(B, K, ms, end_id), _state(B, K, ms, end_id)
    cs, ct = empty((B * K, K), torch.float32), empty((B * K, K), torch.int32)

    def step(st, fn):
        a1 = L.BeamTopkArgs(logits=ptr(lq), ld_logits=ldv, s_logits=0.05, batch=B, beam=K, vocab=V, max_step=ms, end_id=end_id,
                            step_ptr=ptr(st["step"]), length_norm=ptr(ln), alive=ptr(st["alive"]), seq_probs=ptr(st["probs"]),
                            seq_score=ptr(st["score"]), cand_score=ptr(cs), cand_token=ptr(ct))
        L.call("ls100_beam_topk", ctx(), a1)
        a2 = L.BeamUpdateArgs(cand_score=ptr(cs), cand_token=ptr(ct), batch=B, beam=K, max_step=ms, end_id=end_id,
                              step_ptr=ptr(st["step"]), length_norm=ptr(ln), alive=ptr(st["alive"]), anc=ptr(st["anc"]),
                              seq_probs=ptr(st["probs"]), seq_score=ptr(st["score"]),
                              fin_count=ptr(st["fin"]) if fn == "ls100_beam_update" else None,
                              ticket=ptr(st["ticket"]) if fn == "ls100_beam_update" else None,
                              stop_step=ptr(st["stop"]), stop_host=None)
        L.call(fn, ctx(), a2)
        sync_check()
        return a2

    step(sa, "ls100_beam_update")
    good = step(sb, "ls100_beam_update_noalloc")
    bad = L.BeamUpdateArgs(cand_score=good.cand_score, cand_token=good.cand_token, batch=B, beam=9, max_step=ms, end_id=end_id,
                           step_ptr=good.step_ptr, length_norm=good.length_norm, alive=good.alive, anc=good.anc,
                           seq_probs=good.seq_probs, seq_score=good.seq_score, fin_count=None, ticket=None,
                           stop_step=good.stop_step, stop_host=None)
    assert L.lib.ls100_beam_update_noalloc(ctx().handle, C.byref(bad), None) == L.ERR_UNSUPPORTED
    sync_check()
    step(sa, "ls100_beam_update")
    step(sb, "ls100_beam_update_noalloc")
    for key in ("alive", "anc", "probs", "score", "step", "stop"):
        assert torch.equal(sa[key], sb[key]), f"{key} differs after a rejected call"
