"""``lightseq_b200.inference`` — the class surface of the reference's ``lightseq.inference``
pybind module (lightseq/inference/pywrapper/wrapper.cc:919-996) on the B200 engine.

    import lightseq_b200.inference as lsi
    model = lsi.QuantTransformer("model.ls100", max_batch_size=128)
    tokens, scores = model.infer(np.int32 ids [batch, seq_len])   # ([batch, 1, L], [batch, 1])

The native module is required; there is no Python or CPU fallback.
"""
from . import _lib  # noqa: F401  (loads libls100.so first, and fails loudly if it is not built)

try:
    from ._ls100_py import QuantBert, QuantGpt, QuantTransformer, QuantVit  # noqa: F401
except ImportError as e:  # pragma: no cover
    raise ImportError(
        "lightseq_b200._ls100_py is missing: build it with `python -m lightseq_b200.build`") from e
