"""Generates tests/golden/torch_layer_state_keys.json: the state-dict keys and shapes of the REAL reference torch layers
(lightseq/training/ops/pytorch/torch_transformer_layers.py, quantisation enabled) for hidden 64, ffn 128, one head,
vocabulary 40. The exporter test builds a checkpoint with exactly these keys.

Needs a checkout of bytedance/lightseq, named by $LIGHTSEQ_REF or the first argument; the tests only read the committed
json file. Usage:  LIGHTSEQ_REF=<checkout> python tests/golden/gen_state_keys.py
"""
from __future__ import annotations

import importlib.util
import json
import os
import sys
import types
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = os.environ.get("LIGHTSEQ_REF") or (sys.argv[1] if len(sys.argv) > 1 else "")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set LIGHTSEQ_REF (or pass the path) to a checkout of bytedance/lightseq")


def load(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    m = importlib.util.module_from_spec(spec)
    sys.modules[name] = m
    spec.loader.exec_module(m)
    return m


# empty stub packages: the real ``lightseq.training`` __init__ JIT-builds CUDA layers at import
for pkg in ["lightseq", "lightseq.training", "lightseq.training.ops", "lightseq.training.ops.pytorch"]:
    m = types.ModuleType(pkg)
    m.__path__ = [os.path.join(REF, pkg.replace(".", "/"))]
    sys.modules[pkg] = m
for n in ("quantization", "util", "layer_base", "torch_transformer_layers"):
    load("lightseq.training.ops.pytorch." + n, os.path.join(REF, f"lightseq/training/ops/pytorch/{n}.py"))
t = sys.modules["lightseq.training.ops.pytorch.torch_transformer_layers"]
enable_quant = sys.modules["lightseq.training.ops.pytorch.quantization"].enable_quant

common = dict(max_batch_tokens=64, max_seq_len=16, hidden_size=64, intermediate_size=128, nhead=1, attn_prob_dropout_ratio=0.0,
              activation_dropout_ratio=0.0, hidden_dropout_ratio=0.0, pre_layer_norm=True, fp16=False, local_rank=0,
              activation_fn="relu")
enc = t.TransformerEncoderLayer(t.TransformerEncoderLayer.get_config(**common))
dec = t.TransformerDecoderLayer(t.TransformerDecoderLayer.get_config(nlayer=1, **common))
emb = t.TransformerEmbeddingLayer(t.TransformerEmbeddingLayer.get_config(vocab_size=40, embedding_dim=64, max_batch_tokens=64,
                                                                         max_seq_len=16, padding_idx=1, dropout=0.0, fp16=False,
                                                                         local_rank=0))
out = {}
for name, mod in (("encoder_layer", enc), ("decoder_layer", dec), ("embedding", emb)):
    mod.apply(enable_quant)
    out[name] = {k: list(v.shape) for k, v in mod.state_dict().items()}
(HERE / "torch_layer_state_keys.json").write_text(json.dumps(out, indent=1, sort_keys=True) + "\n")
print({k: len(v) for k, v in out.items()})
