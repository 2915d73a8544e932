"""The reference's own PyTorch fake-quant modules, loaded with this repository's synthetic weights.

Test infrastructure, not product code (only tests/, tests/golden/, __graft_entry__ and bench.py's CPU legs may
import it). ``import_reference(root)`` imports lightseq/training/ops/pytorch/{quantization,
torch_transformer_layers}.py from ``root`` (a checkout of bytedance/lightseq, or the tree oracle/make_ref.py
places under oracle/_ref/) without running the package __init__ files that JIT-build CUDA extensions. The builders
wire clip-max values the way the reference stores them (learned quantisers in ``Clip.clip_value_max``, fixed ones in
``_amax``: lightseq/training/pytorch_quantization/nn/modules/tensor_quantizer.py:340-347).

``RefSeq2Seq`` is the encoder-decoder of lightseq/training/cli/fs_modules/ls_transformer.py:253-420 assembled from
those modules (TransformerEmbeddingLayer, TransformerEncoderLayer, TransformerDecoderLayer with its fairseq-style
incremental state, final LayerNorms, output projection sharing the embedding table and quantiser). Every layer
computation is the reference's; the beam-search step between decoder calls exists in the reference only as CUDA
kernels, so it is oracle/beam.py's restatement.
"""
from __future__ import annotations

import os
import sys
import types

import numpy as np

_mods = None


def import_reference(root: str):
    """Returns (quantization module, torch_transformer_layers module) of the reference under ``root``."""
    global _mods
    if _mods is not None:
        return _mods
    root = os.path.abspath(root)
    if not os.path.isdir(os.path.join(root, "lightseq")):
        raise RuntimeError(f"{root}: no lightseq package")
    if root not in sys.path:
        sys.path.insert(0, root)
    import lightseq  # noqa: F401

    for name in ("lightseq.training", "lightseq.training.ops", "lightseq.training.ops.pytorch"):
        if name in sys.modules and getattr(sys.modules[name], "__file__", None):
            continue  # already a real (empty) package, as under oracle/_ref
        m = types.ModuleType(name)
        m.__path__ = [os.path.join(root, *name.split("."))]
        sys.modules[name] = m
    from lightseq.training.ops.pytorch import quantization as qz
    from lightseq.training.ops.pytorch import torch_transformer_layers as tl

    _mods = (qz, tl)
    return _mods


def _torch():
    import torch

    return torch


def set_qlinear(m, amax, name):
    if m.input_quant is not None:
        m.input_quant.clip.clip_value_max.data.fill_(amax[name + ".in"])
    if m.output_quant is not None:
        m.output_quant._amax.fill_(amax[name + ".out"])


def load_linear(m, w, name, amax, w_amax=None):
    torch = _torch()
    m.weight.data.copy_(torch.from_numpy(w[name + ".w"]))
    if m.bias is not None:
        m.bias.data.copy_(torch.from_numpy(w[name + ".b"]))
    m.weight_quant._amax.fill_(amax[w_amax or name + ".w"])
    set_qlinear(m, amax, name)


def load_ln(m, w, name):
    torch = _torch()
    m.weight.data.copy_(torch.from_numpy(w[name + ".g"]))
    m.bias.data.copy_(torch.from_numpy(w[name + ".b"]))


def build_encoder_layer(mods, w, amax, p, hidden, heads, ffn, act="relu", pre_ln=True):
    qz, tl = mods
    cfg = tl.TransformerEncoderLayer.get_config(
        max_batch_tokens=16384, max_seq_len=1024, hidden_size=hidden, intermediate_size=ffn, nhead=heads,
        attn_prob_dropout_ratio=0.0, activation_dropout_ratio=0.0, hidden_dropout_ratio=0.0,
        pre_layer_norm=pre_ln, fp16=False, local_rank=-1, activation_fn=act)
    lyr = tl.TransformerEncoderLayer(cfg)
    load_linear(lyr.self_attn.qkv_proj, w, p + ".qkv", amax)
    load_linear(lyr.self_attn.out_proj, w, p + ".out", amax)
    load_linear(lyr.fc1, w, p + ".fc1", amax)
    load_linear(lyr.fc2, w, p + ".fc2", amax)
    load_ln(lyr.self_attn_layer_norm, w, p + ".ln1")
    load_ln(lyr.final_layer_norm, w, p + ".ln2")
    lyr.eval()
    lyr.apply(qz.enable_quant)
    return lyr


def build_decoder_layer(mods, w, amax, p, hidden, heads, ffn, n_dec, act="relu"):
    qz, tl = mods
    cfg = tl.TransformerDecoderLayer.get_config(
        max_batch_tokens=16384, max_seq_len=1024, hidden_size=hidden, intermediate_size=ffn, nhead=heads,
        attn_prob_dropout_ratio=0.0, activation_dropout_ratio=0.0, hidden_dropout_ratio=0.0,
        pre_layer_norm=True, fp16=False, local_rank=-1, nlayer=n_dec, activation_fn=act)
    lyr = tl.TransformerDecoderLayer(cfg)
    load_linear(lyr.self_attn.qkv_proj, w, p + ".qkv", amax)
    lyr.self_attn.attention_quant._amax.fill_(amax[p + ".kv"])
    load_linear(lyr.self_attn.out_proj, w, p + ".out", amax)
    load_linear(lyr.encoder_attn.q_proj, w, p + ".xq", amax)
    load_linear(lyr.encoder_attn.k_proj, w, p + ".xk", amax)
    load_linear(lyr.encoder_attn.v_proj, w, p + ".xv", amax)
    load_linear(lyr.encoder_attn.out_proj, w, p + ".xout", amax)
    load_linear(lyr.fc1, w, p + ".fc1", amax)
    load_linear(lyr.fc2, w, p + ".fc2", amax)
    load_ln(lyr.self_attn_layer_norm, w, p + ".ln1")
    load_ln(lyr.encoder_attn_layer_norm, w, p + ".ln2")
    load_ln(lyr.final_layer_norm, w, p + ".ln3")
    lyr.eval()
    lyr.apply(qz.enable_quant)
    return lyr


def build_embedding(mods, w, amax, hidden, vocab, pad_id):
    torch = _torch()
    qz, tl = mods
    cfg = tl.TransformerEmbeddingLayer.get_config(
        vocab_size=vocab, embedding_dim=hidden, max_batch_tokens=16384, max_seq_len=1024, padding_idx=pad_id,
        dropout=0.0, fp16=False, local_rank=-1)
    emb = tl.TransformerEmbeddingLayer(cfg)
    emb.emb_lookup.weight.data.copy_(torch.from_numpy(w["emb"]))
    emb.emb_quant.clip.clip_value_max.data.fill_(amax["emb"])
    emb.eval()
    emb.apply(qz.enable_quant)
    return emb


class RefSeq2Seq:
    """``cfg`` is an oracle.model.Config; weights and clip-max tables as lightseq_b200.synth makes them."""

    def __init__(self, mods, cfg, w, amax):
        torch = _torch()
        qz, tl = mods
        self.cfg, self.amax = cfg, amax
        H, heads, F, V = cfg.hidden, cfg.heads, cfg.ffn, cfg.vocab
        self.emb = build_embedding(mods, w, amax, H, V, cfg.pad_id)
        self.enc_layers = [build_encoder_layer(mods, w, amax, f"enc.{l}", H, heads, F, cfg.act) for l in range(cfg.n_enc)]
        self.dec_layers = [build_decoder_layer(mods, w, amax, f"dec.{l}", H, heads, F, cfg.n_dec, cfg.act)
                           for l in range(cfg.n_dec)]
        self.enc_ln = torch.nn.LayerNorm(H)
        load_ln(self.enc_ln, w, "enc.ln")
        self.dec_ln = torch.nn.LayerNorm(H)
        load_ln(self.dec_ln, w, "dec.ln")
        proj = qz.QuantLinear(H, V, bias=False)
        proj.weight_quant = self.emb.emb_quant
        proj.weight = self.emb.emb_lookup.weight
        set_qlinear(proj, amax, "logits")
        proj.eval()
        proj.apply(qz.enable_quant)
        self.proj = proj

    def encode(self, src: np.ndarray):
        torch = _torch()
        with torch.no_grad():
            t = torch.from_numpy(src.astype(np.int64))
            pad = t.eq(self.cfg.pad_id)
            x = self.emb(t)
            for lyr in self.enc_layers:
                x = lyr(x, pad)
            return self.enc_ln(x), pad

    def generate(self, src: np.ndarray, max_len=None, early_stop: bool = True):
        """Beam search with the bookkeeping of oracle.model.Seq2Seq.generate; returns (tokens [B, n], scores [B], n)."""
        torch = _torch()
        from .beam import beam_step, length_norm

        cfg = self.cfg
        B, S = src.shape
        K = cfg.beam
        s_l = np.float32(self.amax["logits.out"] / 127.0)
        with torch.no_grad():
            enc_out, pad = self.encode(src)
            enc_tbc = enc_out.repeat_interleave(K, dim=0).transpose(0, 1).contiguous()  # [S, B*K, H]
            pad_t = pad.repeat_interleave(K, dim=0)
            max_decode = min(cfg.max_step, S + cfg.extra_decode_length) - 1
            if max_len is not None:
                max_decode = min(max_decode, max_len)
            alive = np.full((B, K, cfg.max_step), cfg.end_id, dtype=np.int32)
            alive[:, :, 0] = cfg.start_id
            probs = np.full((B, K), -1000.0, dtype=np.float32)
            probs[:, 0] = 0.0
            score = np.zeros((B, K), dtype=np.float32)
            inc = {}
            cur = 0
            for cur in range(max_decode - 1):
                tok = torch.from_numpy(alive[:, :, cur].reshape(-1, 1).astype(np.int64))
                x = self.emb(tok, cur)
                for lyr in self.dec_layers:
                    x, _, _ = lyr(x, encoder_out=enc_tbc, encoder_padding_mask=pad_t, incremental_state=inc)
                logits = self.proj(self.dec_ln(x))[:, 0].numpy()
                lq = np.rint(logits / s_l).astype(np.int8)  # the output quantiser's integers
                ln = length_norm(cur + 1, cfg.length_penalty)
                alive, probs, score, parent, n_fin = beam_step(lq.reshape(B, K, -1), s_l, alive, probs, score, cur, ln, cfg.end_id)
                if early_stop and n_fin == B * K:
                    break
                flat = torch.from_numpy((parent + np.arange(B)[:, None] * K).reshape(-1))
                for state in inc.values():  # what MultiheadAttention.reorder_incremental_state does
                    for name, t in state.items():
                        if t is not None:
                            state[name] = t.index_select(0, flat)
            else:
                cur = max(max_decode - 1, 0)
        n = cur + 1
        return alive[:, 0, 1:n + 1].copy(), score[:, 0].copy(), n
