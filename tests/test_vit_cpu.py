"""The oracle's ViT patch embedding against a literal loop over the reference kernel's index arithmetic
(ker_patch_emb, lightseq/inference/kernels/embKernels.cc.cu:565-606), and the synthetic ViT builder."""
import numpy as np

from lightseq_b200 import synth
from oracle import model as om

F32 = np.float32


def test_patch_embed_follows_the_reference_indexing():
    B, C, image, patch, H = 2, 3, 12, 4, 8
    w = synth.vit_weights(hidden=H, heads=1, ffn=4, n_layer=0, image=image, patch=patch, channels=C, seed=2)
    px = synth.vit_inputs(batch=B, image=image, channels=C, seed=1)
    got = om.patch_embed(w, px, patch)
    g = image // patch
    want = np.zeros((B, 1 + g * g, H), F32)
    for b in range(B):
        for h in range(H):
            want[b, 0, h] = w["cls"][h] + w["pos"][0, h]
            for n in range(g * g):
                pr, pc = divmod(n, g)
                acc = 0.0
                for idx in range(C * patch * patch):
                    c, rem = divmod(idx, patch * patch)
                    r, q = divmod(rem, patch)
                    acc += float(px[b, c, pr * patch + r, pc * patch + q]) * float(w["conv.w"][h, idx])
                want[b, 1 + n, h] = F32(F32(F32(acc) + w["conv.b"][h]) + w["pos"][1 + n, h])
    assert np.array_equal(got, want)


def test_make_vit_model_is_complete():
    conf, amax, w = synth.make_vit(None, hidden=64, heads=1, ffn=128, n_layer=2, image=16, patch=4, seed=3)
    assert int(conf["max_step"]) == 17 and int(conf["image_size"]) == 16 and int(conf["patch_size"]) == 4 and int(conf["pre_ln"]) == 1
    assert w["conv.w"].shape == (64, 48) and w["pos"].shape == (17, 64) and "conv.w" not in amax
    for l in range(2):
        for n in ("qkv", "out", "fc1", "fc2"):
            for k in (".w", ".in", ".out"):
                assert amax[f"enc.{l}.{n}{k}"] > 0
    cfg = om.Config(hidden=64, heads=1, ffn=128, n_enc=2, n_dec=0, act="gelu", pre_ln=True)
    y = om.Vit(cfg, om.State(w=w, amax=amax), 4).forward(synth.vit_inputs(batch=2, image=16, seed=5))
    assert y.shape == (2, 17, 64) and np.isfinite(y).all() and abs(float(y.std()) - 1.0) < 0.05  # final LayerNorm
