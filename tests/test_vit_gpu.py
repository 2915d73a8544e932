"""QuantVit: the patch-embedding kernel against the oracle (bit-exact: float64 dot products rounded once) and the
engine (pybind surface) against the numpy oracle on seeded synthetic ViT-shaped models. As for BERT, every stage is
bit-exact except attention, whose rare one-step int8 flips spread through the later quantisers of that image; the
tolerances on the fp32 output are those of tests/test_bert_gpu.py."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from lightseq_b200 import _lib as L  # noqa: E402
from lightseq_b200 import synth  # noqa: E402
from oracle import model as om  # noqa: E402

F32 = np.float32


@pytest.mark.parametrize("B,C,image,patch,H", [(3, 3, 32, 8, 128), (2, 3, 224, 16, 768), (5, 1, 28, 7, 64), (1, 3, 48, 16, 300)])
def test_patch_embed_is_bit_exact(B, C, image, patch, H):
    w = synth.vit_weights(hidden=H, heads=max(H // 64, 1), ffn=4, n_layer=0, image=image, patch=patch, channels=C, seed=B)
    px = synth.vit_inputs(batch=B, image=image, channels=C, seed=7)
    ref = om.patch_embed(w, px, patch)
    ctx = L.Context(0)
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=F32)).cuda()  # noqa: E731
    dpx, dwt, db, dpos, dcls = d(px), d(w["conv.w"].T), d(w["conv.b"]), d(w["pos"]), d(w["cls"])
    out = torch.empty(ref.shape, dtype=torch.float32, device="cuda")
    args = L.PatchEmbedArgs(pixels=dpx.data_ptr(), conv_wt=dwt.data_ptr(), conv_bias=db.data_ptr(), pos=dpos.data_ptr(),
                            cls=dcls.data_ptr(), batch=B, channels=C, image=image, patch=patch, hidden=H, out=out.data_ptr())
    L.call("ls100_patch_embed", ctx, args)
    torch.cuda.synchronize()
    assert ctx.poll_error() == 0
    assert np.array_equal(out.cpu().numpy(), ref)


@pytest.mark.parametrize("hidden,heads,ffn,layers,image,patch,batch", [(128, 2, 256, 2, 32, 8, 5), (768, 12, 3072, 2, 112, 16, 3)])
def test_vit_output_matches_oracle(tmp_path, hidden, heads, ffn, layers, image, patch, batch):
    import lightseq_b200.inference as lsi

    path = str(tmp_path / "vit.ls100")
    conf, amax, w = synth.make_vit(path, hidden=hidden, heads=heads, ffn=ffn, n_layer=layers, image=image, patch=patch, seed=13)
    cfg = om.Config(hidden=hidden, heads=heads, ffn=ffn, n_enc=layers, n_dec=0, act="gelu", pre_ln=True)
    px = synth.vit_inputs(batch=batch, image=image, seed=3)
    ref = om.Vit(cfg, om.State(w=w, amax=amax), patch).forward(px)
    model = lsi.QuantVit(path, batch)
    out = model.infer(px)
    assert out.shape == ref.shape == (batch, 1 + (image // patch) ** 2, hidden) and out.dtype == np.float32
    d = np.abs(out - ref)
    print("vit max abs", d.max(), "mean abs", d.mean(), "exact fraction", (d == 0).mean())
    assert d.max() < 6e-2 and d.mean() < 5e-3
    assert np.array_equal(out, model.infer(px))  # deterministic
    with pytest.raises(RuntimeError, match="max_batch_size"):
        model.infer(np.zeros((batch + 1, 3, image, image), F32))
    with pytest.raises(RuntimeError, match="pixel_input"):
        model.infer(np.zeros((1, 3, image // 2, image // 2), F32))
