"""Pins oracle/torch_twin.py (the float twin used for encoder-level parity) to the reference's
own W8A8Linear: layer outputs bit for bit, and the small encoder's embeddings."""
import numpy as np
import pytest
import torch

from oracle.torch_twin import RefW8A8Linear, replace_linears
from tests.golden.make_golden import TINY, tiny_images

TDT = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}
COMBOS = [("per_channel", "per_token", None, 0), ("per_tensor", "per_tensor", None, 0),
          ("per_group", "per_group_token", 32, 0), ("per_channel", "per_token", None, 1),
          ("per_group", "per_token", 128, 0)]


@pytest.mark.parametrize("dt", ["f16", "bf16", "f32"])
def test_twin_linear_equals_reference_class(golden, dt):
    g = golden("w8a8_linear")
    x = torch.from_numpy(g[f"{dt}/x"]).to(TDT[dt])
    w = torch.from_numpy(g[f"{dt}/w"]).to(TDT[dt])
    b = torch.from_numpy(g[f"{dt}/b"]).to(TDT[dt])
    for wq, aq, gs, qo in COMBOS:
        lin = torch.nn.Linear(256, 72)
        lin.weight.data, lin.bias.data = w.clone(), b.clone()
        y = RefW8A8Linear.from_float(lin, 8, wq, aq, bool(qo), gs)(x.clone())
        assert np.array_equal(y.float().numpy(), g[f"{dt}/y/{wq}/{aq}/{gs}/{qo}"]), (wq, aq, gs, qo)


def test_twin_encoder_equals_reference_encoder(golden):
    from sam_quantization_b200.sam_encoder import build_encoder
    g = golden("encoder_tiny")
    for tag, kw in (("w8a8", dict(weight_quant="per_channel", act_quant="per_token", quantize_output=False)),
                    ("w8a8_qout", dict(weight_quant="per_channel", act_quant="per_token", quantize_output=True))):
        model = build_encoder(seed=5, dtype=torch.float32, attn_dtype=None, **TINY)
        replace_linears(model, lambda lin: RefW8A8Linear.from_float(lin, 8, **kw))
        with torch.no_grad():
            emb = model(tiny_images()).numpy()
        want = g[f"{tag}/embedding"]
        assert np.abs(emb - want).max() <= 1e-4 * np.abs(want).max()


def test_twin_random_hadamard_equals_reference(golden):
    """The twin's Q = hadU(diag(signs)) is the reference's ``random_hadamard_matrix(seed=123)``
    byte for byte (digest recorded from the reference's function)."""
    import hashlib
    from oracle.torch_twin import random_hadamard_Q
    g = golden("hadamard")
    sizes = sorted(int(k.split("/")[1]) for k in g.files if k.startswith("randhad/") and k.endswith("/sha256"))
    assert sizes
    for n in sizes:
        if n & (n - 1):
            continue                                      # the twin's helper covers powers of two
        signs, Q = random_hadamard_Q(n, 123)
        assert hashlib.sha256(Q.numpy().tobytes()).hexdigest() == str(g[f"randhad/{n}/sha256"])
        assert torch.equal((Q * signs.view(-1, 1))[0], torch.full((n,), 1.0 / n ** 0.5, dtype=torch.float64))   # Q = diag(signs) H / sqrt(n)


def test_twin_rotation_is_an_exact_change_of_basis():
    """Weights rotated by the twin's restatement of ``rotate_model_sam`` plus the online
    transforms of ``ActQuantWrapper`` (sign flip + transform before qkv / lin1, full transform
    before lin2, across-heads transform before proj) reproduce the unrotated float encoder."""
    import copy
    from oracle.torch_twin import RefActQuantWrapper, random_hadamard_Q, rotate_encoder_weights
    from sam_quantization_b200.sam_encoder import build_encoder
    kw = dict(TINY)
    kw.update(embed_dim=32, num_heads=4)
    model = build_encoder(seed=9, dtype=torch.float32, attn_dtype=None, **kw)
    rot = copy.deepcopy(model)
    signs, Q = random_hadamard_Q(32, 123)
    rotate_encoder_weights(rot, Q, 32, 4)
    replace_linears(rot, lambda lin: RefActQuantWrapper(lin, weight_quant=None))
    for blk in rot.image_encoder.blocks:
        blk.attn.qkv.pre_signs = blk.mlp.lin1.pre_signs = signs
        blk.mlp.lin2.online_full_had = True
        blk.attn.proj.online_partial_had, blk.attn.proj.had_dim = True, 8
    x = tiny_images()
    with torch.no_grad():
        a, b = model(x), rot(x)
    assert (a - b).abs().max() <= 2e-4 * a.abs().max()
    # and the rotation did change the weights
    assert not torch.allclose(model.image_encoder.blocks[0].attn.qkv.weight, rot.image_encoder.blocks[0].attn.qkv.module.weight)
