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
