"""Host-side pieces of the path that need no GPU: the calibration statistic against the oracle,
and the method re-binding helper of quarot/monkeypatch.py against the reference's behaviour."""
import importlib.util
import os

import numpy as np
import pytest
import torch
from torch import nn

from oracle import oracle as O

REFERENCE_MONKEYPATCH = "/root/reference/quarot/monkeypatch.py"


# ---- get_act_scales_sam (RTN_quantization/calibration.py:16-69) -------------------------------

def _tiny_encoder(seed=11):
    from sam_quantization_b200.sam_encoder import build_encoder
    return build_encoder("vit_b", img_size=64, window_size=2, seed=seed, dtype=torch.float32, device="cpu",
                         attn_dtype=None, embed_dim=32, depth=3, num_heads=2, global_attn_indexes=(1,), out_chans=8)


def test_get_act_scales_sam_equals_oracle_running_max():
    """The statistic of every hooked linear equals the oracle's ``act_scales_running_max`` over
    the inputs that linear saw, captured here by independent hooks; names, count and dtype follow
    the reference (fp32 on the CPU, keys ``image_encoder.blocks.{i}.attn.qkv`` ...)."""
    from sam_quantization_b200.RTN_quantization import get_act_scales_sam
    model = _tiny_encoder()
    g = torch.Generator().manual_seed(5)
    batches = [torch.randn(2, 3, 64, 64, generator=g) * (1 + i) for i in range(3)]

    seen = {}
    hooks = []
    for name, mod in model.image_encoder.named_modules():
        if isinstance(mod, nn.Linear):
            hooks.append(mod.register_forward_hook(
                lambda m, inp, out, name=name: seen.setdefault("image_encoder." + name, []).append(inp[0].detach().numpy().copy())))
    with torch.no_grad():
        for b in batches:
            model.image_encoder(b)
    for h in hooks:
        h.remove()

    scales = get_act_scales_sam(model, iter(batches), num_samples=8)
    assert sorted(scales) == sorted(seen)
    assert len(scales) == 3 * 4                          # qkv, proj, lin1, lin2 of three blocks
    for name, inputs in seen.items():
        want = O.act_scales_running_max(inputs)
        got = scales[name]
        assert got.dtype == torch.float32 and got.device.type == "cpu"
        assert got.shape == (inputs[0].shape[-1],)
        assert np.array_equal(got.numpy(), want), name
    # hooks are gone afterwards and num_samples bounds the batches consumed
    assert all(len(m._forward_hooks) == 0 for m in model.modules())
    first_only = get_act_scales_sam(model, iter(batches), num_samples=1)
    for name, inputs in seen.items():
        assert np.array_equal(first_only[name].numpy(), O.act_scales_running_max(inputs[:1])), name


def test_get_act_scales_sam_half_inputs_are_widened():
    """fp16 activations are reduced in their own dtype and widened to fp32 (calibration.py:43-46)."""
    from sam_quantization_b200.RTN_quantization import get_act_scales_sam

    class Enc(nn.Module):
        def __init__(self):
            super().__init__()
            self.blocks = nn.ModuleList([nn.ModuleDict({"attn": nn.ModuleDict({"qkv": nn.Linear(8, 8)})})])

        def forward(self, x):
            return self.blocks[0]["attn"]["qkv"](x)

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.image_encoder = Enc()

    model = Model().to(torch.bfloat16)
    x = (torch.randn(4, 5, 8, generator=torch.Generator().manual_seed(1)) * 3).to(torch.bfloat16)
    scales = get_act_scales_sam(model, [x])
    want = O.act_scales_running_max([x.float().numpy()])
    assert np.array_equal(scales["image_encoder.blocks.0.attn.qkv"].numpy(), want)


# ---- quarot/monkeypatch.py:5-28 -----------------------------------------------------------------

def helper(v):
    return v + 1


def indirect(v):
    return helper(v)


class Host:
    bonus = 100

    def method(self, v, *, scale=2):
        """doc of method"""
        return helper(v) * scale + indirect(v) + self.bonus


def _times_ten(fn):
    def wrapped(*a, **k):
        wrapped.calls += 1
        return fn(*a, **k) * 10
    wrapped.calls = 0
    return wrapped


def _exercise(mp):
    a, b = Host(), Host()
    before = a.method(1)                                  # helper(1)*2 + indirect(1) + 100 = 4 + 2 + 100
    wrapper = mp.add_wrapper_after_function_call_in_method(a, "method", "helper", _times_ten)
    after = a.method(1)                                   # direct call wrapped (20*2), indirect call not
    return {
        "before": before, "after": after, "other_instance": b.method(1), "module_global_untouched": helper(1),
        "calls": wrapper.calls, "kw": a.method(1, scale=3), "doc": a.method.__doc__, "name": a.method.__name__,
        "bound_to": a.method.__self__ is a, "class_untouched": Host.method is type(b).method and "method" not in vars(b),
    }


def test_add_wrapper_after_function_call_in_method():
    from sam_quantization_b200.quarot import monkeypatch as mine
    got = _exercise(mine)
    assert got == {"before": 106, "after": 142, "other_instance": 106, "module_global_untouched": 2, "calls": 1,
                   "kw": 162, "doc": "doc of method", "name": "method", "bound_to": True, "class_untouched": True}
    f = mine.copy_func_with_new_globals(indirect, {"helper": lambda v: -v})
    assert f(3) == -3 and indirect(3) == 4 and f.__name__ == "indirect"


@pytest.mark.skipif(not os.path.exists(REFERENCE_MONKEYPATCH), reason="reference checkout not present")
def test_monkeypatch_behaves_like_the_reference_module():
    """Where the reference checkout is mounted, the same scenario run through its own module
    gives the same observations."""
    spec = importlib.util.spec_from_file_location("ref_monkeypatch", REFERENCE_MONKEYPATCH)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    from sam_quantization_b200.quarot import monkeypatch as mine
    assert _exercise(mine) == _exercise(ref)


# ---- argument checks that run before any kernel --------------------------------------------------

def test_group_sizes_the_int8_gemm_cannot_run_are_rejected_at_construction():
    """The reference's float path takes any group size that divides the width; the int8 GEMM needs
    multiples of 32 and at most 160 groups, and says so when the module is built, not at the
    first forward."""
    from sam_quantization_b200.RTN_quantization import W8A8Linear
    from sam_quantization_b200.quarot.utils import ActQuantWrapper
    lin = nn.Linear(96, 8)
    with pytest.raises(ValueError, match="multiples of 32"):
        W8A8Linear.from_float(lin, 8, weight_quant="per_group", act_quant="per_token", group_size=24)
    with pytest.raises(ValueError, match="multiples of 32"):
        W8A8Linear.from_float(lin, 8, weight_quant="per_channel", act_quant="per_group_token", group_size=48)
    with pytest.raises(ValueError, match="multiples of 32"):
        ActQuantWrapper(lin, act_quant="per_group_token", weight_quant="per_group", group_size=16)
    with pytest.raises(AssertionError):
        W8A8Linear.from_float(lin, 8, weight_quant="per_group", group_size=64)       # does not divide 96
    with pytest.raises(ValueError, match="160 groups"):
        W8A8Linear.from_float(nn.Linear(32 * 161, 8), 8, weight_quant="per_group", group_size=32)


def test_half_precision_hadamard_with_an_explicit_factor_is_refused():
    """``fp32_had=False`` with a non-power-of-two transform length raises instead of returning the
    one-rounding fp32 result under the name of the reference's two-rounding half path."""
    from sam_quantization_b200.quarot.utils import ActQuantWrapper
    w = ActQuantWrapper(nn.Linear(96, 8), weight_quant=None)
    w.online_full_had, w.K, w.fp32_had = True, 12, False
    with pytest.raises(NotImplementedError, match="fp32_had=True"):
        w._hadamard_spec(torch.zeros(2, 96))
    w.fp32_had = True
    w.had_K = torch.ones(12, 12)
    assert w._hadamard_spec(torch.zeros(2, 96)).had_k == 12
    w.K, w.fp32_had, w.had_K = 1, False, None           # powers of two: both settings run the same kernel
    assert w._hadamard_spec(torch.zeros(2, 96)).had_k == 1
