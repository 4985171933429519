"""The vLLM adapter's host logic on the CPU, against fake layer objects (no vLLM model, no GPU): the weight-loading
hook of the sparse MoE path (clone -> vLLM's own processing -> 2:4 conversion -> apply swapped -> zero-stride stubs) and
the dense NVFP4 linear kernel's two methods.  The conversion and the ops are injected stand-ins built on the oracle."""
import types

import numpy as np
import torch

import oracle
from util import bf16_bits, oracle_quantize_fn


def _oracle_convert(weights, scales, g_scales, device="cpu", batch_size=16):
    comp, meta = [], []
    for e in range(weights.shape[0]):
        c, m = oracle.sparse_2of4_pack(weights[e].numpy())
        comp.append(torch.from_numpy(c)), meta.append(torch.from_numpy(m))
    return torch.stack(comp), torch.stack(meta), scales.view(torch.uint8).transpose(1, 2).contiguous(), g_scales.float()


def _fake_moe_layer(E=3, I=16, H=32, seed=0):
    import synth
    w13 = synth.make_dense_experts(E, 2 * I, H, seed, "cpu", oracle_quantize_fn)
    w2 = synth.make_dense_experts(E, H, I, seed + 1, "cpu", oracle_quantize_fn)
    P = lambda t: torch.nn.Parameter(t, requires_grad=False)
    layer = types.SimpleNamespace(
        w13_weight=P(w13["codes"].clone()), w2_weight=P(w2["codes"].clone()),
        w13_weight_scale=P(w13["sf"].clone()), w2_weight_scale=P(w2["sf"].clone()),
        w13_weight_scale_2=P((1.0 / w13["gs"]).reshape(E, 1).repeat(1, 2)), w2_weight_scale_2=P(1.0 / w2["gs"]))
    return layer, w13, w2


def test_moe_hook_converts_swaps_apply_and_stubs_the_originals():
    from dgx_vllm_b200 import vllm_adapter as va
    E, I, H = 3, 16, 32
    layer, w13, w2 = _fake_moe_layer(E, I, H)
    shapes = {n: tuple(getattr(layer, n).shape) for n in va._STUBBED_PARAMS}
    calls = []

    class Experts:
        def apply(self, *a):
            raise AssertionError("the original apply must have been replaced")

    method = types.SimpleNamespace(moe_mk=None)

    def original(m, l):                       # vLLM's own routine: repacks (here: scrambles) the weights, builds moe_mk
        calls.append("original")
        l.w13_weight.data.zero_()
        m.moe_mk = types.SimpleNamespace(fused_experts=Experts())

    captured = {}

    def make_apply(*args):
        captured["args"] = args
        return lambda *a: "v7"

    assert va.process_moe_layer(method, layer, original, convert_fn=_oracle_convert, device="cpu", make_apply=make_apply)
    assert calls == ["original"]
    assert method.moe_mk.fused_experts.apply() == "v7"
    # the closure got the 2:4 tensors of the ORIGINAL (pre-repacking) weights, first-column global scales, sizes
    c13, m13, s13, g13, c2, m2, s2, g2, inter, hidden = captured["args"]
    assert (inter, hidden) == (I, H)
    oc, om = oracle.sparse_2of4_pack(w13["codes"][1].numpy())
    np.testing.assert_array_equal(c13[1].numpy(), oc)
    np.testing.assert_array_equal(m13[1].numpy(), om)
    np.testing.assert_array_equal(s13[1].numpy(), w13["sf"][1].numpy().T)
    np.testing.assert_allclose(g13.numpy(), (1.0 / w13["gs"]).numpy(), rtol=1e-6)
    assert tuple(c2.shape) == (E, I // 4, H) and tuple(m2.shape) == (E, I // 8, H) and tuple(g2.shape) == (E,)
    # every original tensor is now a one-element stub that keeps its shape
    for n in va._STUBBED_PARAMS:
        p = getattr(layer, n)
        assert tuple(p.shape) == shapes[n] and set(p.data.stride()) == {0} and p.data.untyped_storage().nbytes() <= 8


def test_moe_hook_leaves_the_layer_alone_without_a_modular_kernel():
    from dgx_vllm_b200 import vllm_adapter as va
    layer, _, _ = _fake_moe_layer()
    method = types.SimpleNamespace()
    assert not va.process_moe_layer(method, layer, lambda m, l: None, convert_fn=_oracle_convert, device="cpu")
    assert layer.w13_weight.data.stride() != (0, 0, 0)


def test_apply_closure_call_shape():
    from dgx_vllm_b200 import vllm_adapter as va
    seen = {}

    def fused(hidden, tw, ids, emap, *rest):
        seen["tw_dtype"], seen["ids_dtype"], seen["emap"], seen["tail"] = tw.dtype, ids.dtype, emap, rest[-2:]
        return hidden.float() * 2

    fn = va.make_v7_apply_fn(*range(8), 16, 32, fused_fn=fused)
    out = torch.zeros(5, 32, dtype=torch.bfloat16)
    hidden = torch.ones(3, 32, dtype=torch.bfloat16)
    ret = fn(out, hidden, None, None, torch.ones(3, 2, dtype=torch.bfloat16), torch.zeros(3, 2, dtype=torch.int64), "silu", 8,
             None, None, None, None, None, None, True)
    assert ret is out and torch.all(out[:3] == 2) and torch.all(out[3:] == 0)
    assert seen["tw_dtype"] == torch.float32 and seen["ids_dtype"] == torch.int64 and seen["emap"] is None
    assert seen["tail"] == (16, True)


def test_dense_linear_kernel_methods_with_oracle_stand_ins():
    from dgx_vllm_b200 import vllm_adapter as va
    g = torch.Generator().manual_seed(0)
    M, N, K = 4, 32, 64
    x = torch.randn(2, M // 2, K, generator=g).bfloat16()
    w = (0.02 * torch.randn(N, K, generator=g)).bfloat16()
    gx, gw = float(oracle.global_scale(x.float().numpy())), float(oracle.global_scale(w.float().numpy()))
    wc, wsf = oracle.quantize_bf16(bf16_bits(w), gw)
    layer = types.SimpleNamespace(weight=torch.nn.Parameter(torch.from_numpy(wc), requires_grad=False),
                                  weight_scale=torch.nn.Parameter(torch.from_numpy(wsf), requires_grad=False),
                                  input_global_scale_inv=torch.tensor([gx]), alpha=torch.tensor([1.0 / (gx * gw)]),
                                  output_size_per_partition=N)
    swz = lambda sf: torch.from_numpy(oracle.sf_linear_to_swizzled(sf.numpy()))

    def quant(x2, gs, swizzled):
        c, s = oracle.quantize_bf16(bf16_bits(x2), float(gs[0]))
        return torch.from_numpy(c), torch.from_numpy(oracle.sf_linear_to_swizzled(s))

    def mm(a, b, sfa, sfb, alpha, dtype):
        ad = oracle.dequantize(a.numpy(), oracle.sf_swizzled_to_linear(sfa.numpy(), a.shape[0], K // 16), 1.0)
        bd = oracle.dequantize(b.numpy(), oracle.sf_swizzled_to_linear(sfb.numpy(), b.shape[0], K // 16), 1.0)
        return torch.from_numpy(oracle.matmul_nt(ad, bd) * float(alpha[0])).to(dtype)

    core = va.Nvfp4LinearCore(swizzle_fn=swz, quant_fn=quant, mm_fn=mm)
    core.process_weights_after_loading(layer)
    assert tuple(layer.weight_scale.shape) == (128, 4)                       # padded 128x4 tiles
    bias = torch.ones(N, dtype=torch.bfloat16)
    out = core.apply_weights(layer, x, bias)
    assert tuple(out.shape) == (2, M // 2, N) and out.dtype == torch.bfloat16
    ref = oracle.nvfp4_linear(bf16_bits(x.reshape(M, K)), gx, wc, wsf, gw) + 1.0
    assert np.max(np.abs(out.float().numpy().reshape(M, N) - ref)) <= 1e-2 * np.max(np.abs(ref))
