"""GPU parity of the quantizer (C ABI through dgx_vllm_b200.ops) against the oracle and goldens:
codes and scales must be bit-exact."""
import os

import numpy as np
import pytest
import torch

import oracle
from util import bf16_bits, from_bf16_bits, to_np

pytestmark = pytest.mark.gpu


def _quant(x, gs, swz):
    from dgx_vllm_b200 import scaled_fp4_quant
    g = torch.tensor([gs], dtype=torch.float32, device="cuda")
    codes, sf = scaled_fp4_quant(x.cuda(), g, is_sf_swizzled_layout=swz)
    torch.cuda.synchronize()
    return to_np(codes), to_np(sf)


def test_c1_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "dense_c1.npz"))
    x = from_bf16_bits(g["x_bits"])
    codes, sf = _quant(x, float(g["gs_x"][0]), False)
    np.testing.assert_array_equal(codes, g["x_codes"])
    np.testing.assert_array_equal(sf, g["x_sf"])
    codes2, sfs = _quant(x, float(g["gs_x"][0]), True)
    np.testing.assert_array_equal(codes2, g["x_codes"])
    np.testing.assert_array_equal(sfs, oracle.sf_linear_to_swizzled(g["x_sf"]))


@pytest.mark.parametrize("name", ["amax", "one", "big", "tiny"])
def test_kat_golden(golden_dir, name):
    g = np.load(os.path.join(golden_dir, "quant_kat.npz"))
    gs = float(g[f"gs_{name}"][0])
    codes, sf = _quant(from_bf16_bits(g["x_bits"]), gs, False)
    ocodes, osf = oracle.quantize_bf16(g["x_bits"], gs)
    np.testing.assert_array_equal(sf, g[f"sf_{name}"])
    np.testing.assert_array_equal(sf, osf)
    np.testing.assert_array_equal(codes, ocodes)


@pytest.mark.parametrize("M,K", [(1, 16), (7, 64), (129, 80), (300, 4096), (128, 2048), (5, 8192)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_random_shapes(M, K, dtype):
    gen = torch.Generator().manual_seed(M * 131 + K)
    x = (torch.randn(M, K, generator=gen) * torch.logspace(-3, 1, M).unsqueeze(1)).to(dtype)
    gs = float(oracle.global_scale(x.float().numpy()))
    if dtype == torch.bfloat16:
        ocodes, osf = oracle.quantize_bf16(bf16_bits(x), gs)
    else:
        ocodes, osf = oracle.quantize_f32(x.float().numpy(), gs)
    for swz in (False, True):
        codes, sf = _quant(x, gs, swz)
        np.testing.assert_array_equal(codes, ocodes)
        if swz:
            np.testing.assert_array_equal(sf, oracle.sf_linear_to_swizzled(osf))
        else:
            np.testing.assert_array_equal(sf, osf)


def test_full_size_prefill_activation():
    # the largest activation of the dense prefill configuration: 4096 x 4096 bf16 ~ N(0,1)
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(4096, 4096, generator=gen).to(torch.bfloat16)
    gs = float(oracle.global_scale(x.float().numpy()))
    ocodes, osf = oracle.quantize_bf16(bf16_bits(x), gs)
    codes, sf = _quant(x, gs, True)
    np.testing.assert_array_equal(codes, ocodes)
    np.testing.assert_array_equal(sf, oracle.sf_linear_to_swizzled(osf))
    # size-independent property: dequantized error is bounded by half a code step of each block
    deq = oracle.dequantize(codes, osf, gs)
    blk = np.abs(x.float().numpy()).reshape(4096, 256, 16).max(-1, keepdims=True)
    err = np.abs(deq - x.float().numpy()).reshape(4096, 256, 16)
    assert np.all(err <= blk * 0.25 + 1e-12)


def test_strided_rows_and_empty():
    from dgx_vllm_b200 import scaled_fp4_quant
    gen = torch.Generator().manual_seed(5)
    big = torch.randn(16, 256, generator=gen).to(torch.bfloat16).cuda()
    view = big[:, :128]
    gs = torch.tensor([100.0], dtype=torch.float32, device="cuda")
    codes, sf = scaled_fp4_quant(view, gs, False)
    oc, osf = oracle.quantize_bf16(bf16_bits(view.contiguous()), 100.0)
    np.testing.assert_array_equal(to_np(codes), oc)
    np.testing.assert_array_equal(to_np(sf), osf)
    c0, s0 = scaled_fp4_quant(big[:0], gs, False)
    assert c0.shape == (0, 128) and s0.shape == (0, 16)
    with pytest.raises(RuntimeError):
        scaled_fp4_quant(big[:, :24], gs, False)          # K not a multiple of 16
    with pytest.raises(RuntimeError):
        scaled_fp4_quant(big.cpu(), gs.cpu(), False)      # no CPU path
