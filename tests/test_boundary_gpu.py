"""GPU tests of the drop-in boundary: the ops called exactly the way the reference's own call sites call them, the
reference's declared C API (cutlass_nvfp4/cuda_fp4_gemm.h) through ctypes, and the fused layer's status word."""
import ctypes
import importlib
import os
import sys

import numpy as np
import pytest
import torch

import oracle
from util import bf16_bits, oracle_quantize_fn, rel_err, to_np

pytestmark = pytest.mark.gpu
TOL = 1e-2
KEYS = ("comp_T", "meta_T", "scale_T", "g_scales")


def _layer(E, H, I, seed):
    import synth
    w13 = synth.make_sparse_experts(E, 2 * I, H, seed, "cpu", oracle_quantize_fn)
    w2 = synth.make_sparse_experts(E, H, I, seed + 1, "cpu", oracle_quantize_fn)
    return w13, w2


def _oracle_layer(w13, w2, hidden, tw, ids, I, on_input=False):
    n = lambda d: tuple(d[k].numpy() for k in KEYS)
    return oracle.fused_sparse_moe(hidden.float().numpy(), tw.numpy(), ids.numpy(), None, n(w13), n(w2), I,
                                   apply_router_weight_on_input=on_input, round_fp16=False)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fused_op_called_like_the_reference_apply_closure(dtype):
    # v7_apply, sparse_fp4_kernel/sparse_v7_moe_patch.py:216-230: a CPU empty int32 expert_map, topk_weights.float(),
    # int64 topk_ids straight from the router, and output[:M] = result.to(output.dtype) into a larger buffer
    import synth
    from dgx_vllm_b200 import sparse_fp4_v7 as sp7
    E, H, I, M, topk = 16, 512, 256, 7, 4
    w13, w2 = _layer(E, H, I, 3)
    tw, ids = synth.make_routing(M, E, topk, 5, "cpu")
    hidden = synth.make_hidden(M, H, 6, "cpu", dtype)
    dev13 = [w13[k].cuda() for k in KEYS]
    dev2 = [w2[k].cuda() for k in KEYS]
    _empty_map = torch.empty(0, dtype=torch.int32)                      # on the CPU, as in the reference
    topk_weights = tw.cuda().to(torch.bfloat16)                         # the router's dtype; the closure calls .float()
    topk_ids = ids.cuda().to(torch.int64)
    output = torch.full((M + 3, H), 7.0, dtype=dtype, device="cuda")    # vLLM hands a workspace that may be larger
    result = sp7.fused_sparse_moe_v7(hidden.cuda(), topk_weights.float(), topk_ids, _empty_map, *dev13, *dev2, I, False)
    output[:M] = result.to(output.dtype)
    ref = _oracle_layer(w13, w2, hidden, topk_weights.float().cpu(), ids, I)
    assert rel_err(to_np(output[:M]), ref) < TOL
    assert torch.all(output[M:] == 7.0)
    assert sp7.last_moe_status() == 0


def test_two_gemv_calls_like_sparse_v7_experts_apply():
    # SparseV7Experts.apply, sparse_v7_moe_patch.py:153-193: replicate tokens, batched_sparse_v7 for gate_up, torch SiLU
    # on slices of its output (non-contiguous views), batched_sparse_v7 for down, weighted sum in torch
    import synth
    from dgx_vllm_b200 import sparse_fp4_v7 as sp7
    E, H, I, M, topk = 8, 512, 256, 5, 3
    w13, w2 = _layer(E, H, I, 9)
    tw, ids = synth.make_routing(M, E, topk, 10, "cpu")
    hidden_states = synth.make_hidden(M, H, 11, "cpu", torch.float16).cuda()
    topk_ids, topk_weights = ids.cuda().long(), tw.cuda()
    A = hidden_states.unsqueeze(1).expand(-1, topk, -1).reshape(M * topk, H).contiguous()
    eid = topk_ids.reshape(-1).int()
    gate_up = sp7.batched_sparse_v7(A, *[w13[k].cuda() for k in KEYS], eid)
    gate, up = gate_up[:, :I], gate_up[:, I:]
    intermediate = torch.nn.functional.silu(gate) * up
    down = sp7.batched_sparse_v7(intermediate, *[w2[k].cuda() for k in KEYS], eid)
    reduced = (down.view(M, topk, -1).float() * topk_weights.unsqueeze(-1).float()).sum(1)
    ref = oracle.fused_sparse_moe(hidden_states.float().cpu().numpy(), tw.numpy(), ids.numpy(), None,
                                  tuple(w13[k].numpy() for k in KEYS), tuple(w2[k].numpy() for k in KEYS), I,
                                  round_fp16=True)
    assert rel_err(to_np(reduced), ref) < TOL


def test_reference_patch_module_runs_on_this_library():
    # the reference's own sparse_v7_moe_patch.py, unmodified, importing this package as `sparse_fp4_v7`; needs a
    # checkout of the reference (DGX_VLLM_REFERENCE=/path/to/dgx-vllm)
    root = os.environ.get("DGX_VLLM_REFERENCE")
    if not root or not os.path.exists(os.path.join(root, "sparse_fp4_kernel", "sparse_v7_moe_patch.py")):
        pytest.skip("DGX_VLLM_REFERENCE does not point at a checkout of the reference")
    import synth
    import dgx_vllm_b200.sparse_fp4_v7 as sp7
    saved = sys.modules.get("sparse_fp4_v7")
    sys.modules["sparse_fp4_v7"] = sp7
    sys.path.insert(0, os.path.join(root, "sparse_fp4_kernel"))
    try:
        patch = importlib.import_module("sparse_v7_moe_patch")
        E, H, I, M, topk = 8, 512, 256, 4, 2
        w13, w2 = _layer(E, H, I, 21)
        tw, ids = synth.make_routing(M, E, topk, 22, "cpu")
        hidden = synth.make_hidden(M, H, 23, "cpu")
        experts = patch.SparseV7Experts(*[w13[k].cuda() for k in KEYS], *[w2[k].cuda() for k in KEYS], I, H)
        out = torch.zeros(M, H, dtype=torch.bfloat16, device="cuda")
        experts.apply(out, hidden.cuda(), None, None, tw.cuda(), ids.cuda().long(), "silu", E, None, None, None, None, None,
                      None, False)
        ref = _oracle_layer(w13, w2, hidden, tw, ids, I)
        assert rel_err(to_np(out), ref) < 2e-2              # two bf16 roundings of intermediates in the torch glue
        fn = patch._make_v7_apply_fn(*[w13[k].cuda() for k in KEYS], *[w2[k].cuda() for k in KEYS], I, H)
        out2 = torch.zeros(M + 1, H, dtype=torch.bfloat16, device="cuda")
        fn(out2, hidden.cuda(), None, None, tw.cuda(), ids.cuda().long(), "silu", E, None, None, None, None, None, None, False)
        assert rel_err(to_np(out2[:M]), ref) < TOL
    finally:
        sys.path.pop(0)
        if saved is None:
            sys.modules.pop("sparse_fp4_v7", None)
        else:
            sys.modules["sparse_fp4_v7"] = saved


def test_fused_layer_wait_that_runs_out_sets_the_status_word_and_returns():
    # one-launch layer (<= 256 pairs): with one more finished gate_up item asked for than a pass ever has, and a
    # budget of ~50 us, the first wait gives up, records the status and every later wait is skipped; the kernel
    # returns and the context stays usable.  Nothing is in flight when a wait gives up (a plain counter poll).
    import synth
    from dgx_vllm_b200 import _lib, sparse_fp4_v7 as sp7
    L = _lib.lib()
    E, H, I, M, topk = 16, 2048, 512, 8, 4
    w13, w2 = _layer(E, H, I, 31)
    tw, ids = synth.make_routing(M, E, topk, 32, "cpu")
    hidden = synth.make_hidden(M, H, 33, "cpu")
    args = (hidden.cuda(), tw.cuda(), ids.cuda(), torch.empty(0, dtype=torch.int32), *[w13[k].cuda() for k in KEYS],
            *[w2[k].cuda() for k in KEYS], I, False)
    try:
        L.b200fp4_fused_moe_set_wait_limit(100000, 1)
        sp7.fused_sparse_moe_v7(*args)
        assert sp7.last_moe_status() == -1
    finally:
        L.b200fp4_fused_moe_set_wait_limit(0, 0)
    out = sp7.fused_sparse_moe_v7(*args)                        # the next call clears the word and is correct
    assert sp7.last_moe_status() == 0
    assert rel_err(to_np(out), _oracle_layer(w13, w2, hidden, tw, ids, I)) < TOL


def test_reference_c_api_through_ctypes(golden_dir):
    # cudaFP4Create / SetStream / Quantize / GemmEx / ConvertFromFP32 / ConvertToFP32 / Destroy with the prototypes of
    # cutlass_nvfp4/cuda_fp4_gemm.h, on the reference's CPU-runnable dense case (x 8x2048, W 512x2048)
    from dgx_vllm_b200 import _lib
    L = _lib.lib()
    g = np.load(os.path.join(golden_dir, "dense_c1.npz"))
    x = oracle.bf16_bits_to_f32(g["x_bits"])
    w = oracle.dequantize(g["w_codes"], g["w_sf"], float(g["gs_w"][0]))         # the golden weight, as an fp32 matrix
    M, K = x.shape
    N = w.shape[0]
    assert L.cudaFP4HasHardwareAcceleration() == 1 and L.cudaFP4GetVersion() == L.b200fp4_version()
    assert L.cudaFP4GetErrorString(15) == L.b200fp4_get_error_string(15)
    h = ctypes.c_void_p()
    assert L.cudaFP4Create(ctypes.byref(h)) == 0
    stream = torch.cuda.Stream()
    assert L.cudaFP4SetStream(h, stream.cuda_stream) == 0
    with torch.cuda.stream(stream):
        xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
        q = {}
        for name, t in (("x", xd), ("w", wd)):
            codes = torch.empty(t.shape[0], K // 2, dtype=torch.uint8, device="cuda")
            sf = torch.empty(t.shape[0], K // 16, dtype=torch.uint8, device="cuda")
            gl = ctypes.c_float(0)
            assert L.cudaFP4Quantize(codes.data_ptr(), sf.data_ptr(), ctypes.addressof(gl), t.data_ptr(), t.shape[0], K, 16,
                                     stream.cuda_stream) == 0
            q[name] = (codes, sf, gl.value)
            # bit-exact with the oracle's fp32 quantizer at the same global scale, global = amax / (6 * 448)
            gs = oracle.global_scale(t.cpu().numpy())
            oc, osf = oracle.quantize_f32(t.cpu().numpy(), float(gs))
            np.testing.assert_array_equal(to_np(codes), oc)
            np.testing.assert_array_equal(to_np(sf), osf)
            assert abs(gl.value * float(gs) - 1.0) < 1e-6
        C = torch.empty(M, N, dtype=torch.float32, device="cuda")
        assert L.cudaFP4GemmEx(h, M, N, K, q["x"][0].data_ptr(), q["x"][1].data_ptr(), q["x"][2], q["w"][0].data_ptr(),
                               q["w"][1].data_ptr(), q["w"][2], C.data_ptr(), 16) == 0
        assert L.cudaFP4GemmEx(h, M, N, K, q["x"][0].data_ptr(), q["x"][1].data_ptr(), q["x"][2], q["w"][0].data_ptr(),
                               q["w"][1].data_ptr(), q["w"][2], C.data_ptr(), 32) == 15        # group size 16 only
        stream.synchronize()
        ref = oracle.matmul_nt(oracle.dequantize(to_np(q["x"][0]), to_np(q["x"][1]), 1.0 / q["x"][2]),
                               oracle.dequantize(to_np(q["w"][0]), to_np(q["w"][1]), 1.0 / q["w"][2]))
        assert rel_err(to_np(C), ref) < 1e-4                       # fp32 output: no 16-bit rounding of the result
        # uniform-scale form and the element-wise converters
        vals = torch.tensor([[0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.5, -6.0, 0.25, 0.75, 1.25, 2.5, 5.0, 100.0] * 4] * 128,
                            dtype=torch.float32, device="cuda")
        packed = torch.empty(128, 32, dtype=torch.uint8, device="cuda")
        back = torch.empty_like(vals)
        assert L.cudaFP4ConvertFromFP32(packed.data_ptr(), vals.data_ptr(), 128, 64, stream.cuda_stream) == 0
        assert L.cudaFP4ConvertToFP32(back.data_ptr(), packed.data_ptr(), 128, 64, stream.cuda_stream) == 0
        stream.synchronize()
        want = np.array([oracle.e2m1_decode(oracle.e2m1_encode(float(v))) for v in vals[0].cpu().numpy()], np.float32)
        np.testing.assert_array_equal(to_np(back)[5], want)        # ties to even: 0.25 -> 0, 0.75 -> 1, 2.5 -> 2, 5 -> 4
        C2 = torch.empty(128, 128, dtype=torch.float32, device="cuda")
        assert L.cudaFP4Gemm(h, 128, 128, 64, ctypes.c_float(0.5), packed.data_ptr(), packed.data_ptr(), C2.data_ptr()) == 0
        stream.synchronize()
        assert rel_err(to_np(C2), 0.5 * (to_np(back) @ to_np(back).T)) < 1e-5
    assert L.cudaFP4Destroy(h) == 0


def test_vllm_adapter_hook_and_closure_on_the_gpu():
    # the weight-loading hook on a fake layer that lives on the GPU, with the CUDA converter, then the closure it installs
    # called the way vLLM calls MarlinExperts.apply; the yardstick is the oracle over the oracle's own 2:4 conversion
    import types
    import synth
    from dgx_vllm_b200 import vllm_adapter as va
    E, I, H, M, topk = 8, 128, 256, 6, 2
    w13 = synth.make_dense_experts(E, 2 * I, H, 41, "cpu", oracle_quantize_fn)
    w2 = synth.make_dense_experts(E, H, I, 42, "cpu", oracle_quantize_fn)
    P = lambda t: torch.nn.Parameter(t.cuda(), requires_grad=False)
    layer = types.SimpleNamespace(w13_weight=P(w13["codes"]), w2_weight=P(w2["codes"]), w13_weight_scale=P(w13["sf"]),
                                  w2_weight_scale=P(w2["sf"]), w13_weight_scale_2=P(1.0 / w13["gs"]),
                                  w2_weight_scale_2=P(1.0 / w2["gs"]))
    experts = types.SimpleNamespace(apply=None)
    method = types.SimpleNamespace(moe_mk=None)

    def original(m, l):
        m.moe_mk = types.SimpleNamespace(fused_experts=experts)

    assert va.process_moe_layer(method, layer, original)
    assert layer.w13_weight.data.stride() == (0, 0, 0) and tuple(layer.w13_weight.shape) == (E, 2 * I, H // 2)
    tw, ids = synth.make_routing(M, E, topk, 43, "cpu")
    hidden = synth.make_hidden(M, H, 44, "cpu")
    out = torch.zeros(M + 2, H, dtype=torch.bfloat16, device="cuda")
    ret = experts.apply(out, hidden.cuda(), layer.w13_weight, layer.w2_weight, tw.cuda(), ids.cuda().long(), "silu", E, None,
                        None, None, None, None, None, False)
    assert ret is out

    def sparse(w):
        comp, meta = zip(*[oracle.sparse_2of4_pack(w["codes"][e].numpy()) for e in range(E)])
        return np.stack(comp), np.stack(meta), np.ascontiguousarray(w["sf"].numpy().transpose(0, 2, 1)), (1.0 / w["gs"]).numpy()

    ref = oracle.fused_sparse_moe(hidden.float().numpy(), tw.numpy(), ids.numpy(), None, sparse(w13), sparse(w2), I,
                                  round_fp16=False)
    assert rel_err(to_np(out[:M]), ref) < TOL and torch.all(out[M:] == 0)


def test_vllm_adapter_dense_linear_and_scale_swizzle():
    import types
    from dgx_vllm_b200 import vllm_adapter as va
    g = torch.Generator().manual_seed(5)
    M, N, K = 24, 384, 512
    x = torch.randn(2, M // 2, K, generator=g).bfloat16()
    w = (0.02 * torch.randn(N, K, generator=g)).bfloat16()
    gx, gw = float(oracle.global_scale(x.float().numpy())), float(oracle.global_scale(w.float().numpy()))
    wc, wsf = oracle.quantize_bf16(bf16_bits(w), gw)
    swz = va.swizzle_blockscale(torch.from_numpy(wsf).cuda())
    np.testing.assert_array_equal(to_np(swz), oracle.sf_linear_to_swizzled(wsf))
    layer = types.SimpleNamespace(weight=torch.nn.Parameter(torch.from_numpy(wc).cuda(), requires_grad=False),
                                  weight_scale=torch.nn.Parameter(torch.from_numpy(wsf).cuda().view(torch.float8_e4m3fn), requires_grad=False),
                                  input_global_scale_inv=torch.tensor([gx], device="cuda"),
                                  alpha=torch.tensor([1.0 / (np.float32(gx) * np.float32(gw))], dtype=torch.float32, device="cuda"),
                                  output_size_per_partition=N)
    core = va.Nvfp4LinearCore()
    core.process_weights_after_loading(layer)
    out = core.apply_weights(layer, x.cuda())
    assert tuple(out.shape) == (2, M // 2, N)
    ref = oracle.nvfp4_linear(bf16_bits(x.reshape(M, K)), gx, wc, wsf, gw)
    assert rel_err(to_np(out).reshape(M, N), ref) < TOL


@pytest.mark.parametrize("M,H,E,topk,dtype,renorm", [
    (32, 2048, 512, 10, torch.bfloat16, True),       # the decode configuration's router: 2048 -> 512, top-10
    (1, 2048, 512, 10, torch.bfloat16, True),
    (13, 256, 72, 4, torch.float16, False),          # ragged token block, E not a multiple of 64, plain softmax weights
    (128, 2048, 512, 10, torch.bfloat16, True),
])
def test_router_matches_fp32_torch(M, H, E, topk, dtype, renorm):
    from dgx_vllm_b200.router import moe_router
    g = torch.Generator().manual_seed(M + E)
    hidden = torch.randn(M, H, generator=g).to(dtype)
    gate = (torch.randn(E, H, generator=g) / H ** 0.5).to(dtype)
    tw, ids = moe_router(hidden.cuda(), gate.cuda(), topk, renormalize=renorm)
    logits = hidden.double() @ gate.double().t()
    probs = torch.softmax(logits, dim=-1)
    ref_w, ref_ids = probs.topk(topk, dim=-1)
    if renorm:
        ref_w = ref_w / ref_w.sum(-1, keepdim=True)
    # ids must agree wherever the decision is not a near-tie of the fp32 accumulation (gap to the next logit > 1e-4)
    srt = logits.sort(dim=-1, descending=True).values
    clear = (srt[:, :topk] - srt[:, 1:topk + 1]).min(dim=-1).values > 1e-4
    assert clear.float().mean() > 0.8
    assert torch.equal(ids.cpu()[clear].long(), ref_ids[clear])
    assert (tw.cpu()[clear].double() - ref_w[clear]).abs().max() < 1e-3
    assert torch.allclose(tw.sum(-1).cpu(), torch.ones(M), atol=1e-5) or not renorm
    # and it feeds the fused layer without a host round trip: dtypes and layouts are the ones the ops take
    assert tw.dtype == torch.float32 and ids.dtype == torch.int32 and tw.is_contiguous() and ids.is_contiguous()
