"""GPU parity of the 2:4-sparse MoE GEMV ops (through the C ABI) against the oracle.
Tolerance: max|diff| / max|ref| <= 1e-2 against the fp32 dequantize-then-matmul result."""
import numpy as np
import pytest
import torch

import oracle
from util import oracle_quantize_fn, rel_err, to_np

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _rand_sparse(E, N, K, G, seed):
    rng = np.random.default_rng(seed)
    comp = rng.integers(0, 256, (E, K // 4, N), dtype=np.uint8)
    meta = rng.integers(0, 256, (E, K // 8, N), dtype=np.uint8)
    scale = rng.integers(56, 120, (E, G, N), dtype=np.uint8)      # as bench_v7_scaled.py:153
    g = (rng.random(E) * 1e-3 + 1e-4).astype(np.float32)
    return comp, meta, scale, g


def _cuda(*arrs):
    return [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in arrs]


@pytest.mark.parametrize("E,N,K,G,P", [
    (4, 512, 64, 8, 2),          # the reference's own validation shape (bench_v7_scaled.py:133)
    (4, 512, 64, 4, 3),
    (6, 1024, 2048, 128, 9),     # gate_up projection of the MoE configuration
    (6, 2048, 512, 32, 9),       # down projection
    (3, 144, 96, 6, 5),          # N not a multiple of the 128-column slab
    (3, 40, 48, 6, 4),           # N % 16 != 0 -> scalar kernel
    (2, 64, 64, 2, 3),           # one scale per 32 k -> scalar kernel
])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_batched_sparse_v7(E, N, K, G, P, dtype):
    from dgx_vllm_b200 import sparse_fp4_v7 as sp7
    comp, meta, scale, g = _rand_sparse(E, N, K, G, seed=E * N + K)
    rng = np.random.default_rng(1)
    ids = rng.integers(0, E, P).astype(np.int32)
    A = torch.randn(P, K, generator=torch.Generator().manual_seed(2)).to(dtype)
    out = sp7.batched_sparse_v7(A.cuda(), *_cuda(comp, meta, scale, g, ids))
    assert out.dtype == dtype and tuple(out.shape) == (P, N)
    ref = oracle.batched_sparse_gemv(A.float().numpy(), comp, meta, scale, g, ids)
    assert rel_err(to_np(out), ref) < TOL
    out2 = sp7.batched_sparse_v7(A.cuda(), *_cuda(comp, meta, scale, g, ids))
    assert torch.equal(out, out2)                                  # deterministic


def test_many_tokens_per_expert_and_unmapped_ids():
    from dgx_vllm_b200 import sparse_fp4_v7 as sp7
    E, N, K, G, P = 3, 256, 256, 16, 23
    comp, meta, scale, g = _rand_sparse(E, N, K, G, seed=7)
    ids = np.array([0] * 11 + [2] * 6 + [-1, 5, 1, 1, 1, -7], np.int32)   # >4 per expert, invalid ids
    A = torch.randn(P, K, generator=torch.Generator().manual_seed(3)).to(torch.float16)
    out = to_np(sp7.batched_sparse_v7(A.cuda(), *_cuda(comp, meta, scale, g, ids)))
    safe = np.where((ids >= 0) & (ids < E), ids, -1)
    ref = oracle.batched_sparse_gemv(A.float().numpy(), comp, meta, scale, g, safe)
    assert rel_err(out, ref) < TOL
    assert np.all(out[safe < 0] == 0)


def test_dense_and_packed_variants():
    from dgx_vllm_b200 import sparse_fp4_v7 as sp7
    E, N, K, P = 3, 128, 128, 4
    rng = np.random.default_rng(11)
    dense = rng.integers(0, 256, (E, K // 2, N), dtype=np.uint8)
    scale = rng.integers(56, 120, (E, K // 16, N), dtype=np.uint8)
    g = (rng.random(E) * 1e-3 + 1e-4).astype(np.float32)
    ids = np.array([2, 0, 1, 2], np.int32)
    A = torch.randn(P, K, generator=torch.Generator().manual_seed(4)).to(torch.float16)
    out = sp7.batched_dense_v7(A.cuda(), *_cuda(dense, scale, g, ids))
    assert rel_err(to_np(out), oracle.batched_dense_gemv(A.float().numpy(), dense, scale, g, ids)) < TOL
    comp, meta, scale8, g = _rand_sparse(E, N, K, K // 8, seed=12)
    packed = np.concatenate([comp[:, 0::2], comp[:, 1::2], meta, scale8], axis=2)      # [E, K/8, 4N]
    out = sp7.batched_sparse_packed_v7(A.cuda(), *_cuda(packed, g, ids), K)
    assert rel_err(to_np(out), oracle.batched_sparse_gemv(A.float().numpy(), comp, meta, scale8, g, ids)) < TOL


def _moe_case(E, H, I, B, topk, seed, dtype=torch.bfloat16):
    import synth
    w13 = synth.make_sparse_experts(E, 2 * I, H, seed, "cpu", oracle_quantize_fn)
    w2 = synth.make_sparse_experts(E, H, I, seed + 1, "cpu", oracle_quantize_fn)
    tw, ids = synth.make_routing(B, E, topk, seed + 2, "cpu")
    hidden = synth.make_hidden(B, H, seed + 3, "cpu", dtype)
    return w13, w2, tw, ids, hidden


def _run_fused(w13, w2, tw, ids, hidden, I, emap=None, on_input=False):
    from dgx_vllm_b200 import sparse_fp4_v7 as sp7
    c = lambda d: [d[k].cuda() for k in ("comp_T", "meta_T", "scale_T", "g_scales")]
    emap_t = torch.empty(0, dtype=torch.int32, device="cuda") if emap is None else torch.from_numpy(emap).cuda()
    return sp7.fused_sparse_moe_v7(hidden.cuda(), tw.cuda(), ids.cuda(), emap_t, *c(w13), *c(w2), I, on_input)


def _ref_fused(w13, w2, tw, ids, hidden, I, emap=None, on_input=False):
    n = lambda d: tuple(d[k].numpy() for k in ("comp_T", "meta_T", "scale_T", "g_scales"))
    return oracle.fused_sparse_moe(hidden.float().numpy(), tw.numpy(), ids.numpy(), emap, n(w13), n(w2), I,
                                   apply_router_weight_on_input=on_input, round_fp16=False)


@pytest.mark.parametrize("B", [1, 8, 32])
def test_fused_moe_layer(B):
    # the MoE decode configuration at reduced expert count (shapes per expert are the real ones)
    E, H, I, topk = 16, 2048, 512, 10
    case = _moe_case(E, H, I, B, topk, seed=B)
    out = _run_fused(*case, I)
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == (B, H)
    ref = _ref_fused(*case, I)
    assert rel_err(to_np(out), ref) < TOL
    assert torch.equal(out, _run_fused(*case, I))


def test_fused_moe_expert_map_and_flags():
    E_local, E_global, H, I, B, topk = 4, 8, 256, 128, 5, 3
    w13, w2, _, _, hidden = _moe_case(E_local, H, I, B, topk, seed=9, dtype=torch.float16)
    import synth
    tw, ids = synth.make_routing(B, E_global, topk, 10, "cpu")
    emap = np.array([-1, 0, -1, 1, 2, -1, 3, -1], np.int32)       # half of the global experts are local
    out = _run_fused(w13, w2, tw, ids, hidden, I, emap)
    ref = _ref_fused(w13, w2, tw, ids, hidden, I, emap)
    assert out.dtype == torch.float16
    assert rel_err(to_np(out), ref) < TOL
    out = _run_fused(w13, w2, tw, ids, hidden, I, emap, on_input=True)
    ref = _ref_fused(w13, w2, tw, ids, hidden, I, emap, on_input=True)
    assert rel_err(to_np(out), ref) < TOL


def test_argument_validation():
    from dgx_vllm_b200 import sparse_fp4_v7 as sp7
    comp, meta, scale, g = _rand_sparse(2, 64, 64, 4, seed=1)
    A = torch.randn(2, 64).half()
    ids = np.array([0, 1], np.int32)
    with pytest.raises(RuntimeError):
        sp7.batched_sparse_v7(A, *_cuda(comp, meta, scale, g, ids))               # A on the CPU
    with pytest.raises(RuntimeError):
        sp7.batched_sparse_v7(A.cuda().float(), *_cuda(comp, meta, scale, g, ids))   # wrong dtype
    with pytest.raises(RuntimeError):
        sp7.batched_sparse_v7(A.cuda(), *_cuda(comp, meta[:, :4], scale, g, ids))    # wrong meta shape


def test_ep_records_pack_fused_combine_single_gpu():
    # the expert-parallel kernels without the collectives: two "ranks" emulated on one GPU by
    # swapping the record blocks by hand (what the all-to-all does), against the full-layer oracle
    from dgx_vllm_b200 import _lib
    import synth
    from dgx_vllm_b200._torch_util import workspace
    L = _lib.lib()
    G, E_glob, H, I, B, topk = 2, 8, 256, 128, 5, 3
    E = E_glob // G
    w13 = synth.make_sparse_experts(E_glob, 2 * I, H, 31, "cpu", oracle_quantize_fn)
    w2 = synth.make_sparse_experts(E_glob, H, I, 32, "cpu", oracle_quantize_fn)
    keys = ("comp_T", "meta_T", "scale_T", "g_scales")
    R = L.b200fp4_ep_record_bytes(H, topk)
    assert R % 16 == 0 and R >= H * 2 + topk * 8
    hid, tws, idss, sends = [], [], [], []
    for r in range(G):
        tw, ids = synth.make_routing(B, E_glob, topk, 40 + r, "cpu")
        h = synth.make_hidden(B, H, 50 + r, "cpu")
        send = torch.empty(G * B * R, dtype=torch.uint8, device="cuda")
        hc, ic, wc = h.cuda(), ids.cuda(), tw.cuda()
        _lib.check(L.b200fp4_ep_pack(hc.data_ptr(), ic.data_ptr(), wc.data_ptr(), B, H, topk, G, send.data_ptr(), 0), "pack")
        hid.append(h), tws.append(tw), idss.append(ids), sends.append(send.view(G, B * R))
    torch.cuda.synchronize()
    parts = []
    for r in range(G):                                        # rank r receives block r of every sender
        recv = torch.cat([sends[src][r] for src in range(G)]).contiguous()
        emap = torch.full((E_glob,), -1, dtype=torch.int32)
        emap[r * E:(r + 1) * E] = torch.arange(E, dtype=torch.int32)
        loc13 = [w13[k][r * E:(r + 1) * E].contiguous().cuda() for k in keys]
        loc2 = [w2[k][r * E:(r + 1) * E].contiguous().cuda() for k in keys]
        part = torch.empty(G * B, H, dtype=torch.bfloat16, device="cuda")
        ws = workspace(torch.device("cuda", 0), L.b200fp4_fused_moe_workspace_bytes(G * B, topk, H, I, E))
        emc = emap.cuda()
        _lib.check(L.b200fp4_fused_sparse_moe_records(recv.data_ptr(), R, _lib.BF16, emc.data_ptr(), E_glob,
                                                      *[t.data_ptr() for t in loc13], loc13[2].shape[1],
                                                      *[t.data_ptr() for t in loc2], loc2[2].shape[1],
                                                      part.data_ptr(), _lib.BF16, G * B, topk, H, I, E, _lib.SPARSE_META_ORDERED,
                                                      ws.data_ptr(), ws.numel(), 0), "records")
        torch.cuda.synchronize()
        parts.append(part.view(G, B, H))
    for src in range(G):                                      # combine: rank src gets its block back from every rank
        back = torch.stack([parts[r][src] for r in range(G)]).contiguous()
        out = torch.empty(B, H, dtype=torch.bfloat16, device="cuda")
        _lib.check(L.b200fp4_ep_combine(back.data_ptr(), _lib.BF16, B, H, G, out.data_ptr(), 0), "combine")
        torch.cuda.synchronize()
        n = lambda d: tuple(d[k].numpy() for k in keys)
        ref = oracle.fused_sparse_moe(hid[src].float().numpy(), tws[src].numpy(), idss[src].numpy(), None, n(w13), n(w2), I,
                                      round_fp16=False)
        assert rel_err(to_np(out), ref) < 2e-2                # partial rows travel as bf16


def test_convert_weight_batch_to_v7_matches_oracle_and_reference_golden(golden_dir):
    import os
    from dgx_vllm_b200 import sparse_fp4_v7 as sp7
    rng = np.random.default_rng(5)
    E, N, K = 3, 80, 96
    codes = rng.integers(0, 256, (E, N, K // 2), dtype=np.uint8)
    sf = rng.integers(0, 127, (E, N, K // 16), dtype=np.uint8)
    comp, meta, scale, g = sp7.convert_weight_batch_to_v7(torch.from_numpy(codes), torch.from_numpy(sf), torch.ones(E))
    for e in range(E):
        oc, om = oracle.sparse_2of4_pack(codes[e])                 # bit-exact, ties included (same rule)
        np.testing.assert_array_equal(to_np(comp[e]), oc)
        np.testing.assert_array_equal(to_np(meta[e]), om)
        np.testing.assert_array_equal(to_np(scale[e]), sf[e].T)
    # the reference's own converter output (golden): identical wherever the top-2 choice is unambiguous
    gd = np.load(os.path.join(golden_dir, "sparse_convert.npz"))
    comp, meta, scale, _ = sp7.convert_weight_batch_to_v7(torch.from_numpy(gd["codes"][None]), torch.from_numpy(gd["sf"][None]),
                                                         torch.ones(1))
    nib = gd["nibbles"]
    Nn, Kk = nib.shape
    mag = np.abs(oracle.E2M1_LUT[nib]).reshape(Nn, Kk // 4, 4)
    srt = np.sort(mag, axis=2)
    tie_free = (srt[:, :, 1] != srt[:, :, 2]).T
    np.testing.assert_array_equal(to_np(comp[0])[tie_free], gd["comp_T"][tie_free])
    np.testing.assert_array_equal(to_np(scale[0]), gd["scale_T"])


# ---------------------------------------------------------------------------------------------
# tensor-core path (metadata indices in increasing order, as the reference's converter writes them)

_ORDERED_NIBBLES = np.array([4, 8, 12, 9, 13, 14], dtype=np.uint8)       # i0 | i1 << 2 with i0 < i1


def _rand_sparse_ordered(E, N, K, seed, signed_scales=False):
    rng = np.random.default_rng(seed)
    comp = rng.integers(0, 256, (E, K // 4, N), dtype=np.uint8)
    meta = _ORDERED_NIBBLES[rng.integers(0, 6, (E, K // 8, N))] | (_ORDERED_NIBBLES[rng.integers(0, 6, (E, K // 8, N))] << 4)
    scale = rng.integers(1, 120, (E, K // 16, N), dtype=np.uint8)          # includes E4M3 subnormals
    if signed_scales:
        scale |= (rng.integers(0, 2, scale.shape, dtype=np.uint8) << 7)
    g = (rng.random(E) * 1e-3 + 1e-4).astype(np.float32)
    return comp, meta.astype(np.uint8), scale, g


def test_metadata_ordered_check():
    from dgx_vllm_b200 import sparse_fp4_v7 as sp7
    comp, meta, scale, g = _rand_sparse_ordered(2, 128, 64, 3)
    m = torch.from_numpy(meta).cuda()
    assert sp7.metadata_ordered(m)
    bad = m.clone()
    bad[1, 3, 77] = 0x4E                                                     # low group (2, 3) ok, high group (0, 1) ok
    assert sp7.metadata_ordered(bad)
    bad[1, 3, 77] = 0x41                                                     # low group i0 = 1, i1 = 0
    assert not sp7.metadata_ordered(bad)
    bad[1, 3, 77] = 0x54                                                     # high group i0 = i1 = 1
    assert not sp7.metadata_ordered(bad)


@pytest.mark.parametrize("E,N,K,P,dtype", [
    (4, 512, 128, 9, torch.float16),          # plain slab of 4 column groups, two steps per K-slice
    (3, 1024, 2048, 17, torch.bfloat16),      # several slabs, experts with more than four tokens (two passes)
    (5, 256, 512, 6, torch.bfloat16),         # N only allows two column groups
    (2, 128, 1024, 5, torch.float16),         # N only allows one column group
    (70, 512, 256, 300, torch.bfloat16),      # more items than SMs: every block walks several items
])
def test_batched_sparse_v7_tensor_core_path(E, N, K, P, dtype):
    from dgx_vllm_b200 import sparse_fp4_v7 as sp7
    comp, meta, scale, g = _rand_sparse_ordered(E, N, K, seed=E + N + K)
    rng = np.random.default_rng(5)
    ids = rng.integers(0, E, P).astype(np.int32)
    A = torch.randn(P, K, generator=torch.Generator().manual_seed(6)).to(dtype)
    dev = _cuda(comp, meta, scale, g, ids)
    out = sp7.batched_sparse_v7(A.cuda(), *dev, meta_ordered=True)
    ref = oracle.batched_sparse_gemv(A.float().numpy(), comp, meta, scale, g, ids)
    assert rel_err(to_np(out), ref) < TOL
    general = sp7.batched_sparse_v7(A.cuda(), *dev, meta_ordered=False)
    assert rel_err(to_np(general), ref) < TOL
    assert torch.equal(out, sp7.batched_sparse_v7(A.cuda(), *dev))         # auto-detected, deterministic


def test_tensor_core_path_signed_scales_and_foreign_ids():
    from dgx_vllm_b200 import sparse_fp4_v7 as sp7
    E, N, K, P = 6, 512, 256, 40
    comp, meta, scale, g = _rand_sparse_ordered(E, N, K, seed=11, signed_scales=True)
    ids = np.random.default_rng(2).integers(-1, E + 1, P).astype(np.int32)   # -1 and E are not local
    A = torch.randn(P, K, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    out = to_np(sp7.batched_sparse_v7(A.cuda(), *_cuda(comp, meta, scale, g, ids), meta_ordered=True))
    safe = np.where((ids >= 0) & (ids < E), ids, 0)
    ref = oracle.batched_sparse_gemv(A.float().numpy(), comp, meta, scale, g, safe)
    ref[(ids < 0) | (ids >= E)] = 0
    assert rel_err(out, ref) < TOL
    assert np.all(out[(ids < 0) | (ids >= E)] == 0)


@pytest.mark.parametrize("ordered", [True, False])
@pytest.mark.parametrize("M,topk,E,H,I", [(5, 4, 16, 512, 256), (33, 8, 24, 1024, 128), (1, 2, 8, 2048, 512)])
def test_fused_moe_both_kernels(M, topk, E, H, I, ordered):
    from dgx_vllm_b200 import sparse_fp4_v7 as sp7
    w13, w2, tw, ids, hidden = _moe_case(E, H, I, M, topk, seed=M + E)
    c = lambda d: [d[k].cuda() for k in ("comp_T", "meta_T", "scale_T", "g_scales")]
    out = sp7.fused_sparse_moe_v7(hidden.cuda(), tw.cuda(), ids.cuda(), None, *c(w13), *c(w2), I, False, meta_ordered=ordered)
    ref = _ref_fused(w13, w2, tw, ids, hidden, I)
    assert rel_err(to_np(out), ref) < TOL


def test_bound_layer_object_matches_function():
    from dgx_vllm_b200 import sparse_fp4_v7 as sp7
    E, H, I, B, topk = 16, 1024, 256, 9, 4
    w13, w2, tw, ids, hidden = _moe_case(E, H, I, B, topk, seed=77)
    c = lambda d: [d[k].cuda() for k in ("comp_T", "meta_T", "scale_T", "g_scales")]
    a13, a2 = c(w13), c(w2)
    emap = torch.arange(E, dtype=torch.int32)
    emap[::3] = -1
    emap = emap.cuda()
    layer = sp7.FusedSparseMoE(*a13, *a2, I, expert_map=emap)
    for on_input in (False, True):
        ref = sp7.fused_sparse_moe_v7(hidden.cuda(), tw.cuda(), ids.cuda(), emap, *a13, *a2, I, on_input)
        out = layer(hidden.cuda(), tw.cuda(), ids.cuda(), apply_router_weight_on_input=on_input)
        assert torch.equal(out, ref)
    with pytest.raises(RuntimeError):
        layer(hidden.cuda()[:, :512].contiguous(), tw.cuda(), ids.cuda())


def test_bound_layer_host_buffers_match_device_call():
    """forward_host (host pointers through the C entry point: copies in, layer, copy out, sync) gives the bytes of
    the device call, from pinned and from pageable memory, and checks its arguments."""
    from dgx_vllm_b200 import sparse_fp4_v7 as sp7
    E, H, I, B, topk = 16, 1024, 256, 9, 4
    w13, w2, tw, ids, hidden = _moe_case(E, H, I, B, topk, seed=78)
    c = lambda d: [d[k].cuda() for k in ("comp_T", "meta_T", "scale_T", "g_scales")]
    layer = sp7.FusedSparseMoE(*c(w13), *c(w2), I)
    ref = layer(hidden.cuda(), tw.cuda(), ids.cuda())
    out_pageable = layer.forward_host(hidden, tw, ids, out_host=torch.empty_like(hidden))
    assert torch.equal(out_pageable, ref.cpu())
    out_pinned = layer.forward_host(hidden.pin_memory(), tw.pin_memory(), ids.pin_memory())
    assert out_pinned.is_pinned() and torch.equal(out_pinned, ref.cpu())
    ref_in = layer(hidden.cuda(), tw.cuda(), ids.cuda(), apply_router_weight_on_input=True)
    assert torch.equal(layer.forward_host(hidden, tw, ids, apply_router_weight_on_input=True), ref_in.cpu())
    with pytest.raises(RuntimeError):
        layer.forward_host(hidden.cuda(), tw, ids)
    with pytest.raises(RuntimeError):
        layer.forward_host(hidden, tw, ids.long())


@pytest.mark.parametrize("overlap,direct", [(True, True), (True, False), (False, True), (False, False)])
def test_bound_layer_queued_host_steps_match_device_call(overlap, direct):
    """submit_host keeps several steps in flight (copy stream + two staging slots, or everything on one stream);
    every step's host result equals the device call on that step's inputs, also when a slot is reused at once."""
    from dgx_vllm_b200 import sparse_fp4_v7 as sp7
    E, H, I, B, topk = 16, 1024, 256, 9, 4
    w13, w2, _, _, _ = _moe_case(E, H, I, B, topk, seed=81)
    c = lambda d: [d[k].cuda() for k in ("comp_T", "meta_T", "scale_T", "g_scales")]
    layer = sp7.FusedSparseMoE(*c(w13), *c(w2), I)
    steps = []
    for i in range(6):
        _, _, tw, ids, hidden = _moe_case(E, H, I, B, topk, seed=200 + i)
        steps.append((hidden.pin_memory(), tw.pin_memory(), ids.pin_memory(), torch.empty_like(hidden).pin_memory()))
    refs = [layer(h.cuda(), w.cuda(), i.cuda()).cpu() for h, w, i, _ in steps]
    slots = (0, 1, 0, 0, 1, 1)          # alternating and back-to-back reuse of a staging slot
    events = [layer.submit_host(h, w, i, o, slot=slots[n], overlap_copies=overlap, direct_out=direct) for n, (h, w, i, o) in enumerate(steps)]
    events[2].synchronize()
    assert torch.equal(steps[2][3], refs[2])
    layer.wait_host()
    for (_, _, _, o), ref in zip(steps, refs):
        assert torch.equal(o, ref)
    with pytest.raises(RuntimeError):
        layer.submit_host(steps[0][0].clone(), steps[0][1], steps[0][2], steps[0][3])     # pageable input


@pytest.mark.parametrize("M,topk,E,H,I,separate", [
    (64, 8, 16, 2048, 512, False),      # 32 tokens per expert on average: eight-token passes, one launch
    (64, 8, 16, 2048, 512, True),       # ... and one launch per projection
    (48, 6, 8, 1024, 256, False),       # shapes that take other slab widths
])
def test_fused_moe_eight_token_passes(M, topk, E, H, I, separate):
    from dgx_vllm_b200 import sparse_fp4_v7 as sp7
    w13, w2, tw, ids, hidden = _moe_case(E, H, I, M, topk, seed=M + E + I)
    c = lambda d: [d[k].cuda() for k in ("comp_T", "meta_T", "scale_T", "g_scales")]
    out = sp7.fused_sparse_moe_v7(hidden.cuda(), tw.cuda(), ids.cuda(), None, *c(w13), *c(w2), I, False,
                                  separate_launches=separate)
    ref = _ref_fused(w13, w2, tw, ids, hidden, I)
    assert rel_err(to_np(out), ref) < TOL
    general = sp7.fused_sparse_moe_v7(hidden.cuda(), tw.cuda(), ids.cuda(), None, *c(w13), *c(w2), I, False, meta_ordered=False)
    assert rel_err(to_np(general), ref) < TOL
