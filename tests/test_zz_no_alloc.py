"""The allocation-free sparse GEMV entry point (b200fp4_sparse_gemv_static) against the regular one.

Collected last on purpose (file name): a run that stops at the first failure has then already run
every other test.  Both entry points are called straight through the C ABI with ctypes; the static
one gets no workspace at all -- its scratch is the fixed array inside the library -- and is called
twice in a row with different inputs to show that what the first call left in the shared scratch
does not leak into the second."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _case(seed, P, E=8, N=256, K=512, dtype=torch.bfloat16):
    rng = np.random.default_rng(seed)
    G = K // 16
    t = lambda a: torch.from_numpy(a).cuda()
    comp = t(rng.integers(0, 256, (E, K // 4, N), dtype=np.uint8))
    meta = t(rng.integers(0, 256, (E, K // 8, N), dtype=np.uint8))
    scale = t(rng.integers(56, 120, (E, G, N), dtype=np.uint8))
    g = t((rng.random(E) * 1e-3 + 1e-4).astype(np.float32))
    ids = t(rng.integers(-1, E, P).astype(np.int32))          # includes some -1 (not local) entries
    A = torch.randn(P, K, generator=torch.Generator().manual_seed(seed)).to(dtype).cuda()
    return A, comp, meta, scale, g, ids, (P, N, K, G, E)


def _call(L, static, A, comp, meta, scale, g, ids, dims, ws=None):
    from dgx_vllm_b200 import _lib
    P, N, K, G, E = dims
    out = torch.full((P, N), float("nan"), dtype=A.dtype, device="cuda")
    code = _lib.BF16 if A.dtype == torch.bfloat16 else _lib.F16
    stream = torch.cuda.current_stream().cuda_stream
    common = (A.data_ptr(), code, comp.data_ptr(), meta.data_ptr(), scale.data_ptr(), g.data_ptr(), ids.data_ptr(),
              out.data_ptr(), code, P, N, K, G, E)
    if static:
        rc = L.b200fp4_sparse_gemv_static(*common, stream)
    else:
        rc = L.b200fp4_sparse_gemv(*common, 0, ws.data_ptr(), ws.numel(), stream)
    torch.cuda.synchronize()
    return rc, out


def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row():
    from dgx_vllm_b200 import _lib
    L = _lib.lib()
    ws = torch.empty(L.b200fp4_sparse_workspace_bytes(512, 4096, 4096), dtype=torch.uint8, device="cuda")
    for seed, P, dtype in ((1, 37, torch.bfloat16), (2, 11, torch.float16)):      # two calls in a row, shared scratch
        case = _case(seed, P, dtype=dtype)
        rc_ref, ref = _call(L, False, *case, ws=ws)
        rc_new, got = _call(L, True, *case)
        assert rc_ref == 0 and rc_new == 0
        ref, got = ref.float().cpu().numpy(), got.float().cpu().numpy()
        assert np.isfinite(got).all()
        assert np.max(np.abs(got - ref)) <= TOL * np.max(np.abs(ref))
        ids = case[5].cpu().numpy()
        assert np.all(got[ids < 0] == 0)
        # and against the CPU oracle of the reference's batched_sparse_v7 (same tolerance as the other GEMV parity tests)
        import oracle
        A, comp, meta, scale, g = (t.cpu() for t in case[:5])
        want = oracle.batched_sparse_gemv(A.float().numpy(), comp.numpy(), meta.numpy(), scale.numpy(), g.numpy(), ids)
        assert np.max(np.abs(got - want)) <= TOL * np.max(np.abs(want))


def test_static_scratch_entry_rejects_sizes_beyond_its_fixed_scratch():
    from dgx_vllm_b200 import _lib
    L = _lib.lib()
    A, comp, meta, scale, g, ids, dims = _case(3, 513)          # one pair more than the scratch holds
    rc, out = _call(L, True, A, comp, meta, scale, g, ids, dims)
    assert rc == 15 and b"not supported" in L.b200fp4_get_error_string(rc)
    assert torch.isnan(out.float()).all()                       # nothing was enqueued
