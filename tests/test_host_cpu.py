"""CPU-side checks: the C ABI library loads and exports every declared symbol; host-side logic
(synthetic generators, record packing, expert-parallel dispatch/combine over gloo)."""
import os
import re
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

import oracle
from util import oracle_quantize_fn, rel_err

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from dgx_vllm_b200 import _lib
    hdr = open(os.path.join(ROOT, "include", "b200_nvfp4.h")).read()
    declared = set(re.findall(r"\b(b200fp4_[a-z0-9_]+|cudaFP4[A-Za-z0-9]+)\s*\(", hdr))
    assert declared, "no declarations found"
    L = _lib.lib()
    for name in declared:
        assert hasattr(L, name), f"{name} declared in the header but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert L.b200fp4_version() >= 100
    assert b"success" in L.b200fp4_get_error_string(0)
    assert L.b200fp4_sf_swizzled_bytes(200, 12) == oracle.sf_swizzled_bytes(200, 12)
    assert L.b200fp4_sparse_workspace_bytes(320, 2048, 512) > 0


def test_no_cpu_fallback():
    from dgx_vllm_b200 import scaled_fp4_quant, sparse_fp4_v7
    with pytest.raises(RuntimeError):
        scaled_fp4_quant(torch.zeros(4, 16, dtype=torch.bfloat16), torch.ones(1))
    with pytest.raises(RuntimeError):
        sparse_fp4_v7.batched_sparse_v7(torch.zeros(1, 16).half(), torch.zeros(1, 4, 16, dtype=torch.uint8),
                                        torch.zeros(1, 2, 16, dtype=torch.uint8), torch.zeros(1, 1, 16, dtype=torch.uint8),
                                        torch.ones(1), torch.zeros(1, dtype=torch.int32))


def test_product_does_not_import_oracle():
    pkg = os.path.join(ROOT, "dgx_vllm_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(import|from)\s+oracle\b", src, re.M), f


def test_synth_sparse_experts_are_2of4_and_consistent():
    import synth
    w = synth.make_sparse_experts(2, 32, 64, 0, "cpu", oracle_quantize_fn)
    assert tuple(w["comp_T"].shape) == (2, 16, 32) and tuple(w["meta_T"].shape) == (2, 8, 32)
    meta = w["meta_T"].numpy()
    i0, i1, i2, i3 = meta & 3, (meta >> 2) & 3, (meta >> 4) & 3, (meta >> 6) & 3
    assert np.all(i0 < i1) and np.all(i2 < i3)                    # two distinct, sorted positions per group
    W = oracle.sparse_expand(w["comp_T"][0].numpy(), meta[0], w["scale_T"][0].numpy(), float(w["g_scales"][0]))
    assert np.all((W.reshape(32, 16, 4) != 0).sum(-1) <= 2)
    assert abs(np.abs(W).max() - 0.02 * 4) < 0.06                 # ~N(0, 0.02) magnitudes survive quantization


def test_routing_generators():
    import synth
    w, ids = synth.make_routing(16, 64, 10, 0, "cpu")
    assert ids.dtype == torch.int32 and w.dtype == torch.float32
    assert torch.allclose(w.sum(-1), torch.ones(16), atol=1e-5)
    assert all(len(set(r.tolist())) == 10 for r in ids)
    w, ids = synth.make_routing(256, 64, 10, 0, "cpu", zipf=1.1)
    counts = torch.bincount(ids.flatten().long(), minlength=64).float()
    assert counts.max() > 3 * counts.median()                     # skewed popularity
    assert all(len(set(r.tolist())) == 10 for r in ids)


def test_record_packing_roundtrip():
    from dgx_vllm_b200 import moe_ep
    h = torch.randn(5, 32).bfloat16()
    w = torch.rand(5, 3)
    ids = torch.randint(0, 8, (5, 3), dtype=torch.int32)
    rec = moe_ep.pack_records(h, w, ids)
    h2, w2, i2 = moe_ep.unpack_records(rec, 32, 3, torch.bfloat16)
    assert torch.equal(h, h2) and torch.equal(w, w2) and torch.equal(ids, i2)
    m = moe_ep.expert_map_for_rank(8, 2, 1, "cpu")
    assert m.tolist() == [-1, -1, -1, -1, 0, 1, 2, 3]


_WORKER = r'''
import os, sys
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
import numpy as np, torch, torch.distributed as dist
import oracle
from util import oracle_quantize_fn
import synth
from dgx_vllm_b200.moe_ep import ExpertParallelMoE
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
E, H, I, B, topk = 8, 64, 32, 3, 2
keys = ("comp_T", "meta_T", "scale_T", "g_scales")
full13 = synth.make_sparse_experts(E, 2 * I, H, 1, "cpu", oracle_quantize_fn)
full2 = synth.make_sparse_experts(E, H, I, 2, "cpu", oracle_quantize_fn)
per = E // world
loc13 = {k: full13[k][rank * per:(rank + 1) * per] for k in keys}
loc2 = {k: full2[k][rank * per:(rank + 1) * per] for k in keys}
def local_fn(hidden, tw, ids, emap):       # CPU stand-in for the CUDA op: the oracle
    out = oracle.fused_sparse_moe(hidden.float().numpy(), tw.numpy(), ids.numpy(), emap.numpy(),
                                  tuple(loc13[k].numpy() for k in keys), tuple(loc2[k].numpy() for k in keys), I,
                                  round_fp16=False)
    return torch.from_numpy(out).to(hidden.dtype)
tw, ids = synth.make_routing(B, E, topk, 10 + rank, "cpu")
hidden = synth.make_hidden(B, H, 20 + rank, "cpu")
ref = oracle.fused_sparse_moe(hidden.float().numpy(), tw.numpy(), ids.numpy(), None,
                              tuple(full13[k].numpy() for k in keys), tuple(full2[k].numpy() for k in keys), I,
                              round_fp16=False)
for mode in ("gather", "a2a"):      # all-gather + reduce-scatter of fp32 partial rows; all-to-all both ways
    layer = ExpertParallelMoE(E, I, None, None, local_moe_fn=local_fn, mode=mode)
    out = layer.forward(hidden, tw, ids)
    err = float(np.max(np.abs(out.float().numpy() - ref)) / np.max(np.abs(ref)))
    assert err < 2e-2, (mode, err)          # the stand-in returns 16-bit partial rows per owner rank
    # the host-buffer entry points on CPU ranks: nothing to queue, the result is there on return
    out_host = torch.empty_like(hidden)
    assert layer.submit_host(hidden, tw, ids, out_host, torch.device("cpu")) is None
    layer.wait_host(torch.device("cpu"))
    assert torch.equal(out_host, out)
    assert torch.equal(layer.forward_host(hidden, tw, ids, torch.empty_like(hidden), torch.device("cpu")), out)
print(f"rank {rank} ok err={err:.3e}")
dist.destroy_process_group()
'''


def test_expert_parallel_dispatch_combine_gloo_world2(tmp_path):
    script = tmp_path / "ep_worker.py"
    script.write_text(_WORKER)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(script), ROOT],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout


_SHARD_WORKER = r'''
import os, sys
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
import numpy as np, torch, torch.distributed as dist
import oracle
from dgx_vllm_b200.dense_shard import ColumnShardedNvfp4Linear, shard_rows
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
M, N, K = 5, 256, 128
g = torch.Generator().manual_seed(3)
x = torch.randn(M, K, generator=g).to(torch.bfloat16)
w = (0.02 * torch.randn(N, K, generator=g)).to(torch.bfloat16)
gx = np.float32(448.0 * 6.0 / float(x.float().abs().max())); gw = np.float32(448.0 * 6.0 / float(w.float().abs().max()))
xb = x.view(torch.int16).numpy().view(np.uint16); wb = w.view(torch.int16).numpy().view(np.uint16)
xc, xs = oracle.quantize_bf16(xb, gx); wc, wsf = oracle.quantize_bf16(wb, gw)
ref = oracle.nvfp4_linear(xb, gx, wc, wsf, gw)                      # full [M, N]
b, e = shard_rows(N, world, rank)
def local_fn(x_, layer):                                            # CPU stand-in for quantize + GEMM: the oracle on the shard
    return torch.from_numpy(oracle.nvfp4_linear(xb, gx, wc[layer.begin:layer.end], wsf[layer.begin:layer.end], gw)).to(torch.bfloat16)
layer = ColumnShardedNvfp4Linear(N, torch.tensor([gw]), local_fn=local_fn)
assert (layer.begin, layer.end) == (rank * N // world, (rank + 1) * N // world)
part = layer.forward(x, torch.tensor([gx]))
full = layer.forward(x, torch.tensor([gx]), gather=True)
assert tuple(part.shape) == (M, N // world) and tuple(full.shape) == (M, N)
err = float(np.max(np.abs(full.float().numpy() - ref)) / np.max(np.abs(ref)))
assert err < 1e-2, err
assert torch.equal(full[:, b:e], part)
print(f"rank {rank} ok err={err:.3e}")
dist.destroy_process_group()
'''


def test_column_sharded_linear_gloo_world2(tmp_path):
    from dgx_vllm_b200.dense_shard import shard_rows
    assert shard_rows(14336, 8, 3) == (5376, 7168)
    with pytest.raises(RuntimeError):
        shard_rows(14336, 3, 0)
    script = tmp_path / "shard_worker.py"
    script.write_text(_SHARD_WORKER)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(script), ROOT],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout


_PREFILL_WORKER = r'''
import os, sys
sys.path.insert(0, sys.argv[1])
import torch, torch.distributed as dist
from dgx_vllm_b200.moe_ep import ExpertParallelMoEPrefill
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
E, H, Tl, k = 8, 16, 5, 3
def expert_fn(e, h):                                   # a stand-in expert: scale by (e + 1)
    return (e + 1.0) * h
def local_fn(hidden, tw, ids, emap):                   # contributions of the experts this rank owns
    out = torch.zeros(hidden.shape, dtype=torch.float32)
    for t in range(hidden.shape[0]):
        for j in range(ids.shape[1]):
            if int(emap[int(ids[t, j])]) >= 0:
                out[t] += tw[t, j] * expert_fn(float(ids[t, j]), hidden[t].float())
    return out
g = torch.Generator().manual_seed(100 + rank)
hidden = torch.randn(Tl, H, generator=g)
ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(Tl)]).to(torch.int32)
tw = torch.rand(Tl, k, generator=g)
layer = ExpertParallelMoEPrefill(E, None, local_fn=local_fn)
out = layer.forward(hidden, tw, ids)
ref = torch.zeros(Tl, H)
for t in range(Tl):
    for j in range(k):
        ref[t] += tw[t, j] * expert_fn(float(ids[t, j]), hidden[t])
assert tuple(out.shape) == (Tl, H)
assert torch.allclose(out, ref, rtol=1e-5, atol=1e-5), float((out - ref).abs().max())
print(f"rank {rank} ok")
dist.destroy_process_group()
'''


def test_expert_parallel_prefill_gloo_world2(tmp_path):
    script = tmp_path / "prefill_worker.py"
    script.write_text(_PREFILL_WORKER)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(script), ROOT],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout


def test_torch_custom_ops_registered_with_fake_impls():
    import dgx_vllm_b200.torch_ops  # noqa: F401
    ns = torch.ops.b200_nvfp4
    for name in ("scaled_fp4_quant", "cutlass_scaled_fp4_mm", "cutlass_fp4_group_mm", "batched_sparse_v7", "fused_sparse_moe_v7"):
        assert hasattr(ns, name)
    x = torch.empty(200, 4096, dtype=torch.bfloat16, device="meta")
    codes, sf = ns.scaled_fp4_quant(x, torch.empty(1, device="meta"), True)
    assert tuple(codes.shape) == (200, 2048) and tuple(sf.shape) == (256, 256) and sf.dtype == torch.float8_e4m3fn
    with pytest.raises((RuntimeError, NotImplementedError)):
        ns.scaled_fp4_quant(torch.zeros(4, 16, dtype=torch.bfloat16), torch.ones(1), True)     # no CPU kernel
