#!/usr/bin/env python3
"""Generate the golden vectors under tests/golden/ by RUNNING THE REFERENCE'S OWN PYTHON.

Run once in a container that has the reference tree and vLLM installed:

    python tests/golden/make_golden.py --reference /path/to/dgx-vllm

What is executed:
  * the replacement ``run_nvfp4_emulations`` text that fix_nvfp4_emulation_backend.py:60-102
    injects into vLLM, exec'd on top of vLLM's pure-torch leaf functions ``ref_nvfp4_quant``,
    ``cast_to_fp4`` and ``break_fp4_bytes`` (CPU tensors only, so no Triton path is taken);
  * ``unpack_fp4_nibbles`` / ``apply_2of4_sparsity_fast`` / ``convert_expert_to_v7_gpu`` imported
    from sparse_fp4_kernel/sparse_v7_moe_patch.py (on CPU tensors).

The tests never need the reference or vLLM: they read the .npz files written here.
"""
import argparse
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def values_to_codes(v: torch.Tensor) -> np.ndarray:
    """float E2M1 values [M,K] -> packed codes [M,K/2]; sign bit from signbit (so -0.0 -> 0x8)."""
    lut = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    mag = (v.abs().unsqueeze(-1) == lut).to(torch.uint8).argmax(-1).to(torch.uint8)
    assert torch.equal(lut[mag.long()], v.abs())
    code = mag | (torch.signbit(v).to(torch.uint8) << 3)
    return (code[:, 0::2] | (code[:, 1::2] << 4)).numpy().copy()


def load_reference_emulation(ref_root: str):
    from vllm.model_executor.layers.quantization.utils import nvfp4_emulation_utils as U
    ns = {}
    src = open(os.path.join(ref_root, "fix_nvfp4_emulation_backend.py")).read()
    # the patch file defines `new_func = '''def run_nvfp4_emulations(...) ...'''`
    start = src.index("new_func = '''") + len("new_func = '''")
    end = src.index("'''", start)
    env = {"torch": torch, "ref_nvfp4_quant": U.ref_nvfp4_quant, "break_fp4_bytes": U.break_fp4_bytes}
    exec(src[start:end], env, ns)
    return U, ns["run_nvfp4_emulations"]


def load_reference_sparse(ref_root: str):
    p = os.path.join(ref_root, "sparse_fp4_kernel", "sparse_v7_moe_patch.py")
    spec = importlib.util.spec_from_file_location("ref_sparse_v7_moe_patch", p)
    mod = importlib.util.module_from_spec(spec)
    os.environ.pop("VLLM_NVFP4_SPARSE_V7", None)
    spec.loader.exec_module(mod)
    return mod


def quantize_weight(U, w: torch.Tensor):
    gs = (448.0 * 6.0 / w.abs().max().float()).reshape(1).to(torch.float32)
    vals, sf = U.ref_nvfp4_quant(w, gs, 16)
    return values_to_codes(vals), sf.to(torch.float8_e4m3fn).view(torch.uint8).numpy().copy(), gs


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of Avarok-Cybersecurity/dgx-vllm")
    args = ap.parse_args()
    U, run_emul = load_reference_emulation(args.reference)
    S = load_reference_sparse(args.reference)

    # ---- (1) the reference's CPU-runnable dense case: x 8x2048 bf16 N(0,1), W 512x2048 N(0,0.02), seed 0
    g = torch.Generator().manual_seed(0)
    x = torch.randn(8, 2048, generator=g).to(torch.bfloat16)
    w = (0.02 * torch.randn(512, 2048, generator=g)).to(torch.float32)
    gs_x = (448.0 * 6.0 / x.abs().max().float()).reshape(1).to(torch.float32)
    w_codes, w_sf, gs_w = quantize_weight(U, w)
    x_vals, x_sf = U.ref_nvfp4_quant(x, gs_x, 16)
    out = run_emul(x, gs_x, torch.from_numpy(w_codes), torch.from_numpy(w_sf).view(torch.float8_e4m3fn), gs_w)
    np.savez_compressed(
        os.path.join(HERE, "dense_c1.npz"),
        x_bits=bf16_bits(x), gs_x=gs_x.numpy(), w_f32_first_rows=w[:4].numpy(),
        w_codes=w_codes, w_sf=w_sf, gs_w=gs_w.numpy(),
        x_codes=values_to_codes(x_vals), x_values=x_vals.numpy(),
        x_sf=x_sf.to(torch.float8_e4m3fn).view(torch.uint8).numpy(),
        out_bits=bf16_bits(out))

    # ---- (2) quantizer known-answer cases: ties, zero blocks, subnormal scales, saturation
    rows = []
    ties = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]
    base = torch.zeros(16)
    for amax in [6.0, 3.0, 448.0, 1.0, 0.001, 1e-6]:
        r = base.clone()
        r[0] = amax
        for i, t in enumerate(ties):
            r[1 + i] = t * amax / 6.0
            r[8 + i] = -t * amax / 6.0
        r[15] = -amax
        rows.append(r)
    rows.append(torch.zeros(16))                                   # all-zero block
    r = torch.zeros(16); r[5] = 0.37; rows.append(r)               # single non-zero
    r = torch.zeros(16); r[3] = -0.0; r[4] = -1e-30; rows.append(r)
    g2 = torch.Generator().manual_seed(1)
    rows += list(torch.randn(32, 16, generator=g2) * torch.logspace(-6, 2, 32).unsqueeze(1))
    kat = torch.stack(rows).reshape(-1, 16)
    # lay the blocks out as a [R, 64] matrix (4 blocks per row) so K/16 > 1
    pad = (-kat.shape[0]) % 4
    kat = torch.cat([kat, torch.zeros(pad, 16)]).reshape(-1, 64).to(torch.bfloat16)
    kat_out = {}
    for name, gsv in [("amax", float(448.0 * 6.0 / kat.abs().max().float())), ("one", 1.0), ("big", 2688.0), ("tiny", 1e-3)]:
        gs = torch.tensor([gsv], dtype=torch.float32)
        v, s = U.ref_nvfp4_quant(kat, gs, 16)
        kat_out[f"gs_{name}"] = gs.numpy()
        kat_out[f"values_{name}"] = v.numpy()
        kat_out[f"codes_{name}"] = values_to_codes(v)
        kat_out[f"sf_{name}"] = s.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
        kat_out[f"sf_f32_{name}"] = s.numpy()
    np.savez_compressed(os.path.join(HERE, "quant_kat.npz"), x_bits=bf16_bits(kat), **kat_out)

    # ---- (3) E2M1 thresholds (cast_to_fp4) and the scale-factor swizzle (convert_swizzled_to_linear)
    probe = torch.tensor([0.0, 0.1, 0.25, 0.2500001, 0.5, 0.75, 0.7499999, 1.0, 1.25, 1.2500001, 1.5, 1.75,
                          1.7499999, 2.0, 2.5, 2.5000002, 3.0, 3.5, 3.4999998, 4.0, 5.0, 5.0000005, 6.0])
    probe = torch.cat([probe, -probe])
    cast = U.cast_to_fp4(probe.clone())
    M, KB = 200, 12
    swz = torch.arange(((M + 127) // 128) * 128 * ((KB + 3) // 4) * 4, dtype=torch.int32)
    lin = U.convert_swizzled_to_linear(swz, M, KB * 16, 16)
    np.savez_compressed(os.path.join(HERE, "codec.npz"), probe=probe.numpy(), cast=cast.numpy(),
                        swz_M=M, swz_KB=KB, swz_linear_index=lin.numpy().astype(np.int32),
                        break_in=np.arange(256, dtype=np.uint8).reshape(16, 16),
                        break_out=U.break_fp4_bytes(torch.arange(256, dtype=torch.uint8).reshape(16, 16), torch.float32).numpy())

    # ---- (4) 2:4 converter: reference convert_expert_to_v7_gpu on CPU tensors
    g3 = torch.Generator().manual_seed(2)
    wq = (0.02 * torch.randn(96, 256, generator=g3)).to(torch.float32)
    c, sfw, _ = quantize_weight(U, wq)
    comp_T, meta_T, scale_T = S.convert_expert_to_v7_gpu(
        torch.from_numpy(c), torch.from_numpy(sfw).view(torch.float8_e4m3fn), 0)
    nib = S.unpack_fp4_nibbles(torch.from_numpy(c))
    np.savez_compressed(os.path.join(HERE, "sparse_convert.npz"), codes=c, sf=sfw,
                        nibbles=nib.numpy(), comp_T=comp_T.numpy(), meta_T=meta_T.numpy(),
                        scale_T=scale_T.numpy())
    print("golden vectors written to", HERE)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f"  {f}: {os.path.getsize(os.path.join(HERE, f))} bytes")


if __name__ == "__main__":
    sys.exit(main())
