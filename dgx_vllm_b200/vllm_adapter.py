"""vLLM adapter: what makes the ops of this package serve a real model.

Sparse MoE experts -- the counterpart of the reference's sparse_kernel patch
(sparse_fp4_kernel/sparse_v7_moe_patch.py:200-358):
  * `make_v7_apply_fn`          the closure assigned as `experts.apply` (its `_make_v7_apply_fn`, :200-232)
  * `process_moe_layer`         clone the checkpoint weights, let vLLM's own process_weights_after_loading run,
                                convert the clones to the 2:4 tensors ON THE GPU (one kernel instead of the
                                reference's Python loop over experts, :96-129), swap `apply`, and replace the
                                original tensors by zero-stride stubs that keep their shapes (:300-326)
  * `patch_vllm`                installs it on ModelOptNvFp4FusedMoE, gated by VLLM_NVFP4_SPARSE_V7=1 like the
                                reference (:334-362), and routes vLLM's dense NVFP4 entry points here
Dense NVFP4 linears:
  * `Nvfp4LinearCore` / `linear_kernel_class()`   an NvFp4LinearKernel (vllm/model_executor/kernels/linear/nvfp4/
                                base.py) whose quantizer and GEMM are this library's.

Nothing here imports vLLM at module import time; `patch_vllm` and `linear_kernel_class` do when called."""
from __future__ import annotations

import logging
import os
import time
from typing import Callable, Optional

import torch

logger = logging.getLogger(__name__)

_STUBBED_PARAMS = ("w13_weight", "w2_weight", "w13_weight_scale", "w2_weight_scale", "w13_weight_scale_2",
                   "w2_weight_scale_2")


def make_v7_apply_fn(w13_comp, w13_meta, w13_scale, w13_g_scales, w2_comp, w2_meta, w2_scale, w2_g_scales, inter_size,
                     hidden_size, fused_fn: Optional[Callable] = None):
    """The function vLLM calls in place of MarlinExperts.apply (same 15 positional arguments, no self): writes
    output[:M] and returns output, like v7_apply (sparse_v7_moe_patch.py:216-230).  The weight tensors are validated
    and bound once per expert_map; `fused_fn`, when given, replaces the bound CUDA layer (tests on CPU)."""
    bound = {}

    def layer_for(expert_map):
        key = None if expert_map is None else (expert_map.data_ptr(), expert_map.numel())
        if key not in bound:
            from .sparse_fp4_v7 import FusedSparseMoE
            bound[key] = FusedSparseMoE(w13_comp, w13_meta, w13_scale, w13_g_scales, w2_comp, w2_meta, w2_scale,
                                        w2_g_scales, inter_size, expert_map=expert_map)
        return bound[key]

    def v7_apply(output, hidden_states, w1, w2, topk_weights, topk_ids, activation, global_num_experts, expert_map,
                 a1q_scale, a2_scale, workspace13, workspace2, expert_tokens_meta, apply_router_weight_on_input):
        if fused_fn is not None:
            result = fused_fn(hidden_states, topk_weights.float(), topk_ids, expert_map, w13_comp, w13_meta, w13_scale,
                              w13_g_scales, w2_comp, w2_meta, w2_scale, w2_g_scales, inter_size,
                              apply_router_weight_on_input)
        else:
            if expert_map is not None and not expert_map.is_cuda:
                expert_map = expert_map.to(hidden_states.device)
            result = layer_for(expert_map)(hidden_states, topk_weights, topk_ids,
                                           apply_router_weight_on_input=apply_router_weight_on_input)
        output[:hidden_states.shape[0]] = result.to(output.dtype)
        return output

    return v7_apply


def _zero_stride_stub(param) -> int:
    """param.data := a one-element tensor viewed with the original shape (all strides 0); returns the bytes freed.
    vLLM still reads the shapes of these parameters (moe_problem_size), never their contents."""
    data = param.data
    shape = tuple(data.shape)
    freed = data.numel() * data.element_size()
    stub = torch.zeros(1, device=data.device, dtype=data.dtype)
    param.data = stub.as_strided(shape, [0] * len(shape))
    return freed


def process_moe_layer(method, layer, original: Callable, convert_fn: Optional[Callable] = None, device=None,
                      make_apply: Callable = make_v7_apply_fn) -> bool:
    """What the patched ModelOptNvFp4FusedMoE.process_weights_after_loading does for one layer
    (sparse_v7_moe_patch.py:243-331).  `original(method, layer)` is vLLM's own routine; `convert_fn(weights [E,N,K/2],
    scales [E,N,K/16], g_scales [E], device=) -> (comp_T, meta_T, scale_T, g)` defaults to the CUDA converter.
    Returns True when `apply` was replaced."""
    t0 = time.time()
    # 1. the checkpoint tensors, before the repacking of the original routine destroys them
    src = {name: getattr(layer, name).data.clone() for name in _STUBBED_PARAMS}
    E, inter2, hidden_half = src["w13_weight"].shape
    inter_size, hidden_size = inter2 // 2, hidden_half * 2
    # 2. vLLM's own processing (builds the modular kernel whose experts object gets the new apply)
    original(method, layer)
    experts = getattr(getattr(method, "moe_mk", None), "fused_experts", None)
    if experts is None:
        logger.warning("[b200 sparse] moe_mk.fused_experts not found: layer left on vLLM's own kernels")
        return False
    # 3. 2:4 conversion on the device
    if convert_fn is None:
        from .sparse_fp4_v7 import convert_weight_batch_to_v7 as convert_fn
    if device is None:
        device = src["w13_weight"].device if src["w13_weight"].is_cuda else "cuda"
    gs = lambda t: t[:, 0] if t.dim() > 1 else t
    w13 = convert_fn(src["w13_weight"], src["w13_weight_scale"], gs(src["w13_weight_scale_2"]), device=device)
    w2 = convert_fn(src["w2_weight"], src["w2_weight_scale"], gs(src["w2_weight_scale_2"]), device=device)
    del src
    # 4. the closure shadows the class method on this experts instance; the originals shrink to shape-only stubs
    experts.apply = make_apply(*w13, *w2, inter_size, hidden_size)
    freed = sum(_zero_stride_stub(getattr(layer, name)) for name in _STUBBED_PARAMS if hasattr(layer, name))
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    logger.info("[b200 sparse] %d experts converted in %.1f s, %.1f MB of repacked weights released", E,
                time.time() - t0, freed / 1e6)
    return True


_original_process_weights = None


def patch_vllm(force: bool = False) -> bool:
    """Install the hook on vLLM's ModelOptNvFp4FusedMoE and route its dense NVFP4 ops to this library.  Like the
    reference's module it acts only when VLLM_NVFP4_SPARSE_V7=1 (or force=True).  Idempotent."""
    global _original_process_weights
    if not force and os.environ.get("VLLM_NVFP4_SPARSE_V7", "0") != "1":
        return False
    if _original_process_weights is not None:
        return True
    from vllm.model_executor.layers.quantization.modelopt import ModelOptNvFp4FusedMoE

    from .torch_ops import install_into_vllm
    _original_process_weights = ModelOptNvFp4FusedMoE.process_weights_after_loading

    def patched(self, layer):
        process_moe_layer(self, layer, _original_process_weights)

    ModelOptNvFp4FusedMoE.process_weights_after_loading = patched
    install_into_vllm()
    logger.info("[b200 sparse] vLLM patched: sparse 2:4 MoE experts and dense NVFP4 ops run on libb200nvfp4")
    return True


class Nvfp4LinearCore:
    """process_weights_after_loading / apply_weights of a dense NVFP4 linear on this library's quantizer and GEMM
    (the two methods an NvFp4LinearKernel must provide).  The layer carries vLLM's attribute names: weight
    [N,K/2] u8, weight_scale [N,K/16] e4m3 (linear in the checkpoint), input_global_scale_inv (= 448*6/amax),
    alpha (= 1 / (input scale * weight scale)), output_size_per_partition."""

    def __init__(self, swizzle_fn: Optional[Callable] = None, quant_fn: Optional[Callable] = None,
                 mm_fn: Optional[Callable] = None):
        self._swizzle, self._quant, self._mm = swizzle_fn, quant_fn, mm_fn

    def process_weights_after_loading(self, layer) -> None:
        swz = self._swizzle or swizzle_blockscale
        layer.weight_scale = torch.nn.Parameter(swz(layer.weight_scale.data), requires_grad=False)
        layer.weight = torch.nn.Parameter(layer.weight.data.contiguous(), requires_grad=False)

    def apply_weights(self, layer, x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        from . import ops
        out_shape = [*x.shape[:-1], layer.output_size_per_partition]
        x2 = x.reshape(-1, x.shape[-1])
        if self._quant is None and self._mm is None:
            # quantizer and GEMM queued by one library call
            out = ops.nvfp4_linear(x2, layer.input_global_scale_inv, layer.weight, layer.weight_scale, layer.alpha)
        else:
            quant, mm = self._quant or ops.scaled_fp4_quant, self._mm or ops.cutlass_scaled_fp4_mm
            codes, sf = quant(x2, layer.input_global_scale_inv, True)
            out = mm(codes, layer.weight, sf, layer.weight_scale, layer.alpha, x.dtype)
        if bias is not None:
            out = out + bias
        return out.view(*out_shape)


def swizzle_blockscale(sf_linear: torch.Tensor) -> torch.Tensor:
    """[rows, K/16] e4m3 block scales -> the padded 128x4 tile layout the GEMM reads (swizzle_blockscale,
    vllm/model_executor/layers/quantization/utils/nvfp4_utils.py:38-51), on the GPU."""
    from . import _lib
    from ._torch_util import ptr, require, require_cuda, stream_ptr
    dev = require_cuda(sf_linear)
    require(sf_linear.dim() == 2 and sf_linear.element_size() == 1 and sf_linear.is_contiguous(),
            "block scales must be a contiguous [rows, K/16] one-byte tensor")
    rows, kb = sf_linear.shape
    out = torch.empty(((rows + 127) // 128 * 128, (kb + 3) // 4 * 4), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().b200fp4_sf_swizzle(ptr(sf_linear), rows, kb, ptr(out), stream_ptr(dev)), "swizzle_blockscale")
    return out.view(torch.float8_e4m3fn)


def linear_kernel_class():
    """An NvFp4LinearKernel subclass for vLLM's kernel registry (imports vLLM)."""
    from vllm.model_executor.kernels.linear.nvfp4.base import NvFp4LinearKernel

    class B200NvFp4LinearKernel(NvFp4LinearKernel):
        _core = Nvfp4LinearCore()

        @classmethod
        def is_supported(cls, compute_capability=None):
            from . import _lib
            ok = _lib.lib().b200fp4_has_hardware_acceleration() == 1
            return (True, None) if ok else (False, "needs an sm_100 device")

        @classmethod
        def can_implement(cls, config):
            return True, None

        def process_weights_after_loading(self, layer):
            self._core.process_weights_after_loading(layer)

        def apply_weights(self, layer, x, bias=None):
            return self._core.apply_weights(layer, x, bias)

    return B200NvFp4LinearKernel


if os.environ.get("VLLM_NVFP4_SPARSE_V7", "0") == "1" and os.environ.get("B200_NVFP4_AUTOPATCH", "0") == "1":
    patch_vllm()
