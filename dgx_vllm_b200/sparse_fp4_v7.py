"""Drop-in mirror of the reference's `sparse_fp4_v7` extension module.

Same function names, positional order and tensor formats as the pybind module defined at
sparse_fp4_kernel/sparse_fp4_v7.cu:744-749 of Avarok-Cybersecurity/dgx-vllm, backed by the
sm_100a kernels in libb200nvfp4.so.  Differences a caller can observe:
  * arguments are validated (device, dtype, shape, contiguity) and a RuntimeError is raised on
    misuse, where the reference has undefined behaviour;
  * bf16 activations are taken natively and the result comes back in the activation dtype
    (the reference casts bf16 to fp16 first and always returns fp16); pass out_dtype to force one;
  * expert ids outside [0, E) -- e.g. -1 from an expert-parallel expert_map -- give a zero
    contribution instead of an out-of-bounds read;
  * when every 4-group's two metadata indices are in increasing order -- which is how the
    reference's converter writes them (sparse_v7_moe_patch.py:59-60) -- the GEMVs run on the tensor
    cores.  The mirrors check each metadata tensor object once (`metadata_ordered`) unless the
    caller passes `meta_ordered=`; tensors with other index pairs take the general kernel, which
    accepts anything the reference kernel accepts.  (A block scale's sign bit, never set by an
    NVFP4 quantizer, is honoured by the tensor-core kernel and ignored by the general one.)
"""
from __future__ import annotations

import torch

from . import _lib
from ._torch_util import dtype_code, ptr, require, require_cuda, stream_ptr, workspace

STATUS_INTERNAL_ERROR = 14       # B200FP4_STATUS_INTERNAL_ERROR: a bounded device wait expired


def _check_act(A: torch.Tensor, name: str) -> None:
    require(A.dim() == 2, f"{name} must be 2-D")
    require(A.dtype in (torch.float16, torch.bfloat16), f"{name} must be float16 or bfloat16")
    require(A.is_contiguous(), f"{name} must be contiguous")


def _check_u8(t: torch.Tensor, name: str, ndim: int = 3) -> None:
    require(t.dim() == ndim, f"{name} must be {ndim}-D")
    require(t.dtype in (torch.uint8, torch.float8_e4m3fn), f"{name} must be uint8")
    require(t.is_contiguous(), f"{name} must be contiguous")


def _ids_i32(ids: torch.Tensor) -> torch.Tensor:
    ids = ids.reshape(-1)
    if ids.dtype != torch.int32:
        ids = ids.to(torch.int32)
    return ids.contiguous()


def _out_dtype(A: torch.Tensor, out_dtype) -> torch.dtype:
    return A.dtype if out_dtype is None else out_dtype


def metadata_ordered(meta: torch.Tensor) -> bool:
    """True if in every byte of `meta` (two 4-groups: i0 | i1<<2 | i0'<<4 | i1'<<6) i0 < i1 and i0' < i1'.

    The answer is remembered on the tensor object (with its version counter, so an in-place update
    is checked again).  The first call per tensor reads the whole tensor and synchronises; while a
    CUDA graph is being captured an unseen tensor is reported as not ordered instead (the general
    kernel is always valid)."""
    seen = getattr(meta, "_b200fp4_meta_ordered", None)
    if seen is not None and seen[0] == meta._version:
        return seen[1]
    if meta.is_cuda and torch.cuda.is_current_stream_capturing():
        return False
    flat = meta.reshape(-1).view(torch.uint8)
    ok = True
    step = 1 << 26
    for off in range(0, flat.numel(), step):
        m = flat[off:off + step]
        lo, hi = m & 0x33, (m >> 2) & 0x33          # (i0, i0') and (i1, i1') in bits 0-1 and 4-5
        if not bool(((hi & 3) > (lo & 3)).all() and ((hi >> 4) > (lo >> 4)).all()):
            ok = False
            break
    try:
        meta._b200fp4_meta_ordered = (meta._version, ok)
    except AttributeError:
        pass
    return ok


def _flags(meta_ordered, *metas) -> int:
    if meta_ordered is None:
        meta_ordered = all(metadata_ordered(m) for m in metas)
    return _lib.SPARSE_META_ORDERED if meta_ordered else 0


def batched_sparse_v7(A, B_comp_T, Meta_T_pk, scales_T, g_scales, expert_ids, *, out_dtype=None, meta_ordered=None):
    """out[p] = A[p] . W[expert_ids[p]]^T with W given in 2:4 compressed NVFP4 form
    (batched_sparse_v7, sparse_fp4_v7.cu:374-406).

    A [P,K] f16/bf16; B_comp_T [E,K/4,N] u8; Meta_T_pk [E,K/8,N] u8; scales_T [E,G,N] e4m3 bytes
    (G = K/16 or K/8 vectorised, any divisor of K/8 otherwise); g_scales [E] f32; expert_ids [P].
    meta_ordered: promise (True) / deny (False) ordered metadata indices, or None to check once."""
    dev = require_cuda(A, B_comp_T, Meta_T_pk, scales_T, g_scales, expert_ids)
    _check_act(A, "A")
    _check_u8(B_comp_T, "B_comp_T"), _check_u8(Meta_T_pk, "Meta_T_pk"), _check_u8(scales_T, "scales_T")
    P, K = A.shape
    E, K4, N = B_comp_T.shape
    G = scales_T.shape[1]
    require(K4 * 4 == K and K % 8 == 0, "B_comp_T must be [E, K/4, N]")
    require(tuple(Meta_T_pk.shape) == (E, K // 8, N), "Meta_T_pk must be [E, K/8, N]")
    require(scales_T.shape[0] == E and scales_T.shape[2] == N and (K // 8) % G == 0, "scales_T must be [E, G, N]")
    require(g_scales.dtype == torch.float32 and g_scales.numel() >= E and g_scales.is_contiguous(), "g_scales must be f32 [E]")
    ids = _ids_i32(expert_ids)
    require(ids.numel() == P, "expert_ids must have one entry per row of A")
    out = torch.empty((P, N), dtype=_out_dtype(A, out_dtype), device=dev)
    L = _lib.lib()
    nws = L.b200fp4_sparse_workspace_bytes(P, K, E)
    ws = workspace(dev, nws)
    with torch.cuda.device(dev):
        _lib.check(L.b200fp4_sparse_gemv(ptr(A), dtype_code(A.dtype), ptr(B_comp_T), ptr(Meta_T_pk), ptr(scales_T),
                                         ptr(g_scales), ptr(ids), ptr(out), dtype_code(out.dtype), P, N, K, G, E,
                                         _flags(meta_ordered, Meta_T_pk), ptr(ws), ws.numel(), stream_ptr(dev)),
                   "batched_sparse_v7")
    return out


def batched_dense_v7(A, B_dense_T, scales_T, g_scales, expert_ids, *, out_dtype=None):
    """Dense-code variant (batched_dense_v7, sparse_fp4_v7.cu:341-372): B_dense_T [E,K/2,N] u8."""
    dev = require_cuda(A, B_dense_T, scales_T, g_scales, expert_ids)
    _check_act(A, "A")
    _check_u8(B_dense_T, "B_dense_T"), _check_u8(scales_T, "scales_T")
    P, K = A.shape
    E, K2, N = B_dense_T.shape
    G = scales_T.shape[1]
    require(K2 * 2 == K, "B_dense_T must be [E, K/2, N]")
    require(scales_T.shape[0] == E and scales_T.shape[2] == N and K % G == 0 and (K // G) % 2 == 0, "scales_T must be [E, G, N]")
    require(g_scales.dtype == torch.float32 and g_scales.numel() >= E and g_scales.is_contiguous(), "g_scales must be f32 [E]")
    ids = _ids_i32(expert_ids)
    require(ids.numel() == P, "expert_ids must have one entry per row of A")
    out = torch.empty((P, N), dtype=_out_dtype(A, out_dtype), device=dev)
    L = _lib.lib()
    with torch.cuda.device(dev):
        _lib.check(L.b200fp4_dense_gemv(ptr(A), dtype_code(A.dtype), ptr(B_dense_T), ptr(scales_T), ptr(g_scales),
                                        ptr(ids), ptr(out), dtype_code(out.dtype), P, N, K, G, E, 0, 0,
                                        stream_ptr(dev)), "batched_dense_v7")
    return out


def batched_sparse_packed_v7(A, B_packed_T, g_scales, expert_ids, orig_K, *, out_dtype=None):
    """Interleaved-tensor variant (batched_sparse_packed_v7, sparse_fp4_v7.cu:408-436):
    B_packed_T [E, K/8, 4N] = comp0 | comp1 | meta | scale per row, one scale per 8 k."""
    dev = require_cuda(A, B_packed_T, g_scales, expert_ids)
    _check_act(A, "A")
    _check_u8(B_packed_T, "B_packed_T")
    P, K = A.shape
    require(int(orig_K) == K, "orig_K must equal A.shape[1]")
    E, K8, N4 = B_packed_T.shape
    require(K8 * 8 == K and N4 % 4 == 0, "B_packed_T must be [E, K/8, 4N]")
    N = N4 // 4
    require(g_scales.dtype == torch.float32 and g_scales.numel() >= E and g_scales.is_contiguous(), "g_scales must be f32 [E]")
    ids = _ids_i32(expert_ids)
    require(ids.numel() == P, "expert_ids must have one entry per row of A")
    out = torch.empty((P, N), dtype=_out_dtype(A, out_dtype), device=dev)
    L = _lib.lib()
    ws = workspace(dev, L.b200fp4_sparse_workspace_bytes(P, K, E))
    with torch.cuda.device(dev):
        _lib.check(L.b200fp4_sparse_packed_gemv(ptr(A), dtype_code(A.dtype), ptr(B_packed_T), ptr(g_scales), ptr(ids),
                                                ptr(out), dtype_code(out.dtype), P, N, K, E, ptr(ws), ws.numel(),
                                                stream_ptr(dev)), "batched_sparse_packed_v7")
    return out


def fused_sparse_moe_v7(hidden_states, topk_weights, topk_ids, expert_map,
                        w13_comp, w13_meta, w13_scale, w13_g_scales,
                        w2_comp, w2_meta, w2_scale, w2_g_scales,
                        inter_size, apply_router_weight_on_input, *, out_dtype=None, meta_ordered=None,
                        separate_launches=False):
    """One MoE layer for decode (fused_sparse_moe_v7, sparse_fp4_v7.cu:607-742):
    gate_up GEMV -> SiLU(gate)*up -> down GEMV -> router-weighted sum.

    hidden_states [M,H] f16/bf16; topk_weights [M,topk] f32; topk_ids [M,topk] int; expert_map [global_E]
    int32 or an empty tensor / None for identity; w13_* [E,H/4,2I], [E,H/8,2I], [E,G,2I], [E];
    w2_* [E,I/4,H], [E,I/8,H], [E,G,H], [E].  Returns [M,H].  meta_ordered as in batched_sparse_v7;
    separate_launches=True keeps one launch per projection (by default small batches, up to 256
    (token, expert) pairs, run both in one cooperative launch where the shapes allow it)."""
    dev = require_cuda(hidden_states, topk_weights, topk_ids, w13_comp, w13_meta, w13_scale, w13_g_scales,
                       w2_comp, w2_meta, w2_scale, w2_g_scales)
    _check_act(hidden_states, "hidden_states")
    for t, n in ((w13_comp, "w13_comp"), (w13_meta, "w13_meta"), (w13_scale, "w13_scale"), (w2_comp, "w2_comp"),
                 (w2_meta, "w2_meta"), (w2_scale, "w2_scale")):
        _check_u8(t, n)
    M, H = hidden_states.shape
    require(topk_ids.dim() == 2 and topk_ids.shape[0] == M, "topk_ids must be [M, topk]")
    topk = topk_ids.shape[1]
    I = int(inter_size)
    E = w13_comp.shape[0]
    require(tuple(w13_comp.shape) == (E, H // 4, 2 * I), "w13_comp must be [E, H/4, 2I]")
    require(tuple(w13_meta.shape) == (E, H // 8, 2 * I), "w13_meta must be [E, H/8, 2I]")
    require(w13_scale.shape[0] == E and w13_scale.shape[2] == 2 * I, "w13_scale must be [E, G, 2I]")
    require(tuple(w2_comp.shape) == (E, I // 4, H), "w2_comp must be [E, I/4, H]")
    require(tuple(w2_meta.shape) == (E, I // 8, H), "w2_meta must be [E, I/8, H]")
    require(w2_scale.shape[0] == E and w2_scale.shape[2] == H, "w2_scale must be [E, G, H]")
    for g in (w13_g_scales, w2_g_scales):
        require(g.dtype == torch.float32 and g.numel() >= E and g.is_contiguous(), "g_scales must be f32 [E]")
    tw = topk_weights
    if tw.dtype != torch.float32:
        tw = tw.float()
    tw = tw.contiguous()
    require(tuple(tw.shape) == (M, topk), "topk_weights must be [M, topk]")
    ids = _ids_i32(topk_ids)
    emap = None
    if expert_map is not None and expert_map.numel() > 0:
        require(expert_map.is_cuda, "expert_map must be a CUDA tensor")
        emap = expert_map if expert_map.dtype == torch.int32 else expert_map.to(torch.int32)
        emap = emap.contiguous()
    out = torch.empty((M, H), dtype=_out_dtype(hidden_states, out_dtype), device=dev)
    L = _lib.lib()
    ws = workspace(dev, L.b200fp4_fused_moe_workspace_bytes(M, topk, H, I, E))
    with torch.cuda.device(dev):
        _lib.check(L.b200fp4_fused_sparse_moe(
            ptr(hidden_states), dtype_code(hidden_states.dtype), ptr(tw), ptr(ids), ptr(emap),
            0 if emap is None else emap.numel(),
            ptr(w13_comp), ptr(w13_meta), ptr(w13_scale), ptr(w13_g_scales), w13_scale.shape[1],
            ptr(w2_comp), ptr(w2_meta), ptr(w2_scale), ptr(w2_g_scales), w2_scale.shape[1],
            ptr(out), dtype_code(out.dtype), M, topk, H, I, E,
            (_lib.MOE_ROUTER_WEIGHT_ON_INPUT if apply_router_weight_on_input else 0) | _flags(meta_ordered, w13_meta, w2_meta) |
            (_lib.MOE_SEPARATE_LAUNCHES if separate_launches else 0),
            ptr(ws), ws.numel(), stream_ptr(dev)), "fused_sparse_moe_v7")
    return out


def last_moe_status(device=None) -> int:
    """Status word of the most recent fused MoE layer issued through these mirrors on the current stream of
    `device`: 0, or -1 when a bounded wait of the one-launch layer ran out (the result of that call is then not
    valid).  Synchronises the stream (b200fp4_fused_moe_last_status)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    import ctypes
    ws = workspace(dev, 256)
    st = ctypes.c_int(0)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().b200fp4_fused_moe_last_status(ptr(ws), stream_ptr(dev), ctypes.addressof(st)), "last_moe_status")
    return int(st.value)


class FusedSparseMoE:
    """`fused_sparse_moe_v7` with the weight arguments bound once.

    A serving layer calls the op with the same eight weight tensors (and expert_map) every step;
    validating them, testing the metadata order and converting 20 pointers per call costs more host
    time than the kernels need for a small batch.  This object does that work once and keeps
    per-call work to the three activation-side tensors.  Results are identical to the function's."""

    def __init__(self, w13_comp, w13_meta, w13_scale, w13_g_scales, w2_comp, w2_meta, w2_scale, w2_g_scales,
                 inter_size: int, expert_map=None, meta_ordered=None, separate_launches: bool = False):
        dev = require_cuda(w13_comp, w13_meta, w13_scale, w13_g_scales, w2_comp, w2_meta, w2_scale, w2_g_scales)
        for t, n in ((w13_comp, "w13_comp"), (w13_meta, "w13_meta"), (w13_scale, "w13_scale"), (w2_comp, "w2_comp"),
                     (w2_meta, "w2_meta"), (w2_scale, "w2_scale")):
            _check_u8(t, n)
        E, H4, I2 = w13_comp.shape
        self.E, self.H, self.I = E, H4 * 4, int(inter_size)
        H, I = self.H, self.I
        require(I2 == 2 * I, "w13_comp must be [E, H/4, 2I]")
        require(tuple(w13_meta.shape) == (E, H // 8, 2 * I), "w13_meta must be [E, H/8, 2I]")
        require(w13_scale.shape[0] == E and w13_scale.shape[2] == 2 * I, "w13_scale must be [E, G, 2I]")
        require(tuple(w2_comp.shape) == (E, I // 4, H), "w2_comp must be [E, I/4, H]")
        require(tuple(w2_meta.shape) == (E, I // 8, H), "w2_meta must be [E, I/8, H]")
        require(w2_scale.shape[0] == E and w2_scale.shape[2] == H, "w2_scale must be [E, G, H]")
        for g in (w13_g_scales, w2_g_scales):
            require(g.dtype == torch.float32 and g.numel() >= E and g.is_contiguous(), "g_scales must be f32 [E]")
        emap = None
        if expert_map is not None and expert_map.numel() > 0:
            require(expert_map.is_cuda, "expert_map must be a CUDA tensor")
            emap = (expert_map if expert_map.dtype == torch.int32 else expert_map.to(torch.int32)).contiguous()
        self.device = dev
        self._keep = (w13_comp, w13_meta, w13_scale, w13_g_scales, w2_comp, w2_meta, w2_scale, w2_g_scales, emap)
        self._flags = _flags(meta_ordered, w13_meta, w2_meta) | (_lib.MOE_SEPARATE_LAUNCHES if separate_launches else 0)
        self._head = (ptr(emap), 0 if emap is None else emap.numel(),
                      ptr(w13_comp), ptr(w13_meta), ptr(w13_scale), ptr(w13_g_scales), w13_scale.shape[1],
                      ptr(w2_comp), ptr(w2_meta), ptr(w2_scale), ptr(w2_g_scales), w2_scale.shape[1])
        self._lib = _lib.lib()
        self._fn = self._lib.b200fp4_fused_sparse_moe
        self._ws_bytes = {}
        self._host_slots = {}
        self._copy_stream = None

    def __call__(self, hidden_states, topk_weights, topk_ids, apply_router_weight_on_input: bool = False, out=None):
        M, H = hidden_states.shape
        topk = topk_ids.shape[1]
        require(hidden_states.is_cuda and H == self.H and hidden_states.is_contiguous() and
                hidden_states.dtype in (torch.float16, torch.bfloat16), "hidden_states must be a contiguous [M,H] 16-bit CUDA tensor")
        tw = topk_weights if topk_weights.dtype == torch.float32 else topk_weights.float()
        ids = topk_ids if topk_ids.dtype == torch.int32 else topk_ids.to(torch.int32)
        require(tw.is_contiguous() and ids.is_contiguous() and tuple(tw.shape) == (M, topk) and ids.shape[0] == M,
                "topk_weights / topk_ids must be contiguous [M, topk]")
        dev = self.device
        if out is None:
            out = torch.empty((M, H), dtype=hidden_states.dtype, device=dev)
        key = (M, topk)
        nws = self._ws_bytes.get(key)
        if nws is None:
            nws = self._ws_bytes[key] = self._lib.b200fp4_fused_moe_workspace_bytes(M, topk, H, self.I, self.E)
        ws = workspace(dev, nws)
        code = dtype_code(hidden_states.dtype)
        flags = self._flags | (_lib.MOE_ROUTER_WEIGHT_ON_INPUT if apply_router_weight_on_input else 0)
        if torch.cuda.current_device() != dev.index:
            with torch.cuda.device(dev):
                rc = self._fn(hidden_states.data_ptr(), code, tw.data_ptr(), ids.data_ptr(), *self._head, out.data_ptr(),
                              dtype_code(out.dtype), M, topk, H, self.I, self.E, flags, ws.data_ptr(), ws.numel(), stream_ptr(dev))
        else:
            rc = self._fn(hidden_states.data_ptr(), code, tw.data_ptr(), ids.data_ptr(), *self._head, out.data_ptr(),
                          dtype_code(out.dtype), M, topk, H, self.I, self.E, flags, ws.data_ptr(), ws.numel(), stream_ptr(dev))
        _lib.check(rc, "fused_sparse_moe_v7")
        return out


    def forward_host(self, hidden_host, topk_weights_host, topk_ids_host, out_host=None,
                     apply_router_weight_on_input: bool = False):
        """The layer for CPU tensors: hidden [M,H] 16-bit, topk_weights [M,topk] f32, topk_ids [M,topk] i32 in host
        memory (pinned memory keeps the copies asynchronous); returns out_host [M,H], valid on return.  One library
        call does the three copies in, the layer, the copy out and the stream synchronisation."""
        M, H = hidden_host.shape
        topk = topk_ids_host.shape[1]
        require(not hidden_host.is_cuda and not topk_weights_host.is_cuda and not topk_ids_host.is_cuda,
                "forward_host takes CPU tensors")
        require(H == self.H and hidden_host.is_contiguous() and hidden_host.dtype in (torch.float16, torch.bfloat16),
                "hidden_host must be a contiguous [M,H] 16-bit tensor")
        require(topk_weights_host.dtype == torch.float32 and topk_ids_host.dtype == torch.int32 and
                topk_weights_host.is_contiguous() and topk_ids_host.is_contiguous() and
                tuple(topk_weights_host.shape) == (M, topk), "topk_weights f32 / topk_ids i32 must be contiguous [M, topk]")
        if out_host is None:
            out_host = torch.empty((M, H), dtype=hidden_host.dtype, pin_memory=True)
        require(not out_host.is_cuda and out_host.is_contiguous() and tuple(out_host.shape) == (M, H) and
                out_host.dtype in (torch.float16, torch.bfloat16), "out_host must be a contiguous [M,H] 16-bit CPU tensor")
        dev = self.device
        key = ("host", M, topk)
        nws = self._ws_bytes.get(key)
        if nws is None:
            nws = self._ws_bytes[key] = self._lib.b200fp4_fused_moe_host_workspace_bytes(M, topk, H, self.I, self.E)
        ws = workspace(dev, nws)
        flags = self._flags | (_lib.MOE_ROUTER_WEIGHT_ON_INPUT if apply_router_weight_on_input else 0)
        with torch.cuda.device(dev):
            rc = self._lib.b200fp4_fused_sparse_moe_host(
                hidden_host.data_ptr(), dtype_code(hidden_host.dtype), topk_weights_host.data_ptr(), topk_ids_host.data_ptr(),
                *self._head, out_host.data_ptr(), dtype_code(out_host.dtype), M, topk, H, self.I, self.E, flags,
                ws.data_ptr(), ws.numel(), stream_ptr(dev))
        _lib.check(rc, "fused_sparse_moe_v7 (host buffers)")
        return out_host


    def submit_host(self, hidden_host, topk_weights_host, topk_ids_host, out_host, slot: int = 0,
                    overlap_copies: bool = True, direct_out: bool = True, apply_router_weight_on_input: bool = False):
        """forward_host without the wait: queues the copies in, the layer and the copy out and returns a CUDA event
        that completes when out_host holds the result.  Steps submitted with different `slot` values use different
        staging buffers, so with overlap_copies the inputs of one step travel (on a copy stream of this object) while
        the previous step computes; every step in flight needs its own out_host.  With direct_out the layer's last
        kernel stores the result rows and the status word straight into pinned host memory (no copy out is queued:
        a copy between two layers costs the stream about 5 us).  wait_host() waits
        for everything submitted and raises if a layer reported an expired wait."""
        M, H = hidden_host.shape
        topk = topk_ids_host.shape[1]
        require(not hidden_host.is_cuda and not topk_weights_host.is_cuda and not topk_ids_host.is_cuda and
                not out_host.is_cuda, "submit_host takes CPU tensors")
        require(H == self.H and hidden_host.is_contiguous() and hidden_host.dtype in (torch.float16, torch.bfloat16),
                "hidden_host must be a contiguous [M,H] 16-bit tensor")
        require(topk_weights_host.dtype == torch.float32 and topk_ids_host.dtype == torch.int32 and
                topk_weights_host.is_contiguous() and topk_ids_host.is_contiguous() and
                tuple(topk_weights_host.shape) == (M, topk), "topk_weights f32 / topk_ids i32 must be contiguous [M, topk]")
        require(out_host.is_contiguous() and tuple(out_host.shape) == (M, H) and
                out_host.dtype in (torch.float16, torch.bfloat16), "out_host must be a contiguous [M,H] 16-bit CPU tensor")
        require(hidden_host.is_pinned() and topk_weights_host.is_pinned() and topk_ids_host.is_pinned() and
                out_host.is_pinned(), "submit_host needs pinned host tensors (pageable copies would block the queue)")
        dev = self.device
        key = ("host_slot", M, topk, int(slot))
        st = self._host_slots.get(key)
        if st is None:
            nws = self._lib.b200fp4_fused_moe_host_workspace_bytes(M, topk, H, self.I, self.E)
            st = self._host_slots[key] = (torch.empty(nws, dtype=torch.uint8, device=dev),
                                          torch.zeros(1, dtype=torch.int32).pin_memory())
        ws, status = st
        if overlap_copies and self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=dev)
        flags = self._flags | (_lib.MOE_ROUTER_WEIGHT_ON_INPUT if apply_router_weight_on_input else 0)
        flags |= _lib.MOE_HOST_DIRECT_OUT if direct_out else 0
        with torch.cuda.device(dev):
            rc = self._lib.b200fp4_fused_sparse_moe_host_async(
                hidden_host.data_ptr(), dtype_code(hidden_host.dtype), topk_weights_host.data_ptr(), topk_ids_host.data_ptr(),
                *self._head, out_host.data_ptr(), dtype_code(out_host.dtype), status.data_ptr(), M, topk, H, self.I, self.E,
                flags, ws.data_ptr(), ws.numel(), stream_ptr(dev),
                self._copy_stream.cuda_stream if overlap_copies else None)
            _lib.check(rc, "fused_sparse_moe_v7 (host buffers, queued)")
            done = torch.cuda.Event()
            done.record(torch.cuda.current_stream(dev))
        return done

    def wait_host(self):
        """Waits for every step queued by submit_host on the current stream and checks their status words."""
        torch.cuda.current_stream(self.device).synchronize()
        for _, status in self._host_slots.values():
            if int(status[0]) != 0:
                status.zero_()
                raise _lib.B200Fp4Error(STATUS_INTERNAL_ERROR, "fused_sparse_moe_v7 (host buffers, queued)")


def convert_weight_batch_to_v7(weights, scales, g_scales, device="cuda", batch_size=16):
    """NVFP4 expert weights -> the 2:4 tensors the ops above take, on the GPU in two launches.

    Mirrors convert_weight_batch_to_v7 (sparse_fp4_kernel/sparse_v7_moe_patch.py:96-129): weights
    [E,N,K/2] uint8, scales [E,N,G] e4m3, g_scales [E] -> (comp_T [E,K/4,N], meta_T [E,K/8,N],
    scale_T [E,G,N], g_scales f32 on the device).  batch_size is accepted for signature
    compatibility.  Ties between equal magnitudes keep the lower index."""
    dev = torch.device(device)
    w = weights.to(dev).contiguous()
    sc = scales.to(dev).contiguous()
    require(w.dim() == 3 and w.dtype == torch.uint8, "weights must be [E,N,K/2] uint8")
    require(sc.dim() == 3 and sc.shape[:2] == w.shape[:2], "scales must be [E,N,G]")
    E, N, K2 = w.shape
    K, G = K2 * 2, sc.shape[2]
    require(K % 8 == 0, "K must be a multiple of 8")
    comp_T = torch.empty((E, K // 4, N), dtype=torch.uint8, device=dev)
    meta_T = torch.empty((E, K // 8, N), dtype=torch.uint8, device=dev)
    scale_T = torch.empty((E, G, N), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().b200fp4_convert_to_sparse_2of4(ptr(w), ptr(sc), E, N, K, G, ptr(comp_T), ptr(meta_T),
                                                            ptr(scale_T), stream_ptr(dev)), "convert_weight_batch_to_v7")
    return comp_T, meta_T, scale_T, g_scales.float().to(dev)
