"""Expert-parallel MoE layers: E/G experts per GPU.

Decode (`ExpertParallelMoE`), three exchanges behind one interface:
  mode="p2p" (default for CUDA ranks)  this library's own kernels over peer memory (torch symmetric memory gives
      every rank the peers' buffer addresses): a dispatch kernel stores each token's record (activation row, top-k
      global expert ids, router weights) into every rank's record buffer with plain NVLink stores and publishes a
      step-numbered flag; the fused sparse MoE op runs over all ranks' records with `expert_map` masking the experts
      the rank does not own (-1 entries are skipped by the plan kernel, so foreign pairs cost no weight traffic) and
      its last kernel stores the fp32 partial rows straight into the owners' buffers; a combine kernel waits for the
      peers' flags, sums the G partial rows of every token and rounds once.  No collective call per step; every wait
      is bounded and reports through a status word (`p2p_status()`).
  mode="gather"  the same with collectives of the process group: one all-gather of the records, the fused op,
      one reduce-scatter of the fp32 partial rows (default for CPU stand-in ranks; what the benchmark falls back to
      if the peer-memory exchange reports an expired wait).
  mode="a2a"  fixed-capacity all-to-all dispatch of G copies, all-to-all of 16-bit partial rows, fp32 sum at the
      source (kept for comparison).
With top-10 of 512 experts a token has an expert on nearly every rank, so "send a token only where it is needed"
saves nothing over sending every record everywhere; the sizes are fixed, so no split-size exchange or host round
trip sits on the decode path.
Prefill (`ExpertParallelMoEPrefill`): all-gather of the token block, grouped NVFP4 path over the local
experts, reduce-scatter of the partial output rows.

The reference has no multi-GPU code of its own (it serves with tensor parallelism through vLLM);
this layout is the one the path's shard rule prescribes: experts [r*E/G, (r+1)*E/G) live on rank r.

Limits: the fused layer takes at most 65535 (token, expert) pairs per call, i.e. G*B*topk <= 65535
(B <= 819 tokens per rank at 8 ranks and top-10); `forward` raises before anything is enqueued.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def expert_map_for_rank(global_E: int, world: int, rank: int, device) -> torch.Tensor:
    """global expert id -> local id on `rank`, -1 for experts owned elsewhere."""
    per = global_E // world
    m = torch.full((global_E,), -1, dtype=torch.int32)
    m[rank * per:(rank + 1) * per] = torch.arange(per, dtype=torch.int32)
    return m.to(device)


def pack_records(hidden: torch.Tensor, topk_w: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
    """[B,H] act + [B,topk] i32 ids + [B,topk] f32 weights -> [B, H*2 + topk*8] bytes."""
    B = hidden.shape[0]
    return torch.cat((hidden.contiguous().view(torch.uint8).reshape(B, -1),
                      topk_ids.to(torch.int32).contiguous().view(torch.uint8).reshape(B, -1),
                      topk_w.to(torch.float32).contiguous().view(torch.uint8).reshape(B, -1)), dim=1)


def unpack_records(rec: torch.Tensor, H: int, topk: int, dtype: torch.dtype):
    n = rec.shape[0]
    hb = H * 2
    hidden = rec[:, :hb].contiguous().view(dtype).reshape(n, H)
    ids = rec[:, hb:hb + topk * 4].contiguous().view(torch.int32).reshape(n, topk)
    w = rec[:, hb + topk * 4:].contiguous().view(torch.float32).reshape(n, topk)
    return hidden, w, ids


class ExpertParallelMoE:
    """One MoE layer sharded over the ranks of `group`.

    With CUDA tensors the step is: ep_pack kernel -> all_gather -> fused sparse MoE reading the
    gathered records in place (fp32 partial rows) -> reduce_scatter -> cast (5 launches of this
    library + 2 collectives); mode="a2a": ep_pack (G copies) -> all_to_all -> fused layer (16-bit
    partial rows) -> all_to_all -> ep_combine.

    `local_moe_fn(hidden [T,H], topk_w [T,topk] f32, topk_ids [T,topk] i32 (global ids),
    expert_map [global_E] i32) -> [T,H]`, when given, replaces the CUDA ops and the torch
    packing path is used instead (this is how the dispatch/combine logic is tested on CPU ranks).

    `phase_events`: when set to a list of five CUDA events, forward records them before the pack, after
    it, after the dispatch collective, after the local layer and after the combine (benchmark hook)."""

    def __init__(self, global_E: int, inter: int, w13: Optional[dict], w2: Optional[dict], group=None,
                 local_moe_fn: Optional[Callable] = None, mode: Optional[str] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if global_E % self.world != 0:
            raise RuntimeError("the number of experts must be divisible by the number of ranks")
        if mode is None:     # CUDA ranks: this library's own exchange kernels; CPU stand-in ranks: collectives of the process group
            mode = "gather" if local_moe_fn is not None else "p2p"
        if mode not in ("gather", "a2a", "p2p"):
            raise RuntimeError("mode must be 'gather', 'a2a' or 'p2p'")
        self.global_E = global_E
        self.inter = inter
        self.w13, self.w2 = w13, w2
        self.mode = mode
        self.phase_events = None
        self._emap = None
        self._fn = local_moe_fn
        self._bufs = {}
        self._flags = None
        self._bound = None
        self._host_in = {}
        self._copy_stream = None
        self._p2p = None
        self._seq = 0

    def _cuda_local(self, hidden, topk_w, topk_ids, emap):
        if self._bound is None:       # weights are validated and their pointers bound once
            from . import sparse_fp4_v7 as sp7
            k = ("comp_T", "meta_T", "scale_T", "g_scales")
            self._bound = sp7.FusedSparseMoE(*[self.w13[x] for x in k], *[self.w2[x] for x in k], self.inter, expert_map=emap)
        return self._bound(hidden, topk_w, topk_ids)

    def expert_map(self, device) -> torch.Tensor:
        if self._emap is None or self._emap.device != device:
            self._emap = expert_map_for_rank(self.global_E, self.world, self.rank, device)
        return self._emap

    def _forward_torch(self, hidden, topk_w, topk_ids, emap):
        B, H = hidden.shape
        topk = topk_ids.shape[1]
        G = self.world
        rec = pack_records(hidden, topk_w, topk_ids)                       # [B, R]
        if self.mode == "gather":
            recv = torch.empty((G * B, rec.shape[1]), dtype=torch.uint8, device=rec.device)
            dist.all_gather_into_tensor(recv, rec.contiguous(), group=self.group)                # dispatch
            h_all, w_all, ids_all = unpack_records(recv, H, topk, hidden.dtype)
            part = self._fn(h_all, w_all, ids_all, emap).float().contiguous()   # [G*B, H] fp32 partial rows
            if dist.get_backend(self.group) == "gloo":                          # gloo has no reduce-scatter
                dist.all_reduce(part, group=self.group)
                out = part[self.rank * B:(self.rank + 1) * B]
            else:
                out = torch.empty((B, H), dtype=torch.float32, device=part.device)
                dist.reduce_scatter_tensor(out, part, group=self.group)                         # combine
            return out.to(hidden.dtype)
        send = rec.unsqueeze(0).expand(G, B, rec.shape[1]).contiguous()    # one slot block per peer
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv.view(G * B, -1), send.view(G * B, -1), group=self.group)     # dispatch
        h_all, w_all, ids_all = unpack_records(recv.view(G * B, -1), H, topk, hidden.dtype)
        part = self._fn(h_all, w_all, ids_all, emap)                       # [G*B, H] partial rows
        back = torch.empty_like(part)
        dist.all_to_all_single(back, part.contiguous(), group=self.group)  # combine
        return back.view(G, B, H).float().sum(0).to(hidden.dtype)

    def _forward_cuda(self, hidden, topk_w, topk_ids, emap):
        from . import _lib
        from ._torch_util import dtype_code, ptr, require, stream_ptr, workspace
        dev = hidden.device
        B, H = hidden.shape
        topk = topk_ids.shape[1]
        G = self.world
        L = _lib.lib()
        require(hidden.is_contiguous() and hidden.dtype in (torch.bfloat16, torch.float16), "hidden must be contiguous 16-bit")
        require(G * B * topk <= 65535, "the fused layer takes at most 65535 (token, expert) pairs: G*B*topk is larger")
        ids = topk_ids if topk_ids.dtype == torch.int32 else topk_ids.to(torch.int32)
        ids = ids.contiguous()
        tw = topk_w if topk_w.dtype == torch.float32 else topk_w.float()
        tw = tw.contiguous()
        R = L.b200fp4_ep_record_bytes(H, topk)
        gather = self.mode == "gather"
        key = (dev.index, B, H, topk, hidden.dtype, self.mode)
        bufs = self._bufs.get(key)
        if bufs is None:
            if gather:
                bufs = (torch.empty(B * R, dtype=torch.uint8, device=dev), torch.empty(G * B * R, dtype=torch.uint8, device=dev),
                        torch.empty(G * B, H, dtype=torch.float32, device=dev), torch.empty(B, H, dtype=torch.float32, device=dev))
            else:
                bufs = (torch.empty(G * B * R, dtype=torch.uint8, device=dev), torch.empty(G * B * R, dtype=torch.uint8, device=dev),
                        torch.empty(G * B, H, dtype=hidden.dtype, device=dev), torch.empty(G * B, H, dtype=hidden.dtype, device=dev))
            self._bufs[key] = bufs
        send, recv, part, back = bufs
        T = G * B
        E = self.global_E // G
        k = ("comp_T", "meta_T", "scale_T", "g_scales")
        ws = workspace(dev, L.b200fp4_fused_moe_workspace_bytes(T, topk, H, self.inter, E))
        code = dtype_code(hidden.dtype)
        if self._flags is None:   # ordered metadata -> tensor-core GEMVs; checked once per layer
            from .sparse_fp4_v7 import metadata_ordered
            ok = metadata_ordered(self.w13["meta_T"]) and metadata_ordered(self.w2["meta_T"])
            self._flags = _lib.SPARSE_META_ORDERED if ok else 0
            self._wptrs = ([ptr(self.w13[x]) for x in k] + [self.w13["scale_T"].shape[1]] +
                           [ptr(self.w2[x]) for x in k] + [self.w2["scale_T"].shape[1]])
        ev = self.phase_events
        st = torch.cuda.current_stream(dev)
        with torch.cuda.device(dev):
            if ev:
                ev[0].record(st)
            _lib.check(L.b200fp4_ep_pack(ptr(hidden), ptr(ids), ptr(tw), B, H, topk, 1 if gather else G, ptr(send),
                                         st.cuda_stream), "ep_pack")
            if ev:
                ev[1].record(st)
            if gather:
                dist.all_gather_into_tensor(recv, send, group=self.group)                          # dispatch
            else:
                dist.all_to_all_single(recv, send, group=self.group)
            if ev:
                ev[2].record(st)
            _lib.check(L.b200fp4_fused_sparse_moe_records(
                ptr(recv), R, code, ptr(emap), emap.numel(), *self._wptrs,
                ptr(part), dtype_code(part.dtype), T, topk, H, self.inter, E, self._flags, ptr(ws), ws.numel(),
                st.cuda_stream), "fused_sparse_moe_records")
            if ev:
                ev[3].record(st)
            if gather:
                dist.reduce_scatter_tensor(back, part, group=self.group)                           # combine
                out = back.to(hidden.dtype)
            else:
                dist.all_to_all_single(back, part, group=self.group)
                out = torch.empty(B, H, dtype=hidden.dtype, device=dev)
                _lib.check(L.b200fp4_ep_combine(ptr(back), code, B, H, G, ptr(out), st.cuda_stream), "ep_combine")
            if ev:
                ev[4].record(st)
        return out

    # ---- mode="p2p": dispatch and combine by this library's own kernels over peer memory (no NCCL call per step)
    def _p2p_setup(self, dev, B, H, topk):
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib
        G = self.world
        R = _lib.lib().b200fp4_ep_record_bytes(H, topk)
        align = lambda v: (v + 255) // 256 * 256
        off_rec = 1024                                      # [0, 1024): flags [2][G] int32
        off_parts = off_rec + align(G * B * R)
        total = off_parts + G * B * H * 4
        buf = symm_mem.empty(total, dtype=torch.uint8, device=dev)
        buf.zero_()
        group = self.group if self.group is not None else dist.group.WORLD
        hdl = symm_mem.rendezvous(buf, group)
        torch.cuda.synchronize(dev)
        dist.barrier(group=self.group)                      # every rank's flags are zero before anyone publishes one
        base = torch.tensor([int(p) for p in hdl.buffer_ptrs], dtype=torch.int64)
        self._p2p = {
            "key": (dev.index, B, H, topk), "buf": buf, "hdl": hdl, "R": R,
            "flag_ptrs": base.to(dev), "rec_ptrs": (base + off_rec).to(dev), "part_ptrs": (base + off_parts).to(dev),
            "rec_local": buf.data_ptr() + off_rec, "parts_local": buf.data_ptr() + off_parts,
            "scratch": torch.zeros(4, dtype=torch.int32, device=dev),
        }
        self._seq = 0

    def p2p_status(self) -> int:
        """0, or the code of the bounded wait for a peer that ran out in some step since set-up (synchronises)."""
        return 0 if self._p2p is None else int(self._p2p["scratch"][1].item())

    def _forward_p2p(self, hidden, topk_w, topk_ids, emap):
        from . import _lib
        from ._torch_util import dtype_code, ptr, require, stream_ptr, workspace
        dev = hidden.device
        B, H = hidden.shape
        topk = topk_ids.shape[1]
        G = self.world
        L = _lib.lib()
        require(hidden.is_contiguous() and hidden.dtype in (torch.bfloat16, torch.float16), "hidden must be contiguous 16-bit")
        require(G * B * topk <= 65535, "the fused layer takes at most 65535 (token, expert) pairs: G*B*topk is larger")
        require(not torch.cuda.is_current_stream_capturing(), "the peer-memory exchange numbers its steps on the host: not capturable")
        ids = (topk_ids if topk_ids.dtype == torch.int32 else topk_ids.to(torch.int32)).contiguous()
        tw = (topk_w if topk_w.dtype == torch.float32 else topk_w.float()).contiguous()
        if self._p2p is None or self._p2p["key"] != (dev.index, B, H, topk):
            self._p2p_setup(dev, B, H, topk)
        p = self._p2p
        T, E = G * B, self.global_E // G
        k = ("comp_T", "meta_T", "scale_T", "g_scales")
        ws = workspace(dev, L.b200fp4_fused_moe_workspace_bytes(T, topk, H, self.inter, E))
        code = dtype_code(hidden.dtype)
        if self._flags is None:
            from .sparse_fp4_v7 import metadata_ordered
            ok = metadata_ordered(self.w13["meta_T"]) and metadata_ordered(self.w2["meta_T"])
            self._flags = _lib.SPARSE_META_ORDERED if ok else 0
            self._wptrs = ([ptr(self.w13[x]) for x in k] + [self.w13["scale_T"].shape[1]] +
                           [ptr(self.w2[x]) for x in k] + [self.w2["scale_T"].shape[1]])
        self._seq += 1
        out = torch.empty(B, H, dtype=hidden.dtype, device=dev)
        ev = self.phase_events
        st = torch.cuda.current_stream(dev)
        with torch.cuda.device(dev):
            if ev:
                ev[0].record(st)
                ev[1].record(st)
            _lib.check(L.b200fp4_ep_dispatch_p2p(ptr(hidden), ptr(ids), ptr(tw), B, H, topk, G, self.rank, ptr(p["rec_ptrs"]),
                                                 ptr(p["flag_ptrs"]), self._seq, ptr(p["scratch"]), st.cuda_stream), "ep_dispatch_p2p")
            if ev:
                ev[2].record(st)
            _lib.check(L.b200fp4_fused_sparse_moe_records_scatter(
                p["rec_local"], p["R"], code, ptr(emap), emap.numel(), *self._wptrs, ptr(p["part_ptrs"]), B, self.rank * B,
                _lib.F32, T, topk, H, self.inter, E, self._flags, ptr(ws), ws.numel(), st.cuda_stream),
                "fused_sparse_moe_records_scatter")
            if ev:
                ev[3].record(st)
            _lib.check(L.b200fp4_ep_combine_p2p(p["parts_local"], B, H, G, self.rank, ptr(p["flag_ptrs"]), self._seq,
                                                ptr(p["scratch"]), ptr(out), code, st.cuda_stream), "ep_combine_p2p")
            if ev:
                ev[4].record(st)
        return out

    def forward(self, hidden: torch.Tensor, topk_w: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        emap = self.expert_map(hidden.device)
        if self.world == 1:
            fn = self._fn or self._cuda_local
            return fn(hidden, topk_w, topk_ids, emap)
        if self._fn is not None:
            return self._forward_torch(hidden, topk_w, topk_ids, emap)
        if self.mode == "p2p":
            return self._forward_p2p(hidden, topk_w, topk_ids, emap)
        return self._forward_cuda(hidden, topk_w, topk_ids, emap)


    def _bound_layer(self, device):
        if self._bound is None:
            from . import sparse_fp4_v7 as sp7
            k = ("comp_T", "meta_T", "scale_T", "g_scales")
            self._bound = sp7.FusedSparseMoE(*[self.w13[x] for x in k], *[self.w2[x] for x in k], self.inter,
                                             expert_map=self.expert_map(device))
        return self._bound

    def forward_host(self, hidden_host, topk_w_host, topk_ids_host, out_host, device) -> torch.Tensor:
        """forward for CPU tensors (pinned for asynchronous copies); out_host is valid on return.  On one GPU this
        is a single call of the library's host-buffer entry point; with several ranks the copies bracket forward."""
        if self.world == 1 and self._fn is None:
            return self._bound_layer(device).forward_host(hidden_host, topk_w_host, topk_ids_host, out_host=out_host)
        self.submit_host(hidden_host, topk_w_host, topk_ids_host, out_host, device)
        self.wait_host(device)
        return out_host

    def submit_host(self, hidden_host, topk_w_host, topk_ids_host, out_host, device, slot: int = 0):
        """forward_host without the wait, for a caller that keeps several steps in flight (every step in flight has
        its own out_host).  Returns a CUDA event that completes when out_host holds the result; wait_host() waits for
        everything submitted.  On one GPU the inputs of a step travel on a copy stream while the step before it
        computes (steps alternate between staging buffers by `slot`)."""
        if self.world == 1 and self._fn is None:
            return self._bound_layer(device).submit_host(hidden_host, topk_w_host, topk_ids_host, out_host, slot=slot)
        if self._fn is not None:        # CPU ranks (tests): nothing to queue
            out_host.copy_(self.forward(hidden_host.to(device), topk_w_host.to(device), topk_ids_host.to(device)))
            return None
        # several ranks: the inputs travel on a copy stream into one of the staging slots while the previous step
        # computes; the exchange, the local layer and the copy out follow on the current stream
        cur = torch.cuda.current_stream(device)
        key = (int(slot), tuple(hidden_host.shape), tuple(topk_ids_host.shape), hidden_host.dtype)
        st = self._host_in.get(key)
        if st is None:
            if self._copy_stream is None:
                self._copy_stream = torch.cuda.Stream(device=device)
            st = self._host_in[key] = {
                "h": torch.empty(hidden_host.shape, dtype=hidden_host.dtype, device=device),
                "w": torch.empty(topk_w_host.shape, dtype=topk_w_host.dtype, device=device),
                "ids": torch.empty(topk_ids_host.shape, dtype=topk_ids_host.dtype, device=device),
                "loaded": torch.cuda.Event(), "consumed": torch.cuda.Event(), "used": False}
        cs = self._copy_stream
        with torch.cuda.stream(cs):
            if st["used"]:
                cs.wait_event(st["consumed"])
            st["ids"].copy_(topk_ids_host, non_blocking=True)
            st["w"].copy_(topk_w_host, non_blocking=True)
            st["h"].copy_(hidden_host, non_blocking=True)
            st["loaded"].record(cs)
        cur.wait_event(st["loaded"])
        out = self.forward(st["h"], st["w"], st["ids"])
        st["consumed"].record(cur)
        st["used"] = True
        out_host.copy_(out, non_blocking=True)
        done = torch.cuda.Event()
        done.record(cur)
        return done

    def wait_host(self, device) -> None:
        if self.world == 1 and self._fn is None:
            self._bound_layer(device).wait_host()
            return
        if self._fn is None:         # CPU ranks have nothing queued
            torch.cuda.current_stream(device).synchronize()


class ExpertParallelMoEPrefill:
    """One dense-NVFP4 MoE layer for prefill, experts sharded over the ranks of `group`.

    Every rank holds a block of Tl tokens and the weights of its E/G experts (the arguments of
    `grouped_moe.nvfp4_moe_prefill` for those experts).  forward: all-gather of the tokens and of the packed
    routing -> grouped path over the local experts with `expert_map` masking the others (pairs of foreign
    experts contribute nothing) -> reduce-scatter of the 16-bit partial rows -> [Tl, H].

    `local_fn(hidden [T,H], topk_w [T,k], topk_ids [T,k], expert_map [global_E]) -> [T,H]`, when given,
    replaces the CUDA path (CPU ranks in tests; gloo has no reduce-scatter, so an all-reduce + slice
    stands in for it there)."""

    def __init__(self, global_E: int, weights: Optional[tuple], group=None, local_fn: Optional[Callable] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if global_E % self.world != 0:
            raise RuntimeError("the number of experts must be divisible by the number of ranks")
        self.global_E = global_E
        self.weights = weights       # (w13_codes, w13_sf, w13_gs, w2_codes, w2_sf, w2_gs, a1_gs, a2_gs) of the local experts
        self._fn = local_fn
        self._emap = None
        self._alphas = None
        self._bufs = {}
        self._graphs = {}
        self.use_graph = local_fn is None      # CUDA ranks: the local layer's dozen launches replay from one CUDA graph

    def _local(self, hidden, topk_w, topk_ids, emap):
        if self._fn is not None:
            return self._fn(hidden, topk_w, topk_ids, emap)
        from .grouped_moe import nvfp4_moe_alphas, nvfp4_moe_prefill
        if self._alphas is None:     # layer constants
            w = self.weights
            self._alphas = nvfp4_moe_alphas(w[2], w[5], w[6], w[7])
        return nvfp4_moe_prefill(hidden, topk_w, topk_ids, *self.weights, expert_map=emap, alphas=self._alphas)

    def _local_step(self, b, key):
        """The local layer over the gathered buffers.  On CUDA ranks its launches (routing metadata, quantizer, two grouped
        GEMMs, un-permute) are captured once per shape and replayed: with 1/G of the experts per rank the kernels are
        short and a dozen separate Python-level launches would cost more than they run."""
        if not self.use_graph or not b["h"].is_cuda:
            return self._local(b["h"], b["w"], b["i"], self._emap)
        g = self._graphs.get(key)
        if g is None:
            self._local(b["h"], b["w"], b["i"], self._emap)      # first run outside the capture: one-time initialisation
            torch.cuda.synchronize(b["h"].device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = self._local(b["h"], b["w"], b["i"], self._emap)
            g = self._graphs[key] = (graph, out)
        g[0].replay()
        return g[1]

    def forward(self, hidden: torch.Tensor, topk_w: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        if self._emap is None or self._emap.device != hidden.device:
            self._emap = expert_map_for_rank(self.global_E, self.world, self.rank, hidden.device)
        G = self.world
        if G == 1:
            return self._local(hidden, topk_w, topk_ids, self._emap)
        Tl, H = hidden.shape
        k = topk_ids.shape[1]
        # routing travels as one [Tl, 2k] int32 block (ids | weight bits): two all-gathers instead of three
        route = torch.cat((topk_ids.to(torch.int32), topk_w.to(torch.float32).contiguous().view(torch.int32)), dim=1).contiguous()
        key = (Tl, H, k, hidden.dtype, hidden.device)
        b = self._bufs.get(key)
        if b is None:          # gathered inputs live in buffers of their own: their addresses are what a captured graph reads
            b = self._bufs[key] = {
                "h": torch.empty((G * Tl, H), dtype=hidden.dtype, device=hidden.device),
                "r": torch.empty((G * Tl, 2 * k), dtype=torch.int32, device=hidden.device),
                "i": torch.empty((G * Tl, k), dtype=torch.int32, device=hidden.device),
                "w": torch.empty((G * Tl, k), dtype=torch.float32, device=hidden.device)}
        dist.all_gather_into_tensor(b["h"], hidden.contiguous(), group=self.group)
        dist.all_gather_into_tensor(b["r"], route, group=self.group)
        b["i"].copy_(b["r"][:, :k])
        b["w"].view(torch.int32).copy_(b["r"][:, k:])
        part = self._local_step(b, key)                              # [G*Tl, H] partial rows in the activation dtype
        if dist.get_backend(self.group) == "gloo":
            part = part.float().contiguous()
            dist.all_reduce(part, group=self.group)
            return part[self.rank * Tl:(self.rank + 1) * Tl].to(hidden.dtype)
        # the partial rows are summed in their own 16-bit type: half the bytes of an fp32 exchange and no conversion passes;
        # a token has at most min(k, G) non-zero partial rows, well inside the layer's tolerance
        out = torch.empty((Tl, H), dtype=part.dtype, device=hidden.device)
        dist.reduce_scatter_tensor(out, part.contiguous(), group=self.group)
        return out
