"""Grouped-query attention mixer over the paged cache.

Per token: q, k, v projections (one stacked product), RMSNorm of every Q and K
head over head_dim with one gain vector each (the formula of the reference's
head_norm sketch, cuda/attention.cu:169-182; its forward never applies it), rotary
rotation of Q and K, K and V stored in the request's pages, then softmax attention
of each query over the keys of its own request up to its position (and, with
``window`` W, not further back than W keys), query head h reading KV head
h // (heads / kv_heads) with scores scaled by 1/sqrt(head_dim)
(src/model.cpp:1000-1052), and the output projection.

A run with ``writes=False`` reads a cache that another run filled: only the query
side is computed, and the part must have been built with ``has_kv`` False.
"""
from __future__ import annotations

import os

import numpy as np
import torch

from .. import ops, workspace
from ..registry import PartSpec, part_class
from ..weights.loader import TensorSpec
from .base import CacheSpec, Mixer
from .linear import choose_splits, matmul_tn

DECODE_ROWS = 8     # rows a block of the decode variant of the plain attention kernel holds
SPAN_ROWS = 32      # rows of its prompt-portion variant
MMA_DECODE_ROWS = 16   # the same for the tensor-core kernel
MMA_SPAN_ROWS = 128
MAX_SLICES = 64
BLOCKS_PER_SM = 2         # blocks of the decode kernel that are resident at once on one SM
SHORT_CONTEXT = 8192      # contexts up to here count as short for the slicing of decoded tokens' key ranges
SHORT_SLICES = int(os.environ.get("VLLM_CPP_B200_ATTN_SHORT_SLICES", "12"))
# prompt portions run on the tcgen05 kernel where it takes the sizes; 0 keeps them on the mma.sync kernel (comparison runs)
TCGEN05_SPANS = os.environ.get("VLLM_CPP_B200_ATTN_TCGEN05", "1") != "0"
# Steps of single tokens only that run kernel by kernel: norm, rotation and cache store inside the attention kernel
# (0 keeps them a kernel of their own; 2 fuses in captured steps too).  Kernel by kernel a launch less in every layer
# is 7 % of the step (batch 8, 8B sizes: 2.70 -> 2.50 ms for 12 layers).  Inside a captured step it gains nothing
# (1.625 against 1.624 ms; context 2,176: 1.515 against 1.508): the blocks of the attention kernel become resident
# only as the projection's blocks leave, and what the separate kernel did meanwhile they now do after their wait.
FUSED_DECODE = int(os.environ.get("VLLM_CPP_B200_ATTN_FUSED_DECODE", "1"))
# The blocks of a decoded token's key slices run as a thread-block cluster and merge their results through shared
# memory (up to MAX_CLUSTER slices; more are merged by the last block through global memory).  0 switches it off.
CLUSTER_MERGE = os.environ.get("VLLM_CPP_B200_ATTN_CLUSTER", "1") != "0"
# Prompt portions of more than QKV_EPILOGUE_ABOVE tokens with head_dim 128 and whole-head half-split rotation: norm,
# rotation and cache store in the q, k, v projection's epilogue (VLLM_CPP_B200_QKV_EPILOGUE=0 keeps the separate
# kernel).  The epilogue of a block's last unit is not hidden behind a next one, so it pays from about 1,500 tokens on
# (8B sizes, product and norm-rotate-store against the one kernel: 1,024 tokens 60.2 against 62.9 us, 1,536 71.8
# against 63.6, 2,048 100.4 against 94.4, 3,072 142 against 118, 8,192 437 against 326).
QKV_EPILOGUE = os.environ.get("VLLM_CPP_B200_QKV_EPILOGUE", "1") != "0"
QKV_EPILOGUE_ABOVE = int(os.environ.get("VLLM_CPP_B200_QKV_EPILOGUE_ABOVE", "1280"))
# From this many tokens on the epilogue also replaces a projection that would be cut into k-slices: the one kernel
# without slices against the sliced product and the kernel that adds and norms its partial sums, 8B sizes at 256
# tokens 28.8 against 29.4 us, 4B 23.7 against 26.6, 14B 33.0 against 37.9 (768 tokens: 64.8 against 93.3); below,
# the slices win (144 tokens: 27.9 against 22.6).  A step of 256 single tokens: 8.27 -> 8.15 ms.
QKV_EPILOGUE_FOR_SLICES_FROM = 256
MAX_CLUSTER = 8
MAX_CLUSTER_SHARED = 6
# Steps with more (decoded token, KV head) pairs than the decode kernel has resident blocks: persistent blocks walk the
# pairs, their loading warp running ahead from one pair into the next (ops.attn_stream), instead of a block a pair
# that lives for one round trip to memory.  Kernel alone, 8B sizes: 256 tokens over 128 keys 47.3 -> 27.4 us (their
# keys take 20.5 at the copy bandwidth), 128 over 256 36.3 -> 26.2, 64 over 512 28.6 -> 25.6, 256 over 1,024
# 171 -> 156; with a pair a block or fewer it gains nothing (32 tokens over 2,048 keys: 42.2 against 43.2).
# Over long contexts the two forms take the same time alone (64 tokens over 4,096 keys: 157 us), but in the step the
# persistent one is 2 % behind (10.03 -> 10.25 ms): its blocks all end together, so the output projection's blocks are
# not resident, with their first weights on the way, before the attention is over.  So it is taken where the longest
# context is known to be at most STREAM_MAX_CONTEXT, and in captured steps, which serve any context of their class,
# from STREAM_STATIC_PAIRS pairs on, which no pool holds at long contexts.
# VLLM_CPP_B200_ATTN_STREAM=0 keeps a block a pair; 2 sends every step's single tokens this way, one slice each (tests).
STREAM_DECODE = int(os.environ.get("VLLM_CPP_B200_ATTN_STREAM", "1"))
STREAM_MAX_CONTEXT = 2048
STREAM_STATIC_PAIRS = 1184


class AttentionPlan:
    """Work items of the attention kernel for one step and one head layout, on the device."""

    def __init__(self, ctx, nh: int, nkv: int, decode_rows: int = DECODE_ROWS, span_rows: int = SPAN_ROWS,
                 cluster_hd: int | None = None, one_slice: bool = False):
        """``cluster_hd``: the head size, when the kernel that takes the decoded tokens can merge a token's key slices
        within a cluster of its blocks (then the slices are chosen so that all clusters run at once); else None.
        ``one_slice``: no key slices, whatever the contexts."""
        g = nh // nkv
        dev = ctx.device
        # int32 arrays go to the device with the step's own staging buffers where the step has them
        upload = getattr(ctx, "upload", None) or (lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev))
        dec = [i for i, n in enumerate(ctx.host_q_len) if n == 1]
        spans = [i for i, n in enumerate(ctx.host_q_len) if n > 1]
        self.n_dec = len(dec)
        self.decode_only = bool(dec) and not spans     # every entry of the step is one decoded token (or empty)
        self.nslices = 1
        self.longest = None   # the longest context among the single tokens, where the step knows it
        self.cluster = 0      # > 1: a token's key slices are a cluster of that many blocks
        self.dec_items = self.dec_rows = self.span_items = None
        self.n_span_items = 0
        if dec:
            hchunks = -(-g // min(g, decode_rows))
            blocks = len(dec) * nkv * hchunks
            if getattr(ctx, "static", False):
                # a captured step serves every context length up to the bound it was captured for (None: any)
                longest = getattr(ctx, "static_max_ctx", None)
                by_pages = MAX_SLICES if longest is None else max(1, longest // 128)
            else:
                longest = self.longest = max(ctx.host_ctx_len[i] for i in dec)
                by_pages = max(1, longest // 128)   # at least 128 keys a slice
            # as many slices as keep every block resident in one wave; over short contexts no more than
            # SHORT_SLICES, beyond which merging the partial results costs more than the shorter key ranges save
            # (one request at 4,096 keys, 12-layer step: 8 slices 1.437 ms, 12: 1.420, 18: 1.444, 37: 1.495)
            fit = BLOCKS_PER_SM * ops.num_sms() // blocks
            if longest is not None and longest <= SHORT_CONTEXT:
                fit = min(fit, SHORT_SLICES)
            self.nslices = 1 if one_slice else int(max(1, min(MAX_SLICES, by_pages, fit)))
            if cluster_hd is not None and longest is not None and longest <= SHORT_CONTEXT and self.nslices > 1:
                # Over short contexts the slices of a token are a cluster that merges through shared memory, which
                # saves the merge's trip through global memory (3 to 6 us a layer) -- if all the clusters run at
                # once: the largest number of slices, eight at most, of which the device takes that many clusters
                # (a cluster stays within one GPC, so sizes that do not divide a GPC's SMs leave some idle).
                # Clusters of more than six blocks only where every block has an SM to itself: two to an SM, clusters of
                # eight start late (four requests, 12-layer step: six slices 1.433 ms, eight 1.558, none clustered 1.487).
                sms = ops.num_sms()
                for s in range(min(self.nslices, MAX_CLUSTER), 1, -1):
                    alone = blocks * s <= sms
                    if (alone or s <= MAX_CLUSTER_SHARED) and blocks <= ops.attn_mma_max_clusters(cluster_hd, s, alone):
                        self.nslices = self.cluster = s
                        break
            items = np.zeros((len(dec) * self.nslices, ops.ITEM_INTS), dtype=np.int32)
            k = 0
            for n, e in enumerate(dec):
                for s in range(self.nslices):
                    items[k] = (e, 0, 1, s, self.nslices, n)
                    k += 1
            self.dec_items = upload(items)
            self.dec_rows = upload(np.asarray([ctx.host_q_start[e] for e in dec], dtype=np.int32))
            # arrival counters of the key slices (the tensor-core kernel merges in its last-arriving block)
            self.slice_counters = workspace.zeros((len(dec) * nkv * hchunks,), torch.int32, dev)
        if spans:
            nq_max = max(1, span_rows // min(g, span_rows))
            rows = []
            for e in spans:
                n = ctx.host_q_len[e]
                for q0 in range(0, n, nq_max):
                    rows.append((e, q0, min(nq_max, n - q0), 0, 1, 0))
            # longest key ranges first: the blocks that run longest start first, the short ones fill the tail
            rows.sort(key=lambda r: -(ctx.host_ctx_len[r[0]] - ctx.host_q_len[r[0]] + r[1] + r[2]))
            self.n_span_items = len(rows)
            self.span_items = upload(np.asarray(rows, dtype=np.int32).reshape(-1, ops.ITEM_INTS))
            # the queue that the tensor-core kernel's blocks take their work from (left at zero by every launch)
            self.span_work = workspace.zeros((2,), torch.int32, dev)


def stream_pays(plan: AttentionPlan, nkv: int) -> bool:
    """Whether a step's single tokens go to the kernel whose persistent blocks walk the (token, KV head) pairs: more
    pairs than resident blocks, no key slices, and short contexts (known, or implied by the number of pairs)."""
    pairs = plan.n_dec * nkv
    if not STREAM_DECODE or plan.nslices != 1 or pairs <= BLOCKS_PER_SM * ops.num_sms():
        return False
    return plan.longest <= STREAM_MAX_CONTEXT if plan.longest is not None else pairs >= STREAM_STATIC_PAIRS


class GQAAttention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``eps``
    (of the per-head norms), ``qk_norm`` (bool), ``window`` (0: all keys), ``has_kv``
    (bool, default True), ``position`` (a PartSpec of the position family).
    Tensors under ``<prefix>``: q_proj.weight [nh*hd, H], k_proj.weight, v_proj.weight
    [nkv*hd, H], o_proj.weight [H, nh*hd], q_norm.weight, k_norm.weight [hd]."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        p = params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv, self.hd = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        self.eps = float(p.get("eps", 1e-6))
        self.qk_norm = bool(p.get("qk_norm", True))
        self.window = int(p.get("window") or 0)
        self.has_kv = bool(p.get("has_kv", True))
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} query heads are not a multiple of {self.nkv} KV heads")
        if self.hd % 16 or not 16 <= self.hd <= 256:
            raise ValueError(f"head_dim {self.hd} is not supported: the kernels take multiples of 16 from 16 to 256")
        pos: PartSpec = p["position"]
        self.rope = part_class("position", pos.kind)(pos.params, prefix, build)
        # what the position part asks of the norm-rotate-store kernel (a part without these wants all lanes, in halves)
        self.rotary_dim = int(getattr(self.rope, "rotary_dim", self.hd))
        self.interleaved = getattr(self.rope, "pairing", "half") == "interleaved"
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None

    def cache_spec(self):
        return CacheSpec("kv", num_kv_heads=self.nkv, head_dim=self.hd, window=self.window)

    def tensor_specs(self):
        p, H, nh, nkv, hd = self.prefix, self.hidden, self.nh, self.nkv, self.hd
        specs = [TensorSpec(p + "q_proj.weight", (nh * hd, H)), TensorSpec(p + "o_proj.weight", (H, nh * hd))]
        if self.has_kv:
            specs += [TensorSpec(p + "k_proj.weight", (nkv * hd, H)), TensorSpec(p + "v_proj.weight", (nkv * hd, H))]
        if self.qk_norm:
            specs.append(TensorSpec(p + "q_norm.weight", (hd,), "vector"))
            if self.has_kv:
                specs.append(TensorSpec(p + "k_norm.weight", (hd,), "vector"))
        return specs

    def bind(self, store):
        p = self.prefix
        names = [p + "q_proj.weight"] + ([p + "k_proj.weight", p + "v_proj.weight"] if self.has_kv else [])
        self.w_qkv = store.matrices(names)
        self.w_o = store.matrix(p + "o_proj.weight")
        if self.qk_norm:
            self.q_norm_w = store.vector(p + "q_norm.weight")
            if self.has_kv:
                self.k_norm_w = store.vector(p + "k_norm.weight")
                if self.k_norm_w.dtype != self.q_norm_w.dtype:
                    self.k_norm_w = self.k_norm_w.float()
                    self.q_norm_w = self.q_norm_w.float()

    def forward(self, x, ctx, cache, writes=True):
        if writes != self.has_kv:
            raise ValueError("an attention part built with has_kv must write its cache, one without must not")
        T = x.shape[0]
        nh, nkv, hd = self.nh, self.nkv, self.hd
        group = ctx.groups[cache.group]
        # Prompt portions whose projection needs no k-slices: the per-head norm, the rotation and the cache store run in
        # the projection's epilogue (a unit of 128 features is one head), from its 32-bit sums.
        in_epilogue = (QKV_EPILOGUE and x.dtype == torch.bfloat16 and hd == 128 and self.rotary_dim == hd and not self.interleaved
                       and T > min(QKV_EPILOGUE_ABOVE, QKV_EPILOGUE_FOR_SLICES_FROM - 1) and ops.gemm_tma_ok(x, self.w_qkv)
                       and (not self.has_kv or (cache.pages.dtype == torch.bfloat16 and cache.pages.is_contiguous())))
        if in_epilogue:
            sliced = ops.gemm_effective_splits(x.shape[1], choose_splits(self.w_qkv.shape[0], T, x.shape[1])) > 1
            in_epilogue = (T >= QKV_EPILOGUE_FOR_SLICES_FROM) if sliced else (T > QKV_EPILOGUE_ABOVE)
        # (the mixer's input comes from a norm: a short kernel)
        qkv = None if in_epilogue else matmul_tn(x, self.w_qkv, ctx.status, allow_partials=True, after_small_kernel=True)
        out = workspace.empty((T, nh * hd), x.dtype, x.device)
        mma = ops.attn_mma_supported(x.dtype, hd)
        kernel = ops.attn_mma if mma else ops.attn_paged
        dec_rows, span_rows = (MMA_DECODE_ROWS, MMA_SPAN_ROWS) if mma else (DECODE_ROWS, SPAN_ROWS)
        clustered = hd if mma and CLUSTER_MERGE and torch.cuda.is_available() else None
        always_stream = STREAM_DECODE == 2 and mma and ops.attn_stream_supported(x.dtype, hd, cache.pages.shape[3], nh, nkv)
        plan = ctx.plan(("attention", nh, nkv, mma, clustered, always_stream),
                        lambda: AttentionPlan(ctx, nh, nkv, dec_rows, span_rows, clustered, one_slice=always_stream))
        common = dict(nh=nh, nkv=nkv, hd=hd, window=self.window, status=ctx.status, table_row=ctx.slots)
        # many single tokens: more (token, KV head) pairs than blocks that are resident at once
        stream = bool(plan.n_dec) and (always_stream or (
            mma and stream_pays(plan, nkv) and ops.attn_stream_supported(x.dtype, hd, cache.pages.shape[3], nh, nkv)))
        # A step of single tokens only, run kernel by kernel: the attention kernel norms, rotates and stores for itself,
        # straight from the projection's k-slice partial sums (one launch less in every layer).
        if (not stream and qkv is not None and (FUSED_DECODE == 2 or (FUSED_DECODE == 1 and not getattr(ctx, "static", False))) and mma and plan.decode_only and self.has_kv and qkv.dim() == 3 and nh // nkv <= MMA_DECODE_ROWS
                and self.rotary_dim == hd and not self.interleaved
                and ops.attn_mma_fused_supported(x.dtype, hd, cache.pages.shape[3])):
            S = plan.nslices
            cluster = plan.cluster
            part_o = part_ml = None
            if S > 1 and not cluster:
                part_o = workspace.empty((plan.n_dec * nh * S, hd), torch.float32, x.device)
                part_ml = workspace.empty((plan.n_dec * nh * S, 2), torch.float32, x.device)
            ops.attn_mma_decode_fused(qkv, self.q_norm_w, self.k_norm_w, self.eps, self.rope.table,
                                      group.slot_map, out, cache.pages, group.block_table, ctx.q_start, ctx.q_len,
                                      ctx.ctx_len, plan.dec_items, plan.n_dec * S, part_o, part_ml,
                                      plan.slice_counters if S > 1 else None, plan.dec_rows, use_norm=self.qk_norm,
                                      cluster=cluster, **common)
            return matmul_tn(out, self.w_o, ctx.status, out_dtype=torch.float32, allow_partials=True)
        q = workspace.empty((T, nh * hd), x.dtype, x.device)
        if in_epilogue:
            ops.gemm_qkv_rope(self.w_qkv, x, q, cache.pages if self.has_kv else None, group.slot_map, ctx.positions,
                              self.rope.table, self.q_norm_w, self.k_norm_w, self.eps, nh, nkv, ctx.status, use_norm=self.qk_norm)
        else:
            ops.qknorm_rope_kvwrite(qkv, self.q_norm_w, self.k_norm_w, self.eps, self.rope.table, ctx.positions,
                                    group.slot_map, q, cache.pages, nh, nkv, hd, ctx.status,
                                    has_kv=self.has_kv, use_norm=self.qk_norm, rotary_dim=self.rotary_dim,
                                    interleaved=self.interleaved)
        if stream:
            ops.attn_stream(q, out, cache.pages, group.block_table, ctx.q_len, ctx.ctx_len, plan.dec_items, plan.n_dec,
                            plan.dec_rows, **common)
        elif plan.n_dec:
            S = plan.nslices
            cluster = plan.cluster if mma else 0
            part_o = part_ml = None
            if S > 1 and not cluster:
                part_o = workspace.empty((plan.n_dec * nh * S, hd), torch.float32, x.device)
                part_ml = workspace.empty((plan.n_dec * nh * S, 2), torch.float32, x.device)
            if mma:
                ops.attn_mma(q, out, cache.pages, group.block_table, ctx.q_start, ctx.q_len, ctx.ctx_len,
                             plan.dec_items, plan.n_dec * S, dec_rows, part_o, part_ml,
                             slice_counters=plan.slice_counters if S > 1 else None, dec_rows=plan.dec_rows,
                             cluster=cluster, **common)
            else:
                ops.attn_paged(q, out, cache.pages, group.block_table, ctx.q_start, ctx.q_len, ctx.ctx_len,
                               plan.dec_items, plan.n_dec * S, dec_rows, part_o, part_ml, **common)
                if S > 1:
                    ops.attn_merge(part_o, part_ml, plan.dec_rows, out, plan.n_dec, nh, hd, S)
        if plan.n_span_items and mma and TCGEN05_SPANS and ops.attn_tc_supported(x.dtype, hd, cache.pages.shape[3]):
            ops.attn_tc(q, out, cache.pages, group.block_table, ctx.q_start, ctx.q_len, ctx.ctx_len,
                        plan.span_items, plan.n_span_items, work=plan.span_work, **common)
        elif plan.n_span_items:
            kernel(q, out, cache.pages, group.block_table, ctx.q_start, ctx.q_len, ctx.ctx_len,
                   plan.span_items, plan.n_span_items, span_rows, None, None, **common)
        return matmul_tn(out, self.w_o, ctx.status, out_dtype=torch.float32, allow_partials=True)
