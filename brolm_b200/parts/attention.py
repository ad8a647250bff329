"""The attention mixer: grouped-query attention with rotary positions, a
score scale of its own, tanh soft-capping of the scores and an optional
sliding window, over a paged cache.

Formulas as wlejon/brolm computes them (src/gemma2.cpp:349-369): fused q/k/v
projection without bias, rotation of q and k at the absolute position, k and
v into the cache, scores = q.k * scale -> cap * tanh(./cap) -> causal/window
mask -> softmax, then the output projection.  Key j is visible from position
p iff 0 <= p - j < window.

Options beside those: value heads of a size of their own (``v_dim``); an RMS
norm of the whole query row and of the whole key row, one statistic over all
heads, with a gain per element (``qk_norm="whole"``, tensors ``q_norm`` and
``k_norm``); a chunked mask (``chunk`` = C: key j is visible from p iff j <= p
and j >= p - p % C, chunks counted from position 0), kept in the cache as a
ring of C places like a window.  A layer that uses one of them runs its
projection with a float result, the row-wise kernel that norms and fills the
cache, and the exact attention kernel.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..cache import KVSpec
from .base import ParamSpec, Part, register_part
from .linear import linear


class Attention(Part):
    kind = "mixer"
    graph_safe = True

    def __init__(self, hidden: int, n_q: int, n_kv: int, head_dim: int, scale: float, softcap: float = 0.0,
                 window: Optional[int] = None, position: Optional[Part] = None, v_dim: Optional[int] = None,
                 qk_norm: str = "none", eps: float = 0.0, chunk: Optional[int] = None):
        if n_q % n_kv:
            raise ValueError("attention: the number of query heads must be a multiple of the kv heads")
        plain = not (v_dim and v_dim != head_dim) and qk_norm == "none" and not chunk
        if plain and head_dim % 16:
            raise ValueError(f"attention: head_dim {head_dim} is not a multiple of 16; the kernels refuse it")
        if head_dim > 512:
            raise ValueError(f"attention: head_dim {head_dim} is beyond the kernels' limit of 512")
        if qk_norm not in ("none", "whole"):
            raise ValueError(f"attention: unknown qk_norm '{qk_norm}' (none, whole)")
        self.hidden, self.n_q, self.n_kv, self.head_dim = hidden, n_q, n_kv, head_dim
        self.v_dim = int(v_dim) if v_dim else head_dim
        self.scale, self.softcap = float(scale), float(softcap or 0.0)
        self.window = int(window) if window else None
        self.chunk = int(chunk) if chunk else None
        self.qk_norm, self.eps = qk_norm, float(eps)
        self.position = position
        self.q_dim, self.kv_dim, self.v_cols = n_q * head_dim, n_kv * head_dim, n_kv * self.v_dim
        # the options of the second paragraph above: their own row-wise kernel and the exact attention
        self.rowwise = self.v_dim != head_dim or qk_norm != "none" or self.chunk is not None
        if self.rowwise:
            if self.v_dim > 512:
                raise ValueError(f"attention: v_dim {self.v_dim} is beyond the kernels' limit of 512")
            if position is not None:
                raise ValueError("attention: a rotation together with v_dim, qk_norm or chunk is not built")

    def param_specs(self):
        specs = {"q": ParamSpec((self.q_dim, self.hidden)), "k": ParamSpec((self.kv_dim, self.hidden)),
                 "v": ParamSpec((self.v_cols, self.hidden)), "o": ParamSpec((self.hidden, self.n_q * self.v_dim))}
        if self.qk_norm == "whole":
            specs["q_norm"] = ParamSpec((self.q_dim,), "vector")
            specs["k_norm"] = ParamSpec((self.kv_dim,), "vector")
        return specs

    def bind(self, params):
        # one projection for q, k and v: rows [Wq; Wk; Wv]
        kinds = {params[n].dtype for n in ("q", "k", "v")}
        dt = torch.float32 if (len(kinds) > 1 or torch.float32 in kinds) else next(iter(kinds))
        self.w_qkv = torch.cat([params["q"].to(dt), params["k"].to(dt), params["v"].to(dt)], dim=0).contiguous()
        self.w_o = params["o"]
        self.q_gain = self.k_gain = None
        if self.qk_norm == "whole":
            gd = torch.float32 if params["q_norm"].dtype != params["k_norm"].dtype else params["q_norm"].dtype
            self.q_gain, self.k_gain = params["q_norm"].to(gd).contiguous(), params["k_norm"].to(gd).contiguous()
        self.params = {}

    def cache_spec(self):
        if self.rowwise:
            return KVSpec(self.n_kv, self.head_dim, self.window, v_dim=self.v_dim if self.v_dim != self.head_dim else None,
                          chunk=self.chunk)
        return KVSpec(self.n_kv, self.head_dim, self.window)

    def prepare(self, max_positions, device):
        if self.position is not None:
            self.position.prepare(max_positions, device)

    def forward(self, x: torch.Tensor, ctx, entry, writes_cache: bool = True) -> torch.Tensor:
        """x (tokens, hidden) in the step's element type -> (tokens, hidden) float32, or
        [parts, tokens, hidden] partial sums that the residual kernel adds."""
        k_pages, v_pages, table, ring, page = ctx.kv(entry)
        if self.rowwise:
            return self._forward_rowwise(x, ctx, entry, writes_cache)
        rot = self.position.rotary_dim if self.position is not None else 0
        cos_sin = self.position.table if self.position is not None else None
        kept = (k_pages, v_pages, ctx.cache_rows[entry.group_id]) if writes_cache else (None, None, None)
        if kernels.skinny_ok(x, self.w_qkv) and (cos_sin is None or rot == self.head_dim):
            # a few tokens: the rotation and the write into the cache are the product's epilogue
            qkv = torch.empty((x.shape[0], self.q_dim + 2 * self.kv_dim), dtype=ctx.dtype, device=x.device)
            kernels.skinny_qkv_rope(x, self.w_qkv, qkv, ctx.positions, cos_sin, self.n_q, self.n_kv, self.head_dim,
                                    *kept, page)
        elif kernels.stream_rows(x, self.w_qkv) and (cos_sin is None or rot == self.head_dim):
            # 17 to 128 tokens: the weights stream once through tcgen05, cut along K so that every SM takes
            # part; the kernel that rotates q and k and fills the cache adds the slices on its way
            slices = kernels.gemm_stream_parts(x, self.w_qkv)
            sums = torch.empty((slices, x.shape[0], self.q_dim + 2 * self.kv_dim), dtype=torch.float32, device=x.device)
            kernels.gemm_stream(x, self.w_qkv, sums)
            qkv = torch.empty((x.shape[0], self.q_dim + 2 * self.kv_dim), dtype=ctx.dtype, device=x.device)
            kernels.rope_kv_write_parts(sums, qkv, ctx.positions, cos_sin, self.n_q, self.n_kv, self.head_dim, *kept,
                                        page)
        else:
            qkv = linear(x, self.w_qkv, out_dtype=ctx.dtype)
            kernels.rope_kv_write(qkv, ctx.positions, cos_sin, self.n_q, self.n_kv, self.head_dim, rot, *kept, page)
        q = qkv[:, :self.q_dim]
        out = torch.empty((qkv.shape[0], self.q_dim), dtype=ctx.dtype, device=x.device)
        common = dict(n_kv=self.n_kv, group=self.n_q // self.n_kv, head_dim=self.head_dim, scale=self.scale,
                      cap=self.softcap, window=self.window or 0, batch=ctx.batch, max_q_len=ctx.max_q_len)
        if ctx.mode == "prefill" and writes_cache:
            # the step's own keys and values, still packed: a prompt longer than
            # the window needs keys the ring no longer holds
            k = qkv[:, self.q_dim:self.q_dim + self.kv_dim]
            v = qkv[:, self.q_dim + self.kv_dim:]
            self.attend_packed(q, k, v, out, ctx, common)
        else:
            if ctx.mode == "prefill" and self.window and ctx.max_kv_len > ring:
                raise NotImplementedError("a layer that reads another layer's windowed cache cannot take a "
                                          "prompt longer than the ring in one step")
            self.attend_paged(q, out, ctx, common, k_pages, v_pages, table, ring, page)
        return linear(out, self.w_o, out_dtype=torch.float32, parts_ok=True)

    def _forward_rowwise(self, x, ctx, entry, writes_cache):
        """The path of a layer with a whole-row norm, value heads of their own size or a chunked mask."""
        k_pages, v_pages, table, ring, page = ctx.kv(entry)
        if ctx.mode == "prefill" and not writes_cache:
            raise NotImplementedError("a layer of this kind that reads another layer's cache cannot take a prompt")
        proj = linear(x, self.w_qkv, out_dtype=torch.float32)
        qkv = proj if ctx.dtype == torch.float32 else torch.empty(proj.shape, dtype=ctx.dtype, device=x.device)
        kept = (k_pages, v_pages, ctx.cache_rows[entry.group_id]) if writes_cache else (None, None, None)
        kernels.qkv_norm_write(proj, self.q_dim, self.kv_dim, self.v_cols, self.q_gain, self.k_gain, self.eps,
                               ctx.positions, qkv, self.n_kv, *kept, page)
        q = qkv[:, :self.q_dim]
        out = torch.empty((qkv.shape[0], self.n_q * self.v_dim), dtype=ctx.dtype, device=x.device)
        common = dict(n_kv=self.n_kv, group=self.n_q // self.n_kv, head_dim=self.head_dim, scale=self.scale,
                      cap=self.softcap, window=self.window or 0, batch=ctx.batch, max_q_len=ctx.max_q_len,
                      v_dim=self.v_dim, chunk=self.chunk or 0)
        # bfloat16 with key and value rows of one size runs on the tensor cores; all else on the exact kernel
        tensor = self._tensor_cores(ctx) and self.v_dim == self.head_dim and self.head_dim % 16 == 0
        k, v = qkv[:, self.q_dim:self.q_dim + self.kv_dim], qkv[:, self.q_dim + self.kv_dim:]
        if ctx.mode == "prefill" and tensor:
            kernels.attention_prefill_mma(q, out, ctx.cu_q, k, v, **{n: a for n, a in common.items() if n != "v_dim"})
        elif ctx.mode == "prefill":
            kernels.attention_simt(q, out, ctx.cu_q, ctx.kv_len, k=k, v=v, **common)
        elif tensor and page == 64:
            span = min(self.window or (1 << 30), self.chunk or (1 << 30))
            splits = kernels.decode_splits(ctx.batch, self.n_kv, ctx.max_kv_len, span if span < (1 << 30) else 0,
                                           ragged=getattr(ctx, "ragged", False))
            kernels.attention_decode_mma(q, out, ctx.cu_q, ctx.kv_len, k_pages, v_pages, table, ring=ring, page_size=page,
                                         n_splits=splits, **{n: a for n, a in common.items() if n not in ("v_dim", "max_q_len")})
        else:
            kernels.attention_simt(q, out, ctx.cu_q, ctx.kv_len, k_pages=k_pages, v_pages=v_pages, page_table=table,
                                   ring=ring, page_size=page, **common)
        return linear(out, self.w_o, out_dtype=torch.float32, parts_ok=True)

    # bfloat16 runs on the tensor cores when the sizes allow; everything else, and
    # all of float32, takes the exact CUDA-core kernel
    def _tensor_cores(self, ctx) -> bool:
        return ctx.dtype == torch.bfloat16 and self.head_dim <= 256 and self.n_q // self.n_kv <= 16

    def attend_packed(self, q, k, v, out, ctx, common):
        if self._tensor_cores(ctx) and kernels.attention_prefill_tc_ok(self.head_dim, self.n_q // self.n_kv):
            kernels.attention_prefill_tc(q, out, ctx.cu_q, k, v, **common)         # tcgen05, scores in tensor memory
        elif self._tensor_cores(ctx):
            kernels.attention_prefill_mma(q, out, ctx.cu_q, k, v, **common)
        else:
            kernels.attention_simt(q, out, ctx.cu_q, ctx.kv_len, k=k, v=v, **common)

    def attend_paged(self, q, out, ctx, common, k_pages, v_pages, table, ring, page):
        if self._tensor_cores(ctx) and ctx.mode == "decode" and page == 64:
            args = {k: v for k, v in common.items() if k != "max_q_len"}
            splits = kernels.decode_splits(ctx.batch, self.n_kv, ctx.max_kv_len, self.window or 0,
                                           ragged=getattr(ctx, "ragged", False))
            kernels.attention_decode_mma(q, out, ctx.cu_q, ctx.kv_len, k_pages, v_pages, table, ring=ring,
                                         page_size=page, n_splits=splits, **args)
        else:
            kernels.attention_simt(q, out, ctx.cu_q, ctx.kv_len, k_pages=k_pages, v_pages=v_pages, page_table=table,
                                   ring=ring, page_size=page, **common)


register_part("mixer", "attention", Attention)
