"""Grouped-query causal attention over the paged cache, with optional per-head q/k
RMSNorm, optional biases, optional window, and a position encoding chosen by spec.

Order of operations as in the reference's decoder recipe
(crates/model/recipes/src/decoder.rs:229-364): q/k/v projections; per-head RMSNorm of q
and k over head_dim with a weight [head_dim] shared by all heads (:278-293), before the
rotation (:315-335); cache append (:336-342); attention with head h reading kv head
h / (nq / nkv) and scale 1/sqrt(head_dim)
(crates/testing/cpu/reference-ops/src/kernels.rs:251-297); output projection added to the
residual (:358-363).  Biases, where the spec asks for them, are added in 32-bit right
after each projection.

The three projection matrices are concatenated at load into one [(nq + 2 nkv) d, H]
matrix so one GEMM produces q|k|v.
"""
from __future__ import annotations

import math
from typing import List, Mapping, Optional

import torch

from ..csrc import ops
from ..weights.decl import WeightDecl
from . import registry
from .base import CacheNeeds, Mixer, PagedKVNeed
from .linear import linear


class GQAttention(Mixer):
    @property
    def graph_safe(self) -> bool:
        """The kernels read the batch from device memory; the position encoding answers for itself."""
        return bool(self.position.graph_safe)

    def __init__(self, spec, ctx, prefix: str = "") -> None:
        super().__init__(spec, ctx, prefix)
        self.hidden = int(spec["hidden_size"])
        self.nq = int(spec["num_heads"])
        self.nkv = int(spec["num_kv_heads"])
        self.d = int(spec["head_dim"])
        if self.nq % self.nkv:
            raise ValueError(f"{self.nq} query heads are not a multiple of {self.nkv} kv heads")
        self.qk_norm = bool(spec.get("qk_norm", False))
        self.qk_norm_eps = float(spec.get("qk_norm_eps", 1e-6))
        self.bias = bool(spec.get("bias", False))
        self.window = spec.get("window")
        self.scale = 1.0 / math.sqrt(self.d)
        # split-KV decode cuts the keys at multiples of this, fixed per model so that the
        # cut never depends on the batch
        self.decode_chunk = ops.decode_chunk_for(int(spec.get("max_positions", 4096)))
        self.position = registry.build("position", spec["position"], ctx)
        self.rotary_dim = int(spec["position"].get("rotary_dim", 0))
        p = prefix
        self.names = {k: p + v for k, v in {
            "q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
            "qb": "q_proj.bias", "kb": "k_proj.bias", "vb": "v_proj.bias", "ob": "o_proj.bias",
            "qn": "q_norm.weight", "kn": "k_norm.weight"}.items()}
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = self.q_norm = self.k_norm = None

    # ------------------------------------------------------------------ weights
    def declare_weights(self) -> List[WeightDecl]:
        n, d, H = self.names, self.d, self.hidden
        out = [WeightDecl(n["q"], (self.nq * d, H)), WeightDecl(n["k"], (self.nkv * d, H)),
               WeightDecl(n["v"], (self.nkv * d, H)), WeightDecl(n["o"], (H, self.nq * d))]
        if self.bias:
            out += [WeightDecl(n["qb"], (self.nq * d,), "vector", "bias"),
                    WeightDecl(n["kb"], (self.nkv * d,), "vector", "bias"),
                    WeightDecl(n["vb"], (self.nkv * d,), "vector", "bias"),
                    WeightDecl(n["ob"], (H,), "vector", "bias")]
        if self.qk_norm:
            out += [WeightDecl(n["qn"], (d,), "vector", "norm"),
                    WeightDecl(n["kn"], (d,), "vector", "norm")]
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        self.w_qkv = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]], dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        if self.bias:
            self.b_qkv = torch.cat([tensors[n["qb"]], tensors[n["kb"]], tensors[n["vb"]]]).contiguous()
            self.b_o = tensors[n["ob"]].contiguous()
        if self.qk_norm:
            self.q_norm = tensors[n["qn"]].contiguous()
            self.k_norm = tensors[n["kn"]].contiguous()

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(paged=PagedKVNeed(self.nkv, self.d, self.window))

    def scratch_bytes(self, tokens: int) -> int:
        size = torch.empty((), dtype=self.ctx.dtype).element_size()
        width = (self.nq + 2 * self.nkv) * self.d
        return tokens * ((width + 2 * self.nq * self.d) * size + self.rotary_dim * 4)

    # ------------------------------------------------------------------ run
    def forward(self, x: torch.Tensor, residual: torch.Tensor, step, cache) -> None:
        T = x.shape[0]
        ws, dt = self.ctx.workspace, self.ctx.dtype
        width = (self.nq + 2 * self.nkv) * self.d
        qkv = ws.buffer("attn.qkv", (T, width), dt)
        ops.scope("attention.qkv_projection")
        linear(x, self.w_qkv, qkv, self.b_qkv)
        table = step.block_tables[cache.group]
        ops.scope("attention.position_table")
        rope = self.position.table(step)
        if (step.decode_only and cache.k is not None and ops.attention_decode_fused_supported(
                dt, cache.k.dtype, self.nq, self.nkv, self.d, cache.page_size, self.rotary_dim, rope is not None)):
            # one token per sequence: norm, rotation and the cache write of the new key and
            # value happen inside the attention kernel
            o = ws.buffer("attn.o", (T, self.nq * self.d), dt)
            ops.scope("attention.decode (q/k norm, rotation, cache write inside)")
            ops.attention_decode_fused(qkv, o, self.q_norm, self.k_norm, self.qk_norm_eps, rope, cache.k, cache.v,
                                       cache.writable, step.positions, step.cu_q, table, self.window or 0, self.scale,
                                       step.n_seqs, self.nq, self.nkv, self.d,
                                       long_context=step.max_kv_len >= ops.DECODE_LONG_CONTEXT)
            ops.scope("attention.o_projection")
            linear(o, self.w_o, residual, self.b_o, accumulate=True)
            return
        q = ws.buffer("attn.q", (T, self.nq * self.d), dt)
        ops.scope("attention.qk_norm_rotation_cache_write")
        ops.qk_norm_rope_cache(
            qkv, q, self.q_norm, self.k_norm, self.qk_norm_eps, rope,
            self.rotary_dim, step.positions, step.seq_of_token, table, cache.page_size,
            cache.k if cache.writable else None, cache.v if cache.writable else None,
            self.nq, self.nkv, self.d)
        o = ws.buffer("attn.o", (T, self.nq * self.d), dt)
        ops.scope("attention.attention")
        ops.attention(q, o, cache.k, cache.v, step, table, self.window or 0, self.scale,
                      self.nq, self.nkv, self.d, workspace=ws, decode_chunk=self.decode_chunk)
        ops.scope("attention.o_projection")
        linear(o, self.w_o, residual, self.b_o, accumulate=True)


registry.register("mixer", "gqa_attention", GQAttention)
