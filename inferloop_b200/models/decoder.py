"""A decoder assembled from a :class:`ModelSpec`: token table, the blocks in their run
order, final norm and output matrix.  It runs whatever the spec lists; the only thing it
knows is the order embedding -> layers -> selected rows -> norm -> logits, which is the
reference's lowering too (crates/model/recipes/src/decoder.rs:93-154).  Logits are
computed only for the rows that are asked for, as the reference copies only the rows it
reads before its output matrix
(crates/backend/cuda-kernels/src/tile/projection/prompt_logits_kernels.rs:15-49).
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional

import torch

from ..config.spec import ModelSpec
from ..csrc import ops
from ..parts import registry
from ..parts.base import BuildContext, CacheNeeds, Workspace
from ..parts.linear import linear
from ..weights.decl import WeightDecl


class DecoderModel:
    def __init__(self, spec: ModelSpec, ctx: BuildContext) -> None:
        self.spec = spec
        self.ctx = ctx
        self.blocks = [registry.build_block(layer, ctx, layer.prefix) for layer in spec.layers]
        self.final_norm = registry.build_norm(
            spec.final_norm, ctx, _strip_weight(spec.final_norm_name), width=spec.hidden_size)
        self.logits_post = (registry.build("logits", spec.logits_post, ctx) if spec.logits_post is not None else None)
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self._weight_bytes = 0

    # ------------------------------------------------------------------ weights
    def declare_weights(self) -> List[WeightDecl]:
        s = self.spec
        out = [WeightDecl(s.embedding_name, (s.vocab_size, s.hidden_size), role="table")]
        for b in self.blocks:
            out += b.declare_weights()
        out += self.final_norm.declare_weights()
        if s.head_name is not None:
            out.append(WeightDecl(s.head_name, (s.vocab_size, s.hidden_size), root=True))
        names = [d.name for d in out]
        if len(set(names)) != len(names):
            dup = sorted({n for n in names if names.count(n) > 1})
            raise ValueError(f"tensor names declared twice: {dup}")
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        s = self.spec
        self.embedding = tensors[s.embedding_name].contiguous()
        for b in self.blocks:
            b.bind(tensors)
        self.final_norm.bind(tensors)
        self.head = self.embedding if s.head_name is None else tensors[s.head_name].contiguous()
        # Every declared tensor is read once by a step, except the token table, of which a step
        # reads one row per token (unless it is also the output matrix).
        self._weight_bytes = sum(tensors[d.name].numel() * tensors[d.name].element_size() for d in self.declare_weights()
                                 if d.name != s.embedding_name or s.head_name is None)

    def cache_needs(self) -> List[CacheNeeds]:
        return [b.cache_needs() for b in self.blocks]

    def weight_bytes(self) -> int:
        """Bytes of every weight one step reads once: the tensors the parts declared, as they
        were bound (the token table is read by row only, unless it is the output matrix too)."""
        return self._weight_bytes

    @property
    def graph_safe(self) -> bool:
        """Whether embedding, final norm, output matrix and the logits map read the batch from
        device memory alone (the blocks answer for themselves)."""
        return self.final_norm.graph_safe and (self.logits_post is None or self.logits_post.graph_safe)

    def scratch_bytes(self, tokens: int, logit_rows: int) -> int:
        """Workspace a step of `tokens` tokens with `logit_rows` wanted rows asks for: the
        residual stream, the largest block's buffers (blocks share them by name), the
        selected rows and their logits."""
        s = self.spec
        size = torch.empty((), dtype=self.ctx.dtype).element_size()
        blocks = max((b.scratch_bytes(tokens) for b in self.blocks), default=0)
        return (tokens * s.hidden_size * 4 + blocks + logit_rows * s.hidden_size * (4 + size)
                + logit_rows * s.vocab_size * 4)

    # ------------------------------------------------------------------ run
    def forward(self, step, caches) -> torch.Tensor:
        """Run the step's tokens through every run-order entry; returns 32-bit logits
        [len(step.logit_rows), vocab] (a workspace buffer, valid until the next step)."""
        hidden = self.forward_embed(step)
        self.forward_entries(hidden, step, caches, 0, len(self.spec.run_order))
        return self.forward_head(hidden, step)

    # The three pieces of `forward`, for a caller that runs (or records) a step in segments.
    def forward_embed(self, step) -> torch.Tensor:
        s, ws = self.spec, self.ctx.workspace
        hidden = ws.buffer("model.hidden", (step.n_tokens, s.hidden_size), torch.float32)
        ops.scope("embedding")
        ops.embed(step.tokens, self.embedding, hidden)
        if s.embedding_scale is not None and s.embedding_scale != 1.0:
            ops.scale_cap_inplace(hidden, float(s.embedding_scale), 0.0)
        return hidden

    def forward_entries(self, hidden: torch.Tensor, step, caches, first: int, last: int) -> None:
        """Run-order entries first .. last - 1."""
        for entry in self.spec.run_order[first:last]:
            self.blocks[entry.layer].forward(hidden, step, caches.layer_cache(entry))

    def forward_head(self, hidden: torch.Tensor, step) -> torch.Tensor:
        s, ws = self.spec, self.ctx.workspace
        ops.scope("head.rows_norm")
        R = step.n_logit_rows
        if R == 0:
            return ws.buffer("model.logits", (0, s.vocab_size), torch.float32)
        rows = ws.buffer("model.rows", (R, s.hidden_size), torch.float32)
        ops.gather_rows(hidden, step.logit_rows, rows)
        normed = ws.buffer("model.rows_normed", (R, s.hidden_size), self.ctx.dtype)
        self.final_norm.forward(rows, normed)
        logits = ws.buffer("model.logits", (R, s.vocab_size), torch.float32)
        ops.scope("head.output_matrix")
        linear(normed, self.head, logits)
        if self.logits_post is not None:
            ops.scope("head.logits_map")
            self.logits_post.forward(logits)
        ops.scope("other")
        return logits


def _strip_weight(name: str) -> str:
    """"norm.weight" -> "norm." (the norm part appends its own tensor name)."""
    return name[: -len("weight")] if name.endswith("weight") else name


def declare_weights(spec: ModelSpec) -> List[WeightDecl]:
    """The tensors a spec needs, without touching a device."""
    ctx = BuildContext(dtype=torch.float32, device=None, workspace=Workspace(None))
    return DecoderModel(spec, ctx).declare_weights()
