"""The generic decoder: embedding, blocks in plan order, final norm, head.

Built from a ``ModelSpec`` through the part registries; it holds no architecture-specific
code.  The order of the reference's forward pass (cleanroom-transformer/src/cpu_backend.c:218-263):
embed, then per layer norm -> mixer -> residual, norm -> feed-forward -> residual, then the
final norm and the head only at the positions whose logits are wanted (the reference reads
out the last position only, cpu_backend.c:253-259).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..config.spec import ModelSpec
from ..parts.base import BLOCKS, EMBEDDINGS, HEADS, NORMS, BuildContext, CacheNeed, ParamSpec, StateNeed


class _NullOps:
    """Stands in for the kernel library where a model is only described, not run."""

    def __getattr__(self, name):
        raise RuntimeError("this model was built without kernels (description only)")


def describe_context() -> BuildContext:
    return BuildContext(device=torch.device("cpu"), dtype=torch.float32, ops=_NullOps(), workspace=None,
                        max_step_tokens=1)


class DecoderModel:
    def __init__(self, spec: ModelSpec, ctx: BuildContext):
        spec.validate()
        self.spec = spec
        self.ctx = ctx
        self.embedding = EMBEDDINGS.build(spec.embedding, ctx)
        self.blocks = [BLOCKS.get(ls.block)(ls, ctx) for ls in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm, ctx)
        self.head = HEADS.build(spec.head, ctx)
        self.prefix = spec.weight_prefixes[-1]
        self.graph_safe = (all(getattr(part, "graph_safe", True) for _, part in self.named_parts())
                           and all(getattr(b, "graph_safe", True) for b in self.blocks))

    # ------------------------------------------------------------------ weights
    def named_parts(self) -> List[Tuple[str, object]]:
        """(prefix below the decoder's prefix, part) of every part that may own weights."""
        out: List[Tuple[str, object]] = [(self.spec.embedding_prefix, self.embedding)]
        for ls, block in zip(self.spec.layers, self.blocks):
            for sub, part in block.named_parts():
                out.append((ls.prefix + sub, part))
        out.append((self.spec.final_norm_prefix, self.final_norm))
        out.append((self.spec.head_prefix, self.head))
        return out

    def weight_table(self, prefix: Optional[str] = None) -> Dict[str, ParamSpec]:
        prefix = self.prefix if prefix is None else prefix
        table: Dict[str, ParamSpec] = {}
        for sub, part in self.named_parts():
            for p in part.params():
                full = (sub + p.name) if p.absolute else (prefix + sub + p.name)
                if full in table:
                    raise ValueError(f"weights: two parts name the tensor {full}")
                table[full] = p
        return table

    def bind(self, tensors: Dict[str, torch.Tensor], prefix: Optional[str] = None) -> None:
        prefix = self.prefix if prefix is None else prefix
        for sub, part in self.named_parts():
            local = {}
            for p in part.params():
                full = (sub + p.name) if p.absolute else (prefix + sub + p.name)
                if full in tensors:
                    local[p.name] = tensors[full]
            part.bind(local)
        if getattr(self.head, "tied", False):
            stored = self.head.tie(self.embedding.weight)
            if stored is not None and stored is not self.embedding.weight and hasattr(self.embedding, "share"):
                self.embedding.share(stored)       # one copy of the table for both

    def first_weight_name(self) -> str:
        return self.spec.embedding_prefix + self.embedding.params()[0].name

    # ------------------------------------------------------------------ cache needs
    def cache_needs(self) -> Dict[int, CacheNeed]:
        out = {}
        for i, e in enumerate(self.spec.plan):
            need = self.blocks[e.layer].cache_need()
            if need is not None and e.cache_of is None:
                out[i] = need
        return out

    def state_needs(self) -> Dict[int, StateNeed]:
        out = {}
        for i, e in enumerate(self.spec.plan):
            need = self.blocks[e.layer].state_need()
            if need is not None:
                out[i] = need
        return out

    # ------------------------------------------------------------------ accounting
    def step_weight_bytes(self) -> int:
        """Bytes of weights one decode step reads: every plan entry's matrices once, the
        norms, and the head (the embedding table is only gathered from)."""
        total = 0
        for e in self.spec.plan:
            b = self.blocks[e.layer]
            total += sum(p.weight_bytes() for _, p in b.named_parts())
        total += self.final_norm.weight_bytes() + self.head.weight_bytes()
        return total

    def num_parameters(self) -> int:
        n = 0
        for p in self.weight_table().values():
            if p.optional:
                continue
            c = 1
            for s in p.shape:
                c *= s
            n += c
        return n

    # ------------------------------------------------------------------ forward
    def forward(self, step, cache) -> Optional[torch.Tensor]:
        """Runs the step's tokens through the decoder; returns ``[wanted, vocab]`` 32-bit
        logits (None when nothing is wanted)."""
        ws, cap, T = self.ctx.workspace, self.ctx.max_step_tokens, step.num_tokens
        H, V = self.spec.hidden_size, self.spec.vocab_size
        x = ws.buffer("model.x", (cap, H), torch.float32)[:T]
        self.embedding.forward(step.tokens, x)
        # Norms at the seam between two blocks may be folded into the products around them: a block
        # that can says what it needs (fold_request), the block in front prepares it and hands on
        # what it prepared.
        plan, prepared = self.spec.plan, None
        for i, e in enumerate(plan):
            owner = i if e.cache_of is None else e.cache_of
            block = self.blocks[e.layer]
            args = (x, step, cache.view(owner), cache.state_view(i), e.cache_of is None)
            if getattr(block, "folds_norms", False):
                nxt = self.blocks[plan[i + 1].layer] if i + 1 < len(plan) else None
                request = nxt.fold_request(step) if nxt is not None and getattr(nxt, "folds_norms", False) else None
                prepared = block.forward(*args, prepared=prepared, prepare_next=request)
            else:
                block.forward(*args)
                prepared = None
        n = step.num_wanted
        if n == 0:
            return None
        hn = ws.buffer("model.head_in" + step.tag, (n, H), self.ctx.dtype)
        self.final_norm.forward(x, hn, rows=step.want_rows)
        logits = ws.buffer("model.logits" + step.tag, (n, V), torch.float32)
        self.head.forward(hn, logits)
        return logits


def weight_table(spec: ModelSpec, prefix: Optional[str] = None) -> Dict[str, ParamSpec]:
    """The weight table of ``spec`` without building anything on a device."""
    return DecoderModel(spec, describe_context()).weight_table(prefix)
