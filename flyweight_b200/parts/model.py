"""A decoder model put together from a ``ModelSpec``: embedding, the layers in the
order its schedule names them, a final norm and the head.

LFM2 takes embedding rows without scaling (native/src/v2_runtime.cpp:27951-27956) and has
no soft-cap on its logits; ``ModelSpec.embedding_scale`` and ``logit_softcap`` are there for
architectures that have them.  The
head is the embedding table when the spec names none (native/src/v2_runtime.cpp:4190-4191);
the final norm and the head run only on the rows whose logits were asked for.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Mapping, Optional

import torch

from ..config.spec import ModelSpec
from ..kernels import ops
from ..weights.loader import TensorDecl, bind as bind_tensors
from .base import Arrangement, PagedKV, Precision, build_arrangement, build_embedding, build_norm


class DecoderModel:
    def __init__(self, spec: ModelSpec, precision: Precision, device):
        spec.validate()
        self.spec = spec
        self.precision = precision
        self.device = device
        self.layers: List[Arrangement] = [build_arrangement(layer) for layer in spec.layers]
        self.final_norm = build_norm(spec.final_norm)
        # None: rows of the token table times ``embedding_scale``; else a part that builds the first
        # layer's input from the table and whatever else it declares
        self.embedder = build_embedding(spec.embedding) if spec.embedding is not None else None
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        for position, entry in enumerate(spec.schedule):
            layer = self.layers[entry.layer]
            own = layer.state_spec()
            own = own if isinstance(own, tuple) else (own,)
            if entry.cache_of is not None and any(isinstance(s, PagedKV) for s in own):
                raise ValueError(
                    f"schedule position {position} reads the cache of position {entry.cache_of}, "
                    f"but its mixer ({layer.stateful_part().kind}) keeps a cache of its own")

    # ------------------------------------------------------------------ weights
    def declare(self) -> Dict[str, TensorDecl]:
        spec = self.spec
        out = {spec.embedding_tensor: TensorDecl((spec.vocab_size, spec.hidden_size), "embedding")}
        if spec.head_tensor is not None:
            out[spec.head_tensor] = TensorDecl((spec.vocab_size, spec.hidden_size))
        out.update(self.final_norm.declare())
        if self.embedder is not None:
            out.update(self.embedder.declare())
        for layer in self.layers:
            for part in layer.parts():
                out.update(part.declare())
        return out

    def load(self, stored: Mapping[str, torch.Tensor]) -> None:
        """Bind checkpoint tensors by name; one error lists everything that does not fit."""
        tensors = bind_tensors(self.declare(), stored, self.spec.unused_tensors)
        get: Callable[[str], torch.Tensor] = tensors.__getitem__
        spec, precision, device = self.spec, self.precision, self.device
        self.embedding = precision.matrix(get(spec.embedding_tensor), device)
        self.head = (self.embedding if spec.head_tensor is None
                     else precision.matrix(get(spec.head_tensor), device))
        self.final_norm.bind(get, precision, device)
        if self.embedder is not None:
            self.embedder.bind(get, precision, device)
        for layer in self.layers:
            for part in layer.parts():
                part.bind(get, precision, device)

    @property
    def graph_safe(self) -> bool:
        """Every part only launches kernels over the step's device buffers."""
        return all(part.graph_safe for layer in self.layers for part in layer.parts()) \
            and self.final_norm.graph_safe and (self.embedder is None or self.embedder.graph_safe)

    def prepare(self, max_positions: int) -> None:
        for layer in self.layers:
            layer.prepare(max_positions, self.device)

    def state_specs(self) -> list:
        """What each schedule position keeps in the cache manager (a position that reads another's
        pages keeps only the fixed-size state of its own parts); one more entry, behind the
        schedule, for the embedding part when it keeps something."""
        specs = [self.layers[entry.layer].state_spec() for entry in self.spec.schedule]
        if self.embedder is not None and self.embedder.state_spec() is not None:
            specs.append(self.embedder.state_spec())
        return specs

    def cache_sources(self) -> list:
        """For each schedule position the earlier position whose pages it reads, or None."""
        return [entry.cache_of for entry in self.spec.schedule]

    def weight_bytes(self, with_embedding_rows: int = 0, tokens: Optional[int] = None) -> int:
        """Bytes of weights one step reads: every scheduled layer once, the final norm, the
        head, and ``with_embedding_rows`` rows of the embedding table.  ``tokens``: the step's token
        count, for parts that touch only the weights their tokens choose (routed experts)."""
        total = self.final_norm.weight_bytes()
        total += self.head.numel() * self.head.element_size()
        total += with_embedding_rows * self.spec.hidden_size * self.embedding.element_size()
        for entry in self.spec.schedule:
            total += sum(part.weight_bytes() if tokens is None else part.active_weight_bytes(tokens)
                         for part in self.layers[entry.layer].parts())
        return total

    def flops_per_token(self, with_head: bool = False) -> float:
        """Operations of the matrix products one token passes through (every scheduled layer
        once; the head only if asked: it runs on the wanted rows alone)."""
        total = sum(part.flops_per_token() for entry in self.spec.schedule
                    for part in self.layers[entry.layer].parts())
        if with_head:
            total += 2.0 * self.spec.vocab_size * self.spec.hidden_size
        return total

    def context_flops(self, n_tokens: int) -> float:
        """Operations that grow with the context, for one causal prompt of ``n_tokens``."""
        return sum(part.context_flops(n_tokens) for entry in self.spec.schedule
                   for part in self.layers[entry.layer].parts())

    def parameter_count(self) -> int:
        return sum(int(torch.tensor(decl.shape).prod()) for decl in self.declare().values())

    # ------------------------------------------------------------------ one step
    def forward(self, ctx, caches) -> torch.Tensor:
        """Logits [R][V] fp32 at ``ctx.batch.logit_rows`` (an empty tensor if R == 0).
        ``caches[i]`` is the ``LayerCache`` of schedule position i."""
        batch = ctx.batch
        if self.embedder is None:
            x = ops.embed(self.embedding, batch.token_ids, ctx.bad_token_flag, self.spec.embedding_scale)
        else:
            own = len(self.spec.schedule)
            x = self.embedder.forward(ctx, self.embedding, caches[own] if len(caches) > own else None)
        pending = None
        # a schedule that feeds the embedding's output to later executions keeps a copy of it
        first = x.clone() if any(entry.add_embedding for entry in self.spec.schedule) else None
        for position, entry in enumerate(self.spec.schedule):
            if entry.add_embedding:
                if pending is not None:
                    ops.add_(x, pending)
                    pending = None
                ops.add_(x, first)
            # a position that reads another's pages finds them in its own entry (the manager puts
            # them there), beside the fixed-size state that is its own
            x, pending = self.layers[entry.layer].forward(ctx, x, pending, caches[position])
        if batch.n_logit_rows == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=x.device)
        n = self.final_norm.defer(ctx, x, rows=batch.logit_rows) if pending is None else None
        if n is None:
            n = self.final_norm.forward(ctx, x, delta=pending, rows=batch.logit_rows)
        logits = ops.linear(n, self.head, torch.float32)
        if self.spec.logit_scale != 1.0:
            ops.scale_(logits, self.spec.logit_scale)
        if self.spec.logit_softcap > 0:
            ops.softcap_(logits, self.spec.logit_softcap)
        return logits
