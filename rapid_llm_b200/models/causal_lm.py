"""The one model class: a decoder built from a :class:`ModelSpec` and run in its order.

embed -> the layers named by the run order -> final norm over the wanted rows -> output
head, as the reference's skeleton does (``rapid_llm/models/base.py:556-631``), except that
which layer runs when, and whose cache it uses, is read from ``spec.schedule``.
"""

from __future__ import annotations

import torch

from ..config.model_spec import ModelSpec
from ..engine.batch import LayerCache, StepBatch
from ..ops import gemm
from ..parts.base import BLOCKS, EMBEDDINGS, HEADS, NORMS, CacheNeed, StateNeed, StreamAddend, TensorSpec
from ..parts.norm import ADD, PLAIN


class CausalLM:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device | str) -> None:
        spec.validate()
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        context = {"dtype": dtype, "device": self.device}
        self.embedding = EMBEDDINGS.build(spec.embedding, **context)
        self.layers = [
            BLOCKS.get(layer.arrangement)(layer=layer, **context) for layer in spec.layers
        ]
        self.final_norm = NORMS.build(spec.final_norm, **context)
        self.head = HEADS.build(spec.head, **context)
        if hasattr(self.head, "tie_to"):
            self.head.tie_to(self.embedding)
        # a learned row per pass of a looped run of layers, for run orders whose entries open passes
        self._tensor_owner: dict | None = None
        self.pass_offset = None if spec.pass_offset is None else EMBEDDINGS.build(spec.pass_offset, **context)
        if self.device.type == "cuda":
            self._build_kernels()

    def _build_kernels(self) -> None:
        """Compile, side by side, the kernel libraries this model's parts say they launch from (each would
        otherwise be built at its first launch, one after the other)."""
        from concurrent.futures import ThreadPoolExecutor

        from ..ops import build

        names = {"core"}
        for layer in self.layers:
            if hasattr(layer, "uses_libraries"):
                names |= layer.uses_libraries()
        with ThreadPoolExecutor(max_workers=len(names)) as pool:
            list(pool.map(build.build_library, sorted(names)))

    # -- weights ----------------------------------------------------------------- #
    def _owners(self):
        """``(prefix, part)`` for every part that owns checkpoint tensors."""
        yield self.spec.embedding_prefix, self.embedding
        for layer_spec, layer in zip(self.spec.layers, self.layers):
            yield layer_spec.prefix, layer
        yield self.spec.final_norm_prefix, self.final_norm
        yield self.spec.head_prefix, self.head
        if self.pass_offset is not None:
            yield self.spec.pass_offset_prefix, self.pass_offset

    def tensor_specs(self) -> dict[str, TensorSpec]:
        """Every checkpoint tensor by full name, in a fixed order."""
        specs: dict[str, TensorSpec] = {}
        for prefix, part in self._owners():
            for name, spec in part.tensor_specs().items():
                specs[prefix + name] = spec
        return specs

    def load_tensor(self, full_name: str, tensor: torch.Tensor) -> None:
        """Hand a tensor to the part that lists it (prefixes may be empty or begin alike, so a name is looked up
        among the parts' own lists, not matched by its beginning)."""
        if self._tensor_owner is None:
            self._tensor_owner = {prefix + name: (part, name) for prefix, part in self._owners()
                                  for name in part.tensor_specs()}
        if full_name not in self._tensor_owner:
            raise KeyError(full_name)
        part, name = self._tensor_owner[full_name]
        part.load_tensor(name, tensor)

    def finalize(self, loaded: set[str]) -> None:
        for prefix, part in self._owners():
            part.finalize({name[len(prefix):] for name in loaded if name.startswith(prefix)})

    def parameter_bytes(self) -> int:
        return sum(part.parameter_bytes() for _, part in self._owners())

    def activation_bytes_per_token(self) -> int:
        """Bytes of activation buffers one token of a step needs: the widest layer's buffers (the layers
        share them), the embedding's output and the float32 residual stream."""
        element = torch.empty((), dtype=self.dtype).element_size()
        widest = max(layer.workspace_elements_per_token() for layer in self.layers)
        return (widest + 2 * self.spec.hidden_size) * element + 4 * self.spec.hidden_size

    # -- what the cache manager has to provide -------------------------------------- #
    def cache_needs(self) -> list[CacheNeed | None]:
        """One entry per position of the run order; ``None`` = no pages of its own."""
        needs: list[CacheNeed | None] = []
        for entry in self.spec.schedule:
            need = self.layers[entry.layer].cache_need()
            needs.append(None if entry.cache_from is not None else need)
        return needs

    def state_needs(self) -> list[StateNeed | None]:
        """One entry per position of the run order, and one more behind them if the embedding keeps a state
        per request (what :meth:`forward` then expects as the last of ``caches``)."""
        needs = [self.layers[entry.layer].state_need() for entry in self.spec.schedule]
        if hasattr(self.embedding, "state_need"):
            needs.append(self.embedding.state_need())
        return needs

    def step_planners(self) -> list:
        """The distinct host-side planners of the layers (one per key)."""
        planners: dict[tuple, object] = {}
        for layer in self.layers:
            for planner in layer.step_planners():
                planners.setdefault(planner.key, planner)
        return list(planners.values())

    # -- forward ------------------------------------------------------------------- #
    def forward(self, batch: StepBatch, caches: list[LayerCache]) -> torch.Tensor:
        """Logits ``[R, vocab]`` at ``batch.logit_rows``; runs only the tokens of the step."""
        batch.defer_products = True      # the queue is run below, before anything but a kernel reads a result
        own = (caches[len(self.spec.schedule)],) if hasattr(self.embedding, "state_need") else ()
        if getattr(self.embedding, "opens_stream", False):
            x, residual = self.embedding.forward_stream(batch, *own)      # the float32 stream starts at the embedding
            embedded = x
        else:
            x = embedded = self.embedding.forward(batch, *own)
            residual = None
        schedule = self.spec.schedule
        for position, entry in enumerate(schedule):
            # the norm that the next layer starts with may ride on this layer's last product, unless
            # something joins the stream in between
            after = None
            if position + 1 < len(schedule) and schedule[position + 1].pass_index is None:
                after = self.layers[schedule[position + 1].layer].leading_norm()
            if entry.pass_index is None:
                x, residual = self.layers[entry.layer].forward(x, residual, batch, caches[position], then_norm=after)
            else:
                addend = StreamAddend(rows=embedded if entry.add_embedding else None,
                                      vector=self.pass_offset.row(entry.pass_index))
                x, residual = self.layers[entry.layer].forward(x, residual, batch, caches[position], then_norm=after,
                                                               addend=addend)
        if batch.num_logit_rows == 0 or not self.final_norm.reads_deferred:
            gemm.flush()
        if batch.num_logit_rows == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=self.dtype, device=self.device)
        if residual is not None and self.layers[schedule[-1].layer].stream_in_residual:
            hidden = self.final_norm.of_stream(residual, batch, row_index=batch.logit_rows, name="final_normed")
        elif residual is None:
            hidden = self.final_norm.forward(
                x, None, batch, mode=PLAIN, write_residual=False,
                row_index=batch.logit_rows, name="final_normed",
            )
        else:
            hidden = self.final_norm.forward(
                x, residual, batch, mode=ADD, write_residual=False,
                row_index=batch.logit_rows, name="final_normed",
            )
        logits = self.head.forward(hidden, batch)
        gemm.flush()
        return logits
