"""Token embedding and output head.

``x_t = E[id_t]`` without scaling (``rapid_llm/modules/vocab_parallel.py:101-103``); the
head is ``logits = h @ W^T`` without bias over the wanted rows only
(``rapid_llm/models/base.py:625-631``).  With tied embeddings the head has no tensor of its
own and uses the embedding's; a shipped ``lm_head.weight`` wins over the tie
(``rapid_llm/models/weights.py:165-172,197-214``).
"""

from __future__ import annotations

import torch

from ..ops import gemm, kernels
from .base import EMBEDDINGS, HEADS, MATRIX, VECTOR, Part, StateNeed, TensorSpec


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Part):
    """``scale`` multiplies every row (float32 product).  With ``opens_stream`` the float32 products are also the
    residual stream's first value (:meth:`forward_stream`), for models whose layers add to the stream without a
    norm in front: the stream then never passes through the engine's 16-bit dtype."""

    def __init__(self, *, vocab_size: int, hidden_size: int, dtype, device, name: str = "weight",
                 scale: float = 1.0, opens_stream: bool = False) -> None:
        super().__init__(dtype=dtype, device=device)
        self.vocab, self.hidden = int(vocab_size), int(hidden_size)
        self.name = name          # the tensor's name after the part's prefix (may be empty)
        self.scale, self.opens_stream = float(scale), bool(opens_stream)
        self.weight = self.new_storage((self.vocab, self.hidden), MATRIX)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.vocab, self.hidden))}

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        if name != self.name:
            raise KeyError(name)
        self.weight.copy_(tensor)

    def parameter_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, batch) -> torch.Tensor:
        out = batch.workspace.get("embedded", batch.num_tokens, self.hidden, self.dtype)
        return kernels.embedding(out, self.weight, batch.token_ids, batch.fault, batch.feedback, scale=self.scale)

    def forward_stream(self, batch) -> tuple[torch.Tensor, torch.Tensor]:
        """``(rows in the engine's dtype, the float32 residual stream they open)``."""
        out = batch.workspace.get("embedded", batch.num_tokens, self.hidden, self.dtype)
        stream = batch.workspace.get("residual", batch.num_tokens, self.hidden, torch.float32)
        kernels.embedding(out, self.weight, batch.token_ids, batch.fault, batch.feedback, scale=self.scale, stream=stream)
        return out, stream


@EMBEDDINGS.register("summed_embedding")
class SummedEmbedding(TokenEmbedding):
    """A token's row plus a row for the pair (previous token, token) plus a learned row for the position:
    ``x_t = E[id_t] + B[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets] + P[p_t]``, a float32 sum that opens the
    residual stream.  ``B`` has ``buckets + 1`` rows; a request's first token, which has no previous one, takes the
    last.  The request's latest token id is its state (one int32 per slot), so that a portion of a prompt or a single
    decoded token finds the id before its first row."""

    opens_stream = True

    def __init__(self, *, vocab_size: int, hidden_size: int, pair_buckets: int, pair_mul_prev: int, pair_mul_cur: int,
                 max_positions: int, dtype, device, name: str = "weight", pair_name: str = "pair",
                 position_name: str = "positions") -> None:
        super().__init__(vocab_size=vocab_size, hidden_size=hidden_size, dtype=dtype, device=device, name=name,
                         opens_stream=True)
        self.buckets, self.mul_prev, self.mul_cur = int(pair_buckets), int(pair_mul_prev), int(pair_mul_cur)
        self.max_positions = int(max_positions)
        if self.buckets < 1 or self.max_positions < 1:
            raise ValueError("a summed embedding needs at least one pair bucket and one position")
        self.pair_name, self.position_name = pair_name, position_name
        self.pair = self.new_storage((self.buckets + 1, self.hidden), MATRIX)
        self.positions = self.new_storage((self.max_positions, self.hidden), MATRIX)

    def state_need(self) -> StateNeed:
        return StateNeed((1,), torch.int32)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.vocab, self.hidden)),
                self.pair_name: TensorSpec((self.buckets + 1, self.hidden)),
                self.position_name: TensorSpec((self.max_positions, self.hidden))}

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        if name == self.pair_name:
            self.pair.copy_(tensor)
        elif name == self.position_name:
            self.positions.copy_(tensor)
        else:
            super().load_tensor(name, tensor)

    def parameter_bytes(self) -> int:
        return (self.weight.numel() + self.pair.numel() + self.positions.numel()) * self.weight.element_size()

    def forward(self, batch, cache=None) -> torch.Tensor:
        return self.forward_stream(batch, cache)[0]

    def forward_stream(self, batch, cache=None) -> tuple[torch.Tensor, torch.Tensor]:
        if cache is None or cache.state is None:
            raise ValueError("the engine did not give this embedding the state row it asked for")
        out = batch.workspace.get("embedded", batch.num_tokens, self.hidden, self.dtype)
        stream = batch.workspace.get("residual", batch.num_tokens, self.hidden, torch.float32)
        kernels.embedding_sum(out, stream, self.weight, self.pair, self.positions, batch, cache.state,
                              mul_prev=self.mul_prev, mul_cur=self.mul_cur)
        return out, stream


@EMBEDDINGS.register("pass_offset")
class PassOffset(Part):
    """A learned row per pass over a looped run of layers, ``[passes, hidden]``: row ``t`` joins the residual
    stream (a float32 sum) right before the first layer of pass ``t``; kept in float32."""

    def __init__(self, *, passes: int, hidden_size: int, dtype, device, name: str = "step") -> None:
        super().__init__(dtype=dtype, device=device)
        self.passes, self.hidden, self.name = int(passes), int(hidden_size), name
        self.weight = self.new_storage((self.passes, self.hidden), VECTOR)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.passes, self.hidden), VECTOR)}

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        if name != self.name:
            raise KeyError(name)
        self.weight.copy_(tensor.to(torch.float32))

    def parameter_bytes(self) -> int:
        return self.weight.numel() * 4

    def row(self, index: int) -> torch.Tensor:
        return self.weight[index]


@HEADS.register("lm_head")
class LMHead(Part):
    def __init__(self, *, vocab_size: int, hidden_size: int, tied: bool, dtype, device, name: str = "weight") -> None:
        super().__init__(dtype=dtype, device=device)
        self.vocab, self.hidden, self.tied = int(vocab_size), int(hidden_size), bool(tied)
        self.name = name          # the tensor's name after the part's prefix (may be empty)
        self.weight: torch.Tensor | None = None
        self._embedding: TokenEmbedding | None = None

    def tie_to(self, embedding: TokenEmbedding) -> None:
        self._embedding = embedding

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.vocab, self.hidden), optional=self.tied)}

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        if name != self.name:
            raise KeyError(name)
        if self.weight is None:
            self.weight = self.new_storage((self.vocab, self.hidden), MATRIX)
        self.weight.copy_(tensor)

    def finalize(self, loaded: set[str]) -> None:
        if self.name not in loaded:
            if not self.tied or self._embedding is None:
                raise ValueError("the output head has no weight and is not tied to the embedding")
            self.weight = self._embedding.weight  # one tensor, not a copy

    def parameter_bytes(self) -> int:
        if self.weight is None or (self._embedding is not None and self.weight is self._embedding.weight):
            return 0
        return self.weight.numel() * self.weight.element_size()

    def forward(self, hidden_rows: torch.Tensor, batch) -> torch.Tensor:
        out = batch.workspace.get("logits", hidden_rows.shape[0], self.vocab, hidden_rows.dtype, min_rows=64)
        return gemm.linear(hidden_rows, self.weight, out, batch.fault)
