"""Routed feed-forward: every token runs a few of many small gated feed-forwards, chosen by a router.

``z = W_r x`` in float32, ``s = sigmoid(z)``; a token's ``top_k`` experts are those with the largest ``s``
and their weights are those ``s`` (not renormalised).  With ``scale_input`` the weight multiplies what the
expert reads, ``y = sum_e Expert_e(s_e x)``, with ``Expert(h) = down(silu(gate h) * (up h))``; since gate and
up are linear, the kernels multiply the two products by ``s_e`` in float32 instead of rounding ``s_e x``.
A shared expert of the same form (a :class:`~rapid_llm_b200.parts.mlp.SwiGLU` under ``shared.``) may run for
every token; with ``shared_gate`` its result is multiplied by ``sigmoid(w_sg . x)``, one number per token.

Two more options: ``router_bias`` adds a learned number per expert to ``z`` before the choice, and
``weighting="softmax_chosen"`` makes the weights the softmax over the chosen ``z`` alone.  Without ``scale_input``
the weight multiplies the expert's result instead, ``y = sum_e w_e Expert_e(x)``, in the float32 sum over a
token's choices.

``weighting="softmax_all"`` is a third router: ``s = softmax(z)`` over all router rows; the choice is made on
``s + correction`` (a learned number per row, tensor ``correction``) and only among the rows of the ``group_keep``
best of ``num_groups`` equal groups of neighbouring rows (a group ranks by its largest corrected score); the weights
are the chosen rows' ``s`` divided by their sum.  ``identity_experts`` appends that many router rows without tensors:
an identity expert's result is its input, so a token that chooses one gets ``weight * x`` from it (the rows take part
in the softmax and in the groups like any other).  ``expert_limit`` makes the experts clamped units,
``down(g' * sigmoid(expert_alpha * g') * (u' + 1))`` with ``g' = min(gate x, limit)``, ``u' = clamp(up x, +-limit)``.

The step's (token, expert) pairs are grouped by expert on the device (no host round trip, so a decode
step is captured into a graph like any other), the two products run over the groups
(``ops.kernels.grouped_linear``), and a last kernel sums a token's experts in the order of its choices.
Expert weights are stacked: ``[E, 2 F, H]`` (gate rows, then up rows) and ``[E, H, F]``.
"""

from __future__ import annotations

import torch

from ..ops import kernels
from .base import FEED_FORWARDS, MATRIX, VECTOR, FeedForward, TensorSpec
from .mlp import SwiGLU


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, *, hidden_size: int, num_experts: int, top_k: int, expert_size: int,
                 shared_size: int | None = None, shared_gate: bool = False, scale_input: bool = True,
                 expert_prefix: str = "e", router_name: str = "router", shared_prefix: str = "shared.",
                 shared_gate_name: str = "sg", gate_name: str = "gate", up_name: str = "up", down_name: str = "down",
                 router_bias: bool = False, router_bias_name: str = "router.b", weighting: str = "sigmoid",
                 correction_name: str = "correction", num_groups: int = 1, group_keep: int = 1,
                 identity_experts: int = 0, expert_limit: float | None = None, expert_alpha: float = 1.702,
                 dtype, device) -> None:
        super().__init__(dtype=dtype, device=device)
        self.hidden, self.experts, self.top, self.inter = int(hidden_size), int(num_experts), int(top_k), int(expert_size)
        if not 1 <= self.top <= self.experts + int(identity_experts):
            raise ValueError(f"top_k ({top_k}) must lie between 1 and the number of experts ({num_experts})")
        if shared_gate and not shared_size:
            raise ValueError("a shared gate needs a shared expert")
        if weighting not in ("sigmoid", "softmax_chosen", "softmax_all"):
            raise ValueError(f"unknown weighting {weighting!r}: 'sigmoid', 'softmax_chosen' or 'softmax_all'")
        self.scale_input, self.softmax_chosen = bool(scale_input), weighting == "softmax_chosen"
        self.softmax_all = weighting == "softmax_all"
        self.identity, self.groups, self.keep = int(identity_experts), int(num_groups), int(group_keep)
        self.rows = self.experts + self.identity              # router rows a token chooses among
        if not self.softmax_all and (self.identity or self.groups != 1):
            raise ValueError("identity experts and groups belong to weighting 'softmax_all'")
        if self.softmax_all:
            if self.scale_input or router_bias:
                raise ValueError("weighting 'softmax_all' weighs the experts' results and has no bias on the logits")
            if self.identity < 0 or self.groups < 1 or self.rows % self.groups or not 1 <= self.keep <= self.groups:
                raise ValueError(f"{self.groups} groups must divide the {self.rows} router rows, and 1 <= keep <= groups")
            if not 1 <= self.top <= self.keep * (self.rows // self.groups):
                raise ValueError(f"top_k ({top_k}) exceeds the rows of the {self.keep} groups a token may choose from")
        self.clamp = None if expert_limit is None else (float(expert_limit), float(expert_alpha))
        if self.clamp is not None and self.clamp[0] <= 0:
            raise ValueError("expert_limit must be positive")
        self.correction_name = correction_name
        self.correction = self.new_storage((self.rows,), VECTOR) if self.softmax_all else None
        self.router_bias_name = router_bias_name
        self.bias = self.new_storage((self.experts,), VECTOR) if router_bias else None
        self.expert_prefix, self.router_name = expert_prefix, router_name
        self.shared_prefix, self.shared_gate_name = shared_prefix, shared_gate_name
        self.part_names = (gate_name, up_name, down_name)
        self.gate_up = self.new_storage((self.experts, 2 * self.inter, self.hidden), MATRIX)
        self.down = self.new_storage((self.experts, self.hidden, self.inter), MATRIX)
        # router rows, then the shared expert's gate row: one float32 matrix for the router kernel
        self.has_gate = bool(shared_gate)
        self.router = self.new_storage((self.rows + int(self.has_gate), self.hidden), VECTOR)
        self.shared = None
        if shared_size:
            self.shared = SwiGLU(hidden_size=self.hidden, intermediate_size=int(shared_size), dtype=dtype, device=device,
                                 gate_name=gate_name, up_name=up_name, down_name=down_name, suffix="")

    # -- weights ------------------------------------------------------------ #
    def tensor_specs(self) -> dict[str, TensorSpec]:
        gate, up, down = self.part_names
        specs: dict[str, TensorSpec] = {}
        for e in range(self.experts):
            prefix = f"{self.expert_prefix}{e}."
            specs[prefix + gate] = TensorSpec((self.inter, self.hidden))
            specs[prefix + up] = TensorSpec((self.inter, self.hidden))
            specs[prefix + down] = TensorSpec((self.hidden, self.inter))
        specs[self.router_name] = TensorSpec((self.rows, self.hidden), VECTOR)
        if self.correction is not None:
            specs[self.correction_name] = TensorSpec((self.rows,), VECTOR)
        if self.bias is not None:
            specs[self.router_bias_name] = TensorSpec((self.experts,), VECTOR)
        if self.shared is not None:
            for name, spec in self.shared.tensor_specs().items():
                specs[self.shared_prefix + name] = spec
            if self.has_gate:
                specs[self.shared_prefix + self.shared_gate_name] = TensorSpec((1, self.hidden), VECTOR)
        return specs

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        gate, up, down = self.part_names
        if name == self.router_name:
            self.router[: self.rows].copy_(tensor.to(torch.float32))
            return
        if self.correction is not None and name == self.correction_name:
            self.correction.copy_(tensor.to(torch.float32))
            return
        if self.bias is not None and name == self.router_bias_name:
            self.bias.copy_(tensor.to(torch.float32))
            return
        if self.shared is not None and name.startswith(self.shared_prefix):
            rest = name[len(self.shared_prefix):]
            if self.has_gate and rest == self.shared_gate_name:
                self.router[self.rows :].copy_(tensor.to(torch.float32))
            else:
                self.shared.load_tensor(rest, tensor)
            return
        if name.startswith(self.expert_prefix):
            index, _, rest = name[len(self.expert_prefix):].partition(".")
            if index.isdigit() and int(index) < self.experts:
                e = int(index)
                if rest == gate:
                    self.gate_up[e, : self.inter].copy_(tensor)
                    return
                if rest == up:
                    self.gate_up[e, self.inter :].copy_(tensor)
                    return
                if rest == down:
                    self.down[e].copy_(tensor)
                    return
        raise KeyError(name)

    def parameter_bytes(self) -> int:
        total = (self.gate_up.numel() + self.down.numel()) * self.gate_up.element_size() + self.router.numel() * 4
        return total + (0 if self.shared is None else self.shared.parameter_bytes())

    def workspace_elements_per_token(self) -> int:
        own = self.top * (self.inter + 2 * self.hidden + 8) + self.hidden
        return own + (0 if self.shared is None else self.shared.workspace_elements_per_token())

    def uses_libraries(self) -> set[str]:
        return {"moe"} | ({"gemm"} if self.dtype == torch.bfloat16 else set())

    # -- forward ------------------------------------------------------------ #
    # An arrangement whose norm stands BEHIND the sum (``x <- Norm(alpha x + FeedForward(x))``) may hand that norm to
    # ``forward`` as ``closing``: the last kernel then sums a token's experts, forms the sum with the stream and norms it
    # in one pass, and ``forward`` returns the new stream's rounding instead of the feed-forward's own result.
    closes_sums = True

    def forward(self, x, batch, closing=None):
        space, i32, f32 = batch.workspace, torch.int32, torch.float32
        tokens, top, experts = x.shape[0], self.top, self.experts
        pairs = tokens * top
        ids = space.get("moe_ids", tokens, top, i32)
        weights = space.get("moe_weights", tokens, top, f32)
        gates = space.get("moe_gates", tokens, 1, f32) if self.has_gate else None
        kernels.router_topk(x, self.router, experts=self.rows, top=top, ids=ids, weights=weights, gates=gates,
                            bias=self.bias, softmax_chosen=self.softmax_chosen, softmax_all=self.softmax_all,
                            correction=self.correction, groups=self.groups, keep=self.keep)
        order = space.get("moe_sorted", tokens, top, i32).view(-1)
        place = space.get("moe_place", tokens, top, i32).view(-1)
        wide = kernels.moe_wide_takes(x.dtype, self.hidden, self.inter)      # the pipelined bfloat16 tiles
        most = kernels.moe_max_tiles(max(space.max_tokens, tokens) * top, experts)
        meta = space.get("moe_meta", 1, 1 + 3 * most, i32, min_rows=1).view(-1)
        max_tiles = kernels.moe_plan(ids, experts, order, place, meta, batch.fault, wide=wide)
        act = space.get("moe_act", tokens, top * self.inter, x.dtype).view(pairs, self.inter)
        kernels.grouped_linear(x, self.gate_up, order, meta, top=top, by_token=True, max_tiles=max_tiles,
                               pair_weight=weights.view(-1) if self.scale_input else None, out_act=act, wide=wide,
                               clamp=self.clamp)
        each = space.get("moe_each", tokens, top * self.hidden, f32).view(pairs, self.hidden)
        kernels.grouped_linear(act, self.down, order, meta, top=top, by_token=False, max_tiles=max_tiles, out_y=each, wide=wide)
        shared = None if self.shared is None else self.shared.forward(x, batch)
        if closing is not None and shared is None and hasattr(closing.norm, "bias") and closing.norm.gain == 1.0:
            out = space.get("stream_rows", tokens, self.hidden, x.dtype)
            return kernels.moe_combine_layernorm(
                each, top, closing.residual, closing.norm.weight, closing.norm.bias, out, closing.norm.eps,
                stream_scale=closing.alpha, weights=None if self.scale_input else weights.view(-1),
                ids=ids.view(-1) if self.identity else None, experts=experts, x=x if self.identity else None)
        if closing is not None:
            raise ValueError("this feed-forward closes a sum only with a layer norm and without a shared expert")
        out = space.get("moe_out", tokens, self.hidden, x.dtype)
        # pairs whose id lies behind the experts with tensors (identity experts) are in no tile of the plan: the sum
        # takes the token's own row for them
        return kernels.moe_combine(each, top, out, shared=shared, gate=gates,
                                   weights=None if self.scale_input else weights.view(-1),
                                   ids=ids if self.identity else None, experts=experts, x=x if self.identity else None)
