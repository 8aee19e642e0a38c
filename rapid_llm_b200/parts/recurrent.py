"""Mixers that carry a state of fixed size per request: linear recurrences over a matrix ``S``.

All of them keep, per head, a float32 matrix ``S`` of ``key_dim x value_dim`` in the request's state row
and advance it token by token in one kernel (``ops.kernels.linear_scan``), which serves portions of
prompts and single decoded tokens alike:

* :class:`ChannelDeltaRule` (``gated_delta_rule``) — the delta rule with a decay per head and key channel:
  ``S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q``.
* :class:`Retention` (``retention``) — a fixed decay per head, no correction:
  ``S <- gamma S + k v^T; o = S^T q``, queries and keys rotated by position.
* :class:`Lightning` (``lightning``) — the same recurrence with SiLU on q, k and v, no rotation, and one norm
  over the heads side by side: ``S <- gamma S + k v^T; o = S^T q``.
* :class:`ShiftedDecay` (``wkv``) — a decay per token, head and key channel computed from the input, every
  projection reading a blend of the token's row with the row before it, and a bonus for the token's own pair:
  ``o = (S + diag(u) k v^T)^T r; S <- diag(w) S + k v^T``.
* :class:`StateSpaceDual` (``state_space_dual``) — the selective state space in its recurrent form:
  ``S <- exp(-exp(A) dt) S + dt B x^T; y = S^T C + D x``.

Projections are matrix products in the engine's dtype; everything between them and the output projection
that enters the recurrence (short convolutions' results, unit vectors, decays, step sizes, write
strengths, the state, the read-out) is float32 in both precisions.  A mixer with a short convolution also
keeps the convolution's last ``width - 1`` inputs in its state row, behind ``S``.

Every size is a constructor parameter; ``names`` maps the default tensor names to an architecture's own.
"""

from __future__ import annotations

import torch

from ..ops import gemm, kernels
from .base import MATRIX, MIXERS, VECTOR, Mixer, StateNeed, TensorSpec


class _Recurrent(Mixer):
    """What the three share: named tensors, the state row, the libraries they launch from."""

    DEFAULT_NAMES: tuple[str, ...] = ()

    def _set_names(self, names: dict[str, str] | None) -> None:
        self.names = {name: name for name in self.DEFAULT_NAMES}
        self.names.update(names or {})
        self._ours = {theirs: ours for ours, theirs in self.names.items()}

    def _named(self, specs: dict[str, TensorSpec]) -> dict[str, TensorSpec]:
        return {self.names[name]: spec for name, spec in specs.items()}

    def uses_libraries(self) -> set[str]:
        return {"recurrent"} | ({"gemm"} if self.dtype == torch.bfloat16 else set())

    def state_need(self) -> StateNeed:
        return StateNeed((self.state_size + self.tail_size,), torch.float32)

    def _state_views(self, cache) -> tuple[torch.Tensor, torch.Tensor]:
        state = cache.state
        if state is None or state.shape[1] != self.state_size + self.tail_size or state.dtype != torch.float32:
            raise ValueError("the engine did not give this mixer the state row it asked for")
        return state[:, : self.state_size], state[:, self.state_size :]

    def parameter_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._tensors())

    def finalize(self, loaded: set[str]) -> None:
        """The decay's rate ``exp(A_log)`` (float32) is taken once here, for the mixers that have one."""
        if hasattr(self, "a_log"):
            self.rate = torch.exp(self.a_log)


@MIXERS.register("gated_delta_rule")
class ChannelDeltaRule(_Recurrent):
    """Delta rule with a decay per head and key channel.

    ``q, k`` (``num_kv_heads`` heads of ``key_dim``) and ``v`` (``num_heads`` of ``value_dim``) pass a causal
    convolution of ``conv_width`` taps per channel and SiLU; q and k become unit vectors per head
    (``x / sqrt(sum x^2 + unit_eps)``), q times ``key_dim ** -0.5``.  ``beta = sigmoid(W_b x)`` per head;
    ``g = exp(-exp(A_log[h]) * softplus(W_a2 W_a1 x + dt_bias))`` per head and key channel.  The read-out of a
    head is divided by its root mean square, multiplied by ``norm`` (one weight per value channel, shared by
    the heads) and by ``sigmoid(W_g2 W_g1 x)``, then projected.
    """

    DEFAULT_NAMES = ("q", "k", "v", "q.conv", "k.conv", "v.conv", "b", "a1", "a2", "g1", "g2", "A_log", "dt_bias",
                     "norm", "o")

    def __init__(self, *, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int,
                 conv_width: int, decay_rank: int, gate_rank: int, norm_eps: float, unit_eps: float = 1e-6,
                 names: dict[str, str] | None = None, dtype, device) -> None:
        super().__init__(dtype=dtype, device=device)
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads ({num_heads}) must be divisible by num_kv_heads ({num_kv_heads})")
        self._set_names(names)
        self.hidden, self.h, self.hk = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.dim, self.vdim, self.width = int(key_dim), int(value_dim), int(conv_width)
        self.ra, self.rg = int(decay_rank), int(gate_rank)
        self.eps, self.unit_eps = float(norm_eps), float(unit_eps)
        self.cq, self.cv = self.hk * self.dim, self.h * self.vdim
        self.conv_channels = 2 * self.cq + self.cv
        self.state_size = self.h * self.dim * self.vdim
        self.tail_size = (self.width - 1) * self.conv_channels
        self.w_in = self.new_storage((self.conv_channels + self.h, self.hidden), MATRIX)        # q | k | v | b
        self.w_low = self.new_storage((self.ra + self.rg, self.hidden), MATRIX)                 # a1 | g1
        # a2 and g2 as one block-diagonal matrix over the rows of [a1 x | g1 x]
        self.w_high = self.new_storage((self.h * self.dim + self.cv, self.ra + self.rg), MATRIX)
        self.o = self.new_storage((self.hidden, self.cv), MATRIX)
        self.taps = self.new_storage((self.conv_channels, self.width), VECTOR)
        self.a_log = self.new_storage((self.h,), VECTOR)
        self.dt_bias = self.new_storage((self.h * self.dim,), VECTOR)
        self.norm = self.new_storage((self.vdim,), VECTOR)

    def _tensors(self):
        return (self.w_in, self.w_low, self.w_high, self.o, self.taps, self.a_log, self.dt_bias, self.norm)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return self._named({
            "q": TensorSpec((self.cq, self.hidden)),
            "q.conv": TensorSpec((self.cq, self.width), VECTOR),
            "k": TensorSpec((self.cq, self.hidden)),
            "k.conv": TensorSpec((self.cq, self.width), VECTOR),
            "v": TensorSpec((self.cv, self.hidden)),
            "v.conv": TensorSpec((self.cv, self.width), VECTOR),
            "b": TensorSpec((self.h, self.hidden)),
            "A_log": TensorSpec((self.h,), VECTOR),
            "norm": TensorSpec((self.vdim,), VECTOR, init="ones_normal"),
            "a1": TensorSpec((self.ra, self.hidden)),
            "a2": TensorSpec((self.h * self.dim, self.ra)),
            "dt_bias": TensorSpec((self.h * self.dim,), VECTOR),
            "g1": TensorSpec((self.rg, self.hidden)),
            "g2": TensorSpec((self.cv, self.rg)),
            "o": TensorSpec((self.hidden, self.cv)),
        })

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        name = self._ours.get(name, "")
        cq, cv, f32 = self.cq, self.cv, torch.float32
        rows = {"q": (0, cq), "k": (cq, 2 * cq), "v": (2 * cq, 2 * cq + cv)}
        if name in rows:
            self.w_in[rows[name][0] : rows[name][1]].copy_(tensor)
        elif name.endswith(".conv") and name[0] in rows:
            self.taps[rows[name[0]][0] : rows[name[0]][1]].copy_(tensor.to(f32))
        elif name == "b":
            self.w_in[self.conv_channels :].copy_(tensor)
        elif name == "a1":
            self.w_low[: self.ra].copy_(tensor)
        elif name == "g1":
            self.w_low[self.ra :].copy_(tensor)
        elif name == "a2":
            self.w_high[: self.h * self.dim, : self.ra].copy_(tensor)
        elif name == "g2":
            self.w_high[self.h * self.dim :, self.ra :].copy_(tensor)
        elif name == "o":
            self.o.copy_(tensor)
        elif name == "A_log":
            self.a_log.copy_(tensor.to(f32))
        elif name == "dt_bias":
            self.dt_bias.copy_(tensor.to(f32))
        elif name == "norm":
            self.norm.copy_(tensor.to(f32))
        else:
            raise KeyError(name)

    def workspace_elements_per_token(self) -> int:
        return 3 * (self.w_in.shape[0] + self.w_high.shape[0]) + self.ra + self.rg + self.hidden

    def forward(self, x, batch, cache):
        rows, space, f32 = x.shape[0], batch.workspace, torch.float32
        S, tail = self._state_views(cache)
        proj = gemm.linear(x, self.w_in, space.get("delta_in", rows, self.w_in.shape[0], x.dtype), batch.fault)
        low = gemm.linear(x, self.w_low, space.get("delta_low", rows, self.w_low.shape[0], x.dtype), batch.fault)
        high = gemm.linear(low, self.w_high, space.get("delta_high", rows, self.w_high.shape[0], x.dtype), batch.fault)
        conv = space.get("delta_conv", rows, self.conv_channels, f32)
        kernels.causal_conv_silu(proj[:, : self.conv_channels], self.taps, None, tail, conv, batch)
        beta = space.get("delta_beta", rows, self.h, f32)
        kernels.unit_heads(conv[:, : 2 * self.cq], heads=2 * self.hk, dim=self.dim, eps=self.unit_eps, split=self.hk,
                           scale_low=self.dim ** -0.5, scale_high=1.0, gate_in=proj[:, self.conv_channels :], gate_out=beta)
        decay = space.get("delta_decay", rows, self.h * self.dim, f32)
        kernels.decay_gate(high[:, : self.h * self.dim], self.rate, self.dt_bias, self.dim, decay)
        read = space.get("delta_read", rows, self.cv, f32)
        kernels.linear_scan(conv[:, : self.cq], conv[:, self.cq : 2 * self.cq], conv[:, 2 * self.cq :], decay, read, S,
                            batch, heads=self.h, kv_heads=self.hk, dim=self.dim, vdim=self.vdim, beta=beta)
        normed = space.get("delta_normed", rows, self.cv, x.dtype)
        kernels.gated_norm(read, normed, group=self.vdim, gate=high[:, self.h * self.dim :], act=kernels.GATE_SIGMOID,
                           weight=self.norm, eps=self.eps)
        return gemm.linear(normed, self.o, space.get("delta_out", rows, self.hidden, x.dtype), batch.fault)


@MIXERS.register("retention")
class Retention(_Recurrent):
    """Linear attention with a fixed decay per head and neither softmax nor denominator.

    The first ``rotary_dims`` entries of every query and key head rotate by position (entry ``i`` paired with
    ``i + rotary_dims / 2``, angle ``p * rotary_base ** (-2 i / rotary_dims)``); keys are then multiplied by
    ``key_dim ** -0.5``.  The read-out of a head is divided by its root mean square (no weight); the
    concatenated heads are multiplied by ``SiLU(W_g x)`` and projected.
    """

    DEFAULT_NAMES = ("q", "k", "v", "g", "o")

    def __init__(self, *, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, decay, rotary_dims: int,
                 rotary_base: float, norm_eps: float, names: dict[str, str] | None = None, dtype, device) -> None:
        super().__init__(dtype=dtype, device=device)
        self._set_names(names)
        self.hidden, self.h, self.dim, self.vdim = int(hidden_size), int(num_heads), int(key_dim), int(value_dim)
        self.rot, self.eps = int(rotary_dims), float(norm_eps)
        if len(decay) != self.h:
            raise ValueError(f"retention needs one decay per head, got {len(decay)} for {self.h} heads")
        if self.rot % 2 or not 0 <= self.rot <= self.dim:
            raise ValueError(f"rotary_dims ({self.rot}) must be even and within key_dim ({self.dim})")
        self.cq, self.cv = self.h * self.dim, self.h * self.vdim
        self.state_size, self.tail_size = self.h * self.dim * self.vdim, 0
        self.w_in = self.new_storage((2 * self.cq + 2 * self.cv, self.hidden), MATRIX)      # q | k | v | g
        self.o = self.new_storage((self.hidden, self.cv), MATRIX)
        self.decay = torch.tensor([float(d) for d in decay], dtype=torch.float32).to(self.device)
        exponents = torch.arange(0, self.rot, 2, dtype=torch.float32) / max(self.rot, 1)
        self.inv_freq = (1.0 / (torch.tensor(float(rotary_base), dtype=torch.float32) ** exponents)).to(self.device)

    def _tensors(self):
        return (self.w_in, self.o)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return self._named({
            "q": TensorSpec((self.cq, self.hidden)),
            "k": TensorSpec((self.cq, self.hidden)),
            "v": TensorSpec((self.cv, self.hidden)),
            "g": TensorSpec((self.cv, self.hidden)),
            "o": TensorSpec((self.hidden, self.cv)),
        })

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        name = self._ours.get(name, "")
        cq, cv = self.cq, self.cv
        rows = {"q": (0, cq), "k": (cq, 2 * cq), "v": (2 * cq, 2 * cq + cv), "g": (2 * cq + cv, 2 * cq + 2 * cv)}
        if name in rows:
            self.w_in[rows[name][0] : rows[name][1]].copy_(tensor)
        elif name == "o":
            self.o.copy_(tensor)
        else:
            raise KeyError(name)

    def workspace_elements_per_token(self) -> int:
        return 4 * self.w_in.shape[0] + self.hidden

    def forward(self, x, batch, cache):
        rows, space, f32 = x.shape[0], batch.workspace, torch.float32
        S, _ = self._state_views(cache)
        cq, cv = self.cq, self.cv
        proj = gemm.linear(x, self.w_in, space.get("ret_in", rows, self.w_in.shape[0], x.dtype), batch.fault)
        qkv = space.get("ret_qkv", rows, 2 * cq + cv, f32)
        kernels.rotate_heads(proj[:, :cq], proj[:, cq : 2 * cq], proj[:, 2 * cq : 2 * cq + cv], qkv, batch.positions,
                             self.inv_freq, heads=self.h, dim=self.dim, vdim=self.vdim, k_scale=self.dim ** -0.5)
        read = space.get("ret_read", rows, cv, f32)
        kernels.linear_scan(qkv[:, :cq], qkv[:, cq : 2 * cq], qkv[:, 2 * cq :], self.decay, read, S, batch,
                            heads=self.h, kv_heads=self.h, dim=self.dim, vdim=self.vdim)
        normed = space.get("ret_normed", rows, cv, x.dtype)
        kernels.gated_norm(read, normed, group=self.vdim, gate=proj[:, 2 * cq + cv :], act=kernels.GATE_SILU, eps=self.eps)
        return gemm.linear(normed, self.o, space.get("ret_out", rows, self.hidden, x.dtype), batch.fault)


@MIXERS.register("lightning")
class Lightning(_Recurrent):
    """Linear attention with a fixed decay per head: ``q = silu(W_q x)``, ``k = silu(W_k x)``, ``v = silu(W_v x)``,
    per head ``S <- decay_h S + k v^T`` and ``o = S^T q`` with no other scale.  The heads side by side are divided by
    the root mean square of the whole row and multiplied by ``norm`` (one weight per column), then by
    ``sigmoid(W_g x)``, then projected.  The activations' results, the state and the read-out are float32."""

    DEFAULT_NAMES = ("q", "k", "v", "g", "o", "norm")

    def __init__(self, *, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, decay, norm_eps: float,
                 names: dict[str, str] | None = None, dtype, device) -> None:
        super().__init__(dtype=dtype, device=device)
        self._set_names(names)
        self.hidden, self.h, self.dim, self.vdim = int(hidden_size), int(num_heads), int(key_dim), int(value_dim)
        self.eps = float(norm_eps)
        if len(decay) != self.h:
            raise ValueError(f"lightning needs one decay per head, got {len(decay)} for {self.h} heads")
        self.cq, self.cv = self.h * self.dim, self.h * self.vdim
        self.state_size, self.tail_size = self.h * self.dim * self.vdim, 0
        self.w_in = self.new_storage((2 * self.cq + 2 * self.cv, self.hidden), MATRIX)      # q | k | v | g
        self.o = self.new_storage((self.hidden, self.cv), MATRIX)
        self.norm = self.new_storage((self.cv,), VECTOR)
        self.decay = torch.tensor([float(d) for d in decay], dtype=torch.float32).to(self.device)

    def _tensors(self):
        return (self.w_in, self.o, self.norm)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return self._named({
            "q": TensorSpec((self.cq, self.hidden)),
            "k": TensorSpec((self.cq, self.hidden)),
            "v": TensorSpec((self.cv, self.hidden)),
            "g": TensorSpec((self.cv, self.hidden)),
            "o": TensorSpec((self.hidden, self.cv)),
            "norm": TensorSpec((self.cv,), VECTOR, init="ones_normal"),
        })

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        name = self._ours.get(name, "")
        cq, cv = self.cq, self.cv
        rows = {"q": (0, cq), "k": (cq, 2 * cq), "v": (2 * cq, 2 * cq + cv), "g": (2 * cq + cv, 2 * cq + 2 * cv)}
        if name in rows:
            self.w_in[rows[name][0] : rows[name][1]].copy_(tensor)
        elif name == "o":
            self.o.copy_(tensor)
        elif name == "norm":
            self.norm.copy_(tensor.to(torch.float32))
        else:
            raise KeyError(name)

    def workspace_elements_per_token(self) -> int:
        return 4 * self.w_in.shape[0] + self.hidden

    def forward(self, x, batch, cache):
        rows, space, f32 = x.shape[0], batch.workspace, torch.float32
        S, _ = self._state_views(cache)
        cq, cv = self.cq, self.cv
        proj = gemm.linear(x, self.w_in, space.get("lightning_in", rows, self.w_in.shape[0], x.dtype), batch.fault)
        qkv = kernels.activate_rows(proj[:, : 2 * cq + cv], space.get("lightning_qkv", rows, 2 * cq + cv, f32), act=True)
        read = space.get("lightning_read", rows, cv, f32)
        kernels.linear_scan(qkv[:, :cq], qkv[:, cq : 2 * cq], qkv[:, 2 * cq :], self.decay, read, S, batch,
                            heads=self.h, kv_heads=self.h, dim=self.dim, vdim=self.vdim)
        normed = space.get("lightning_normed", rows, cv, x.dtype)
        kernels.gated_norm(read, normed, group=cv, gate=proj[:, 2 * cq + cv :], act=kernels.GATE_SIGMOID,
                           weight=self.norm, eps=self.eps)
        return gemm.linear(normed, self.o, space.get("lightning_out", rows, self.hidden, x.dtype), batch.fault)


@MIXERS.register("state_space_dual")
class StateSpaceDual(_Recurrent):
    """Selective state space with one decay per head and token, in its recurrent form.

    ``W_in x = [z | x | B | C | dt]`` with ``inner = num_heads * head_dim`` columns of ``z`` and ``x``,
    ``groups * state_size`` of ``B`` and ``C`` each (head ``h`` uses group ``h // (num_heads / groups)``) and one
    ``dt`` per head.  ``x, B, C`` pass a causal convolution (``conv_width`` taps and a bias per channel) and
    SiLU; ``dt <- softplus(dt + dt_bias)``.  Per head ``S <- exp(-exp(A_log) dt) S + dt B x^T`` and
    ``y = S^T C + D x``.  ``y * SiLU(z)`` is normed in ``norm_groups`` equal parts (each by its own root mean
    square), multiplied by ``norm`` and projected.
    """

    DEFAULT_NAMES = ("in", "conv", "conv.b", "dt_bias", "A_log", "D", "norm", "o")

    def __init__(self, *, hidden_size: int, num_heads: int, head_dim: int, state_size: int, groups: int,
                 conv_width: int, norm_groups: int, norm_eps: float, names: dict[str, str] | None = None,
                 dtype, device) -> None:
        super().__init__(dtype=dtype, device=device)
        self._set_names(names)
        self.hidden, self.h, self.vdim = int(hidden_size), int(num_heads), int(head_dim)
        self.n, self.groups, self.width = int(state_size), int(groups), int(conv_width)
        self.norm_groups, self.eps = int(norm_groups), float(norm_eps)
        self.inner = self.h * self.vdim
        if self.h % self.groups:
            raise ValueError(f"num_heads ({self.h}) must be divisible by groups ({self.groups})")
        if self.inner % self.norm_groups:
            raise ValueError(f"norm_groups ({self.norm_groups}) must divide the inner size ({self.inner})")
        self.conv_channels = self.inner + 2 * self.groups * self.n
        self.state_size = self.h * self.n * self.vdim
        self.tail_size = (self.width - 1) * self.conv_channels
        self.w_in = self.new_storage((self.inner + self.conv_channels + self.h, self.hidden), MATRIX)
        self.o = self.new_storage((self.hidden, self.inner), MATRIX)
        self.taps = self.new_storage((self.conv_channels, self.width), VECTOR)
        self.conv_bias = self.new_storage((self.conv_channels,), VECTOR)
        self.dt_bias = self.new_storage((self.h,), VECTOR)
        self.a_log = self.new_storage((self.h,), VECTOR)
        self.skip = self.new_storage((self.h,), VECTOR)
        self.norm = self.new_storage((self.inner,), VECTOR)

    def _tensors(self):
        return (self.w_in, self.o, self.taps, self.conv_bias, self.dt_bias, self.a_log, self.skip, self.norm)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return self._named({
            "in": TensorSpec(tuple(self.w_in.shape)),
            "conv": TensorSpec((self.conv_channels, self.width), VECTOR),
            "conv.b": TensorSpec((self.conv_channels,), VECTOR),
            "dt_bias": TensorSpec((self.h,), VECTOR),
            "A_log": TensorSpec((self.h,), VECTOR),
            "D": TensorSpec((self.h,), VECTOR, init="ones_normal"),
            "norm": TensorSpec((self.inner,), VECTOR, init="ones_normal"),
            "o": TensorSpec((self.hidden, self.inner)),
        })

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        name = self._ours.get(name, "")
        vectors = {"conv": self.taps, "conv.b": self.conv_bias, "dt_bias": self.dt_bias, "A_log": self.a_log,
                   "D": self.skip, "norm": self.norm}
        if name == "in":
            self.w_in.copy_(tensor)
        elif name == "o":
            self.o.copy_(tensor)
        elif name in vectors:
            vectors[name].copy_(tensor.to(torch.float32))
        else:
            raise KeyError(name)

    def workspace_elements_per_token(self) -> int:
        return 4 * self.w_in.shape[0] + self.hidden

    def forward(self, x, batch, cache):
        rows, space, f32 = x.shape[0], batch.workspace, torch.float32
        S, tail = self._state_views(cache)
        inner, gn, mixed = self.inner, self.groups * self.n, self.conv_channels
        proj = gemm.linear(x, self.w_in, space.get("ssd_in", rows, self.w_in.shape[0], x.dtype), batch.fault)
        conv = space.get("ssd_conv", rows, mixed, f32)
        kernels.causal_conv_silu(proj[:, inner : inner + mixed], self.taps, self.conv_bias, tail, conv, batch)
        decay, step = space.get("ssd_decay", rows, self.h, f32), space.get("ssd_step", rows, self.h, f32)
        kernels.decay_gate(proj[:, inner + mixed :], self.rate, self.dt_bias, 1, decay, step)
        read = space.get("ssd_read", rows, inner, f32)
        kernels.linear_scan(conv[:, inner + gn :], conv[:, inner : inner + gn], conv[:, :inner], decay, read, S, batch,
                            heads=self.h, kv_heads=self.groups, dim=self.n, vdim=self.vdim, v_scale=step, skip=self.skip)
        normed = space.get("ssd_normed", rows, inner, x.dtype)
        kernels.gated_norm(read, normed, group=inner // self.norm_groups, gate=proj[:, :inner], act=kernels.GATE_SILU,
                           gate_first=True, weight=self.norm, eps=self.eps)
        return gemm.linear(normed, self.o, space.get("ssd_out", rows, self.hidden, x.dtype), batch.fault)


@MIXERS.register("wkv")
class ShiftedDecay(_Recurrent):
    """Linear attention whose projections read blends with the row before, with a decay made from the input.

    With ``x'`` the request's previous row (zeros for its first token) each of r, k, v, g, w reads a blend of its own,
    ``x + (x' - x) * mu_s``.  ``r, k, v = W_r, W_k, W_v`` of their blends (``num_heads`` heads of ``key_dim``; values
    have the keys' size), ``gate = SiLU(W_g .)``, and the decay per head and key channel is
    ``w = exp(-exp(W_w2 tanh(W_w1 .) + w0))``.  Per head ``o = (S + diag(u) k v^T)^T r`` and then
    ``S <- diag(w) S + k v^T``: the bonus ``u`` weighs the token's own pair in its own read-out only.  Every head's
    read-out is divided by its root mean square; the heads side by side are multiplied by ``norm`` (a weight per
    column) and by the gate, then projected.  The blends' arithmetic, the decay, the state and the read-out are
    float32; the request's last row is kept, in float32, behind ``S`` in its state row.
    """

    DEFAULT_NAMES = ("mu.r", "mu.k", "mu.v", "mu.g", "mu.w", "r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o")
    BLENDS = ("r", "k", "v", "g", "w")

    def __init__(self, *, hidden_size: int, num_heads: int, key_dim: int, decay_rank: int, norm_eps: float,
                 names: dict[str, str] | None = None, dtype, device) -> None:
        super().__init__(dtype=dtype, device=device)
        self._set_names(names)
        self.hidden, self.h, self.dim, self.rank = int(hidden_size), int(num_heads), int(key_dim), int(decay_rank)
        self.eps = float(norm_eps)
        self.c = self.h * self.dim
        self.state_size, self.tail_size = self.h * self.dim * self.dim, self.hidden
        self.mu = self.new_storage((len(self.BLENDS), self.hidden), VECTOR)
        self.w_rkvg = self.new_storage((4, self.c, self.hidden), MATRIX)
        self.w1 = self.new_storage((self.rank, self.hidden), MATRIX)
        self.w2 = self.new_storage((self.c, self.rank), MATRIX)
        self.w0 = self.new_storage((self.c,), VECTOR)
        self.bonus = self.new_storage((self.h, self.dim), VECTOR)
        self.norm = self.new_storage((self.c,), VECTOR)
        self.o = self.new_storage((self.hidden, self.c), MATRIX)

    def _tensors(self):
        return (self.mu, self.w_rkvg, self.w1, self.w2, self.w0, self.bonus, self.norm, self.o)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        specs = {f"mu.{which}": TensorSpec((self.hidden,), VECTOR) for which in self.BLENDS}
        for which in ("r", "k", "v", "g"):
            specs[which] = TensorSpec((self.c, self.hidden))
        specs.update({
            "w1": TensorSpec((self.rank, self.hidden)), "w2": TensorSpec((self.c, self.rank)),
            "w0": TensorSpec((self.c,), VECTOR), "u": TensorSpec((self.h, self.dim), VECTOR),
            "norm": TensorSpec((self.c,), VECTOR, init="ones_normal"), "o": TensorSpec((self.hidden, self.c)),
        })
        return self._named(specs)

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        name = self._ours.get(name, "")
        f32 = torch.float32
        if name.startswith("mu.") and name[3:] in self.BLENDS:
            self.mu[self.BLENDS.index(name[3:])].copy_(tensor.to(f32))
        elif name in ("r", "k", "v", "g"):
            self.w_rkvg["rkvg".index(name)].copy_(tensor)
        elif name == "w1":
            self.w1.copy_(tensor)
        elif name == "w2":
            self.w2.copy_(tensor)
        elif name == "o":
            self.o.copy_(tensor)
        elif name == "w0":
            self.w0.copy_(tensor.to(f32))
        elif name == "u":
            self.bonus.copy_(tensor.to(f32))
        elif name == "norm":
            self.norm.copy_(tensor.to(f32))
        else:
            raise KeyError(name)

    def workspace_elements_per_token(self) -> int:
        return 5 * self.hidden + 4 * self.c + 2 * (4 * self.c) + 2 * self.rank + self.hidden

    def forward(self, x, batch, cache):
        rows, space, f32, c = x.shape[0], batch.workspace, torch.float32, self.c
        S, kept = self._state_views(cache)
        blends = kernels.shift_mix(x, self.mu, space.get("wkv_blends", 5 * rows, self.hidden, x.dtype), kept, batch)
        proj = space.get("wkv_proj", 4 * rows, c, x.dtype)               # planes r | k | v | g
        for index in range(4):
            gemm.linear(blends[index * rows : (index + 1) * rows], self.w_rkvg[index],
                        proj[index * rows : (index + 1) * rows], batch.fault)
        low = gemm.linear(blends[4 * rows :], self.w1, space.get("wkv_low", rows, self.rank, x.dtype), batch.fault)
        gemm.flush()
        kernels.tanh_rows(low, low)
        high = gemm.linear(low, self.w2, space.get("wkv_high", rows, c, x.dtype), batch.fault)
        gemm.flush()
        decay = kernels.exp_decay(high, self.w0, space.get("wkv_decay", rows, c, f32))
        rkv = kernels.activate_rows(proj[: 3 * rows], space.get("wkv_rkv", 3 * rows, c, f32), act=False)
        read = space.get("wkv_read", rows, c, f32)
        kernels.linear_scan(rkv[:rows], rkv[rows : 2 * rows], rkv[2 * rows :], decay, read, S, batch, heads=self.h,
                            kv_heads=self.h, dim=self.dim, vdim=self.dim, bonus=self.bonus)
        normed = space.get("wkv_normed", rows, c, x.dtype)
        kernels.gated_norm(read, normed, group=self.dim, gate=proj[3 * rows :], act=kernels.GATE_SILU, weight=self.norm,
                           eps=self.eps)
        return gemm.linear(normed, self.o, space.get("wkv_out", rows, self.hidden, x.dtype), batch.fault)
