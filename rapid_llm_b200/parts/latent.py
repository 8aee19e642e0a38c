"""Attention whose keys and values are products of a short cached latent.

Per token the mixer forms a query latent and a key/value latent from its input ``x``:
``c_q = RMSNorm(W_dq x)``, ``q = W_uq c_q`` (per head ``dim`` plain and ``rot`` rotated numbers), and
``[c | k_r] = W_dkv x`` with ``c`` (``kv_rank`` numbers) RMS-normed and ``k_r`` (``rot`` numbers) rotated by the
position and shared by all heads.  Head ``h`` would have the key ``[W_uk_h c | k_r]`` and the value ``W_uv_h c``, with
the score ``(q_plain . W_uk_h c + q_rot . k_r) * scale``, causal softmax, and the output projection over the heads
side by side.  Only ``c`` and ``k_r`` are cached: one row ``[c | k_r | zeros]`` of ``D = ceil16(kv_rank + rot)``
numbers per token (``CacheNeed.token_shape``).

Nothing is expanded per key.  Since ``q_plain . W_uk_h c = (W_uk_h^T q_plain) . c`` and
``sum_j p_j W_uv_h c_j = W_uv_h sum_j p_j c_j``, a step moves ``W_uk`` to the queries (a product per head,
``ops.gemm.heads_linear``) and ``W_uv`` behind the attention, and the attention in between is the paged kernels'
case of ONE key/value head of width ``D`` shared by all query heads, whose values are the keys' own rows (a cache of
one plane).  The zero-padded columns and the ``k_r`` columns of the attended rows meet no column of ``W_uv``.

Options: ``rotation`` ``"halves"`` (entry ``i`` pairs with ``i + rot / 2``) or ``"neighbours"`` (``2i`` with
``2i + 1``); the nested position part gives the frequencies (``rotary_frequencies``, or ``yarn_frequencies`` with its
magnitude on cosine and sine); ``head_gate`` multiplies head ``h``'s output by ``sigmoid(W_g x)_h``, one number per
head from the mixer's input; ``wide_gate`` multiplies the heads side by side, entry by entry, by ``sigmoid(W_g x)``
(``heads * value_dim`` numbers from the mixer's input).  With ``q_rank=None`` there is no query latent: ``q = W_q x``
directly (tensor ``q``).  Norms, rotation and the gates are float32; the softmax is float32 in the attention kernels.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from ..ops import gemm, kernels
from .attention import DEFAULT_SMS, AttentionItems
from .base import MATRIX, MIXERS, POSITION_ENCODINGS, VECTOR, CacheNeed, Mixer, StepPlanner, TensorSpec


def _up8(count: int) -> int:
    return -(-int(count) // 8) * 8


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    DEFAULT_NAMES = ("dq", "dq.norm", "uq", "q", "dkv", "dkv.norm", "uk", "uv", "g", "o")

    def __init__(self, *, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, value_dim: int, kv_rank: int,
                 q_rank: int | None, scale: float, norm_eps: float, position: PartSpec, rotation: str = "halves",
                 head_gate: bool = False, wide_gate: bool = False, names: dict[str, str] | None = None, dtype, device) -> None:
        super().__init__(dtype=dtype, device=device)
        if rotation not in ("halves", "neighbours"):
            raise ValueError(f"rotation must be 'halves' or 'neighbours', got {rotation!r}")
        self.hidden, self.h = int(hidden_size), int(num_heads)
        self.dim, self.rot, self.vdim = int(head_dim), int(rot_dim), int(value_dim)
        self.kv_rank, self.q_rank = int(kv_rank), int(q_rank or 0)
        self.direct_q = q_rank is None        # no query latent: the queries are a product of the mixer's input
        self.scale, self.eps = float(scale), float(norm_eps)
        self.layout = kernels.ROTATE_HALVES if rotation == "halves" else kernels.ROTATE_NEIGHBOURS
        self.has_gate, self.wide_gate = bool(head_gate), bool(wide_gate)
        if self.has_gate and self.wide_gate:
            raise ValueError("latent attention: a gate per head or a gate per entry, not both")
        if min(self.h, self.dim, self.vdim, self.kv_rank, 1 if self.direct_q else self.q_rank) < 1 or self.rot < 0 or self.rot % 2:
            raise ValueError("latent attention: sizes must be positive and the rotated size even")
        self.d = -(-(self.kv_rank + self.rot) // 16) * 16          # a cached row, and a query as the attention sees it
        # the tensor-core tiles take rows of up to 256 numbers; wider rows (up to 640) run the one-warp-per-row kernel
        # in either precision
        self.wide_row = self.d > 256
        if self.d > 640:
            raise ValueError(f"latent attention: kv_rank + rot_dim = {self.kv_rank + self.rot} exceeds the attention "
                             f"kernels' widest row (640)")
        self.names = {name: name for name in self.DEFAULT_NAMES}
        self.names.update(names or {})
        self._ours = {theirs: ours for ours, theirs in self.names.items()}
        self.position = POSITION_ENCODINGS.build(position, dtype=dtype, device=device)
        if self.rot and (not hasattr(self.position, "inv_freq") or self.position.inv_freq.numel() != self.rot // 2):
            raise ValueError("latent attention rotates by frequencies: a position part with rot_dim / 2 of them")
        self.freq = self.position.inv_freq if self.rot else None
        self.magnitude = float(getattr(self.position, "magnitude", 1.0))

        # one product from the mixer's input: the query latent, [c | k_r], and the heads' gates, each from a column
        # that is a multiple of 8
        self.c_col0 = _up8(self.q_rank)
        self.g_col0 = self.c_col0 + _up8(self.kv_rank + self.rot)
        self.down_rows = self.g_col0 + (_up8(self.h) if self.has_gate else self.h * self.vdim if self.wide_gate else 0)
        self.down = self.new_storage((self.down_rows, self.hidden), MATRIX)
        self.q_norm = self.new_storage((self.q_rank,), VECTOR)
        self.c_norm = self.new_storage((self.kv_rank,), VECTOR)
        self.uq = self.new_storage((self.h * (self.dim + self.rot), self.hidden if self.direct_q else self.q_rank), MATRIX)
        self.g = self.down[self.g_col0 :] if self.wide_gate else None      # the wide gate's rows, behind the latent's
        self.uk_t = self.new_storage((self.h, self.kv_rank, self.dim), MATRIX)      # W_uk_h^T: plain query -> latent
        self.uv = self.new_storage((self.h, self.vdim, self.kv_rank), MATRIX)
        self.o = self.new_storage((self.hidden, self.h * self.vdim), MATRIX)
        device = torch.device(device)
        sms = torch.cuda.get_device_properties(device).multi_processor_count if device.type == "cuda" else DEFAULT_SMS
        # the mma.sync tiles read a cache of one plane; the tcgen05 tiles do not
        self._items = AttentionItems(self.h, 1, self.d, sms, None, tensor_core=False)

    # -- needs ----------------------------------------------------------------- #
    def cache_need(self) -> CacheNeed:
        return CacheNeed("full", token_shape=(self.d,))

    def step_planner(self) -> StepPlanner | None:
        return self._items if self.dtype == torch.bfloat16 and not self.wide_row else None

    def uses_libraries(self) -> set[str]:
        found = {"latent"}
        if self.dtype == torch.bfloat16:
            from ..ops.build import attention_library
            found |= {"gemm"} | (set() if self.wide_row else {attention_library(self.d)})
        return found

    # -- weights --------------------------------------------------------------- #
    def tensor_specs(self) -> dict[str, TensorSpec]:
        specs = {
            "dq": TensorSpec((self.q_rank, self.hidden)),
            "dq.norm": TensorSpec((self.q_rank,), VECTOR, init="ones_normal"),
            "uq": TensorSpec((self.h * (self.dim + self.rot), self.q_rank)),
            "dkv": TensorSpec((self.kv_rank + self.rot, self.hidden)),
            "dkv.norm": TensorSpec((self.kv_rank,), VECTOR, init="ones_normal"),
            "uk": TensorSpec((self.h * self.dim, self.kv_rank)),
            "uv": TensorSpec((self.h * self.vdim, self.kv_rank)),
            "o": TensorSpec((self.hidden, self.h * self.vdim)),
        }
        if self.direct_q:
            del specs["dq"], specs["dq.norm"], specs["uq"]
            specs["q"] = TensorSpec((self.h * (self.dim + self.rot), self.hidden))
        if self.has_gate:
            specs["g"] = TensorSpec((self.h, self.hidden))
        if self.wide_gate:
            specs["g"] = TensorSpec((self.h * self.vdim, self.hidden))
        return {self.names[name]: spec for name, spec in specs.items()}

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        name = self._ours.get(name, "")
        if name == "dq":
            self.down[: self.q_rank].copy_(tensor)
        elif name == "dkv":
            self.down[self.c_col0 : self.c_col0 + self.kv_rank + self.rot].copy_(tensor)
        elif name == "g" and self.has_gate:
            self.down[self.g_col0 : self.g_col0 + self.h].copy_(tensor)
        elif name == "g" and self.wide_gate:
            self.g.copy_(tensor)
        elif name == "q" and self.direct_q:
            self.uq.copy_(tensor)
        elif name == "dq.norm":
            self.q_norm.copy_(tensor.to(torch.float32))
        elif name == "dkv.norm":
            self.c_norm.copy_(tensor.to(torch.float32))
        elif name == "uq":
            self.uq.copy_(tensor)
        elif name == "uk":
            self.uk_t.copy_(tensor.view(self.h, self.dim, self.kv_rank).transpose(1, 2))
        elif name == "uv":
            self.uv.copy_(tensor.view(self.h, self.vdim, self.kv_rank))
        elif name == "o":
            self.o.copy_(tensor)
        else:
            raise KeyError(name)

    def parameter_bytes(self) -> int:
        matrices = (self.down, self.uq, self.uk_t, self.uv, self.o)
        return sum(m.numel() for m in matrices) * self.down.element_size() + (self.q_rank + self.kv_rank) * 4

    def workspace_elements_per_token(self) -> int:
        return (self.down_rows + self.q_rank + self.h * (self.dim + self.rot) + 2 * self.h * self.d
                + (2 if self.wide_gate else 1) * self.h * self.vdim + self.hidden)

    # -- forward --------------------------------------------------------------- #
    def forward(self, x, batch, cache):
        if cache.group is None or cache.pages is None or not cache.writes:
            raise ValueError("latent attention needs a cache group of its own; the engine did not give this layer one")
        group, space, rows = batch.groups[cache.group], batch.workspace, x.shape[0]
        pages = cache.pages                                       # [pages, page_size, D]
        down = gemm.linear(x, self.down, space.get("latent_down", rows, self.down_rows, x.dtype), batch.fault)
        gemm.flush()
        c_q = space.get("latent_cq", rows, self.q_rank, x.dtype)      # no columns without a query latent
        kernels.latent_norm_write(
            down, q_col0=0, q_rank=self.q_rank, c_col0=self.c_col0, kv_rank=self.kv_rank, rot=self.rot,
            q_weight=self.q_norm, c_weight=self.c_norm, eps=self.eps, q_out=c_q, cache=pages, kv_dest=group.kv_dest,
            positions=batch.positions, freq=self.freq, magnitude=self.magnitude, layout=self.layout, fault=batch.fault)
        q = gemm.linear(x if self.direct_q else c_q, self.uq, space.get("latent_q", rows, self.uq.shape[0], x.dtype), batch.fault)
        gemm.flush()
        wide = space.get("latent_wide", rows, self.h * self.d, x.dtype)
        gemm.heads_linear(q, self.uk_t, wide)                  # columns [0, kv_rank) of every head
        kernels.latent_rotate_queries(q, wide, heads=self.h, dim=self.dim, rot=self.rot, kv_rank=self.kv_rank,
                                      positions=batch.positions, freq=self.freq, magnitude=self.magnitude,
                                      layout=self.layout)
        attended = space.get("latent_attended", rows, self.h * self.d, x.dtype)
        self._attend(wide, pages.view(pages.shape[0], 1, 1, pages.shape[1], self.d), attended, batch, group)
        values = space.get("latent_values", rows, self.h * self.vdim, x.dtype)
        gemm.heads_linear(attended, self.uv, values)
        if self.has_gate:
            kernels.sigmoid_scale_heads(values, down[:, self.g_col0 :], heads=self.h)
        if self.wide_gate:
            values = kernels.sigmoid_gate(values, down[:, self.g_col0 :], space.get("latent_gated", rows, self.h * self.vdim, x.dtype))
        return gemm.linear(values, self.o, space.get("latent_out", rows, self.hidden, x.dtype), batch.fault)

    def _attend(self, q, pages, out, batch, group) -> None:
        if q.dtype == torch.bfloat16 and not self.wide_row:
            plan = batch.extras[self._items.key]
            splits = plan["splits"]
            part_out = part_lse = None
            if splits > 1:
                rows = q.shape[0] * self.h * splits
                part_out = batch.workspace.get("attn_part_out", rows, self.d, torch.float32, min_rows=rows)
                part_lse = batch.workspace.get("attn_part_lse", rows, 1, torch.float32, min_rows=rows)
            kernels.attention_mma(
                q, pages, out, chunk_items=plan["chunk_items"], decode_items=plan["decode_items"], splits=splits,
                part_out=part_out, part_lse=part_lse, cu_seqlens=batch.cu_seqlens, entry_start=batch.entry_start,
                entry_slot=batch.entry_slot, block_table=group.block_table, num_heads=self.h, num_kv_heads=1,
                head_dim=self.d, window=0, scale=self.scale, fault=batch.fault, decode_kernel="mma",
                decode_rows=plan.get("decode_rows", 0), chunk_rows=kernels.CHUNK_TILE_ROWS)
            return
        kernels.attention_generic(
            q, pages, out, positions=batch.positions, token_slot=batch.token_slot, block_table=group.block_table,
            num_heads=self.h, num_kv_heads=1, head_dim=self.d, window=0, scale=self.scale, fault=batch.fault)
