"""Grouped-query attention over the paged cache.

Order of operations is the reference's (``rapid_llm/models/base.py:121-165``): one fused
QKV product with columns ``[q | k | v]`` (``rapid_llm/modules/linear.py:236-271``), per-head
RMSNorm of q and k over the head dimension before the rotation (``:134-137``), rotation of q
and k, K/V written to the cache (``rapid_llm/modules/attention.py:126-138``), attention of
every query over its request's cached keys with ``kv_head = q_head // group`` and scale
``head_dim ** -0.5`` (``:62``), output projection without bias.

Every size is a constructor parameter; the window (0 = all keys) and whether q/k are
normed differ per layer if the specification says so, and so does ``qkv_bias`` (a bias on the
q, k and v projections, which this architecture does not have and its predecessor has; added in
float32 in the product's epilogue).  A layer that reads another entry's
cache (``cache.writes`` false) projects queries only.

Two more options serve architectures beside the reference's: a value size that differs from the
query/key size (``value_dim``), and an output gate (``gate="sigmoid"``: the concatenated heads are
multiplied by ``sigmoid(W_g x)`` before the output projection).  The kernels and the cache keep one
head size for keys and values, a multiple of 16: where the two sizes differ, or are no such multiple,
every head is laid out in the larger one rounded up, with zero weight rows (and zero columns of the
output projection) for the padding, which changes no score and no output; the q/k norm's mean is
taken over the true size.  ``names`` maps the tensors' default names to an architecture's own.

A third group of options serves mixers whose q, k and v pass a short causal convolution behind their
projections (``conv_width`` taps per channel, no activation; the last ``conv_width - 1`` projected rows of
a request are its state, ``state_need()``): the path from the projection to the cache then runs in float32
(convolution, rotation from frequencies instead of tables, ``unit_after_rotation``: q and k divided by
their root mean square after the rotation, without a weight).  ``softcap`` squashes a scaled score ``s``
to ``softcap * tanh(s / softcap)``; ``sink`` adds one learned term ``exp(sink[head])`` to every row's
denominator, without a key or a value; ``value_mix`` blends a layer's values with those of the first
such layer of the model for the same tokens (``"first"`` leaves them in a buffer of the step,
``"later"`` reads them: ``v <- (1 - m) v + m v_first`` with the learned number ``m``), and the blended
values are what is cached.

``qk_norm_over="row"`` norms q (and k) over the WHOLE projection at once, before it is split into heads:
``q <- q * rsqrt(mean(q^2) + eps) * w`` with the mean over all ``heads * head_dim`` entries and one weight per
entry; rotation angles then come from frequencies (position kind ``rotary_frequencies``), and norm, rotation and the
cache's store are one kernel.  ``cache_window`` says how many positions the layer's pages must keep when that differs
from its own ``window``: a layer whose cache another layer reads with a wider window (or without one: 0) keeps what
that reader needs.
"""

from __future__ import annotations

import numpy as np
import torch

from ..config.model_spec import PartSpec
from ..ops import gemm, kernels
from .base import (
    MATRIX, MIXERS, POSITION_ENCODINGS, VECTOR, CacheNeed, Mixer, StateNeed, StepPlanner, StepShape, TensorSpec,
)

DEFAULT_SMS = 148         # a B200's; planning on the host without a device (tests) assumes it
MAX_SPLITS = 16
CLUSTER_SPLITS = 16       # the largest thread-block cluster (beyond 8 the kernel asks for it)
TC_CHUNK_MIN_CTAS = 32    # measured: from here on the unsplit tcgen05 chunk kernel beats the split mma.sync tiles
TC_CHUNK_SHORT_CONTEXT = 1024   # ... and below this context it does so with any number of CTAs
MIN_KEYS_PER_SPLIT = 256
PADDING_FREE_BLOCKS = 32  # blocks of 128 keys from which a decode bucket's padding rows stop counting as clusters


# Clusters of the tcgen05 decode kernel a B200 runs at one time, by cluster size (one CTA per multiprocessor, a
# cluster inside one GPC); what planning on the host without a device assumes.
DEFAULT_DECODE_CLUSTERS = {1: 148, 2: 74, 3: 45, 4: 33, 5: 26, 6: 22, 7: 15, 8: 15, 9: 15, 10: 11,
                           11: 7, 12: 7, 13: 7, 14: 7, 15: 7, 16: 7}


def cluster_splits(tiles: int, clusters: dict[int, int]) -> int:
    """Key ranges per tile of a decode-only step on the tcgen05 decode kernel, which merges them inside one
    thread-block cluster: the largest cluster size of which ``tiles`` clusters still run at one time.  (Two
    requests of 8 kv heads are 16 tiles: 16 clusters of 8 would fill 128 multiprocessors, but only 15 such
    clusters fit the GPCs, so the sixteenth would wait for a whole round; 16 clusters of 6 run together.)"""
    best = 1
    for size, count in clusters.items():
        if size > best and size <= CLUSTER_SPLITS and count >= tiles:
            best = size
    return best


class AttentionItems(StepPlanner):
    """Cuts a step into the work items of the tensor-core attention kernels.

    Every entry's packed rows (token, head of the group) are tiled: entries of one token, or
    of at most 16 packed rows, into decode tiles of 16 rows; the others into chunk tiles.  When
    the tiles are too few to fill the GPU, each tile's key range is split into ``splits`` parts
    (the same number for the whole step): in a decode-only step a function of the number of entries and
    of a coarse class of the longest context, so that a captured decode graph replays the same launches at nearly every
    context length (where the tcgen05 decode kernel merges the parts inside a thread-block cluster: the
    largest cluster of which that many run at one time); bounded by the longest context otherwise.  Chunk tiles have 256 rows
    for the tcgen05 kernel, which takes head size 128, the usual page sizes and unsplit key
    ranges, and 64 rows for the mma.sync kernel otherwise.  The tcgen05 kernel is several times
    faster per key, so it also runs, unsplit, where a split would have been wanted, unless its
    CTAs are few and the context long (a few dozen prompt tokens behind thousands of cached ones).
    The longest tiles come first in the list, and the kernels' grids start them in that order.
    The reference picks its split size per launch in the same spirit
    (``rapid_llm/kernels/ops/attention/flashdecoding.py:43-112``).
    """

    def __init__(self, group: int, num_kv_heads: int, head_dim: int = 0, sms: int = DEFAULT_SMS,
                 decode_clusters: dict[int, int] | None = None, tensor_core: bool = True,
                 decode_tensor_core: bool = True) -> None:
        self.group, self.num_kv_heads, self.head_dim = int(group), int(num_kv_heads), int(head_dim)
        # decode_tensor_core False: the mixer's scores are squashed or its softmax has a sink, which the tcgen05 chunk
        # tiles and the mma.sync tiles compute, the tcgen05 decode tiles not; tensor_core False: mma.sync tiles only
        self.tensor_core = bool(tensor_core)
        self.decode_tensor_core = self.tensor_core and bool(decode_tensor_core)
        self.decode_clusters = dict(decode_clusters or DEFAULT_DECODE_CLUSTERS)
        # work items the kernels want in flight: two CTAs per multiprocessor, one in a decode-only
        # step, whose kernel keeps a whole multiprocessor's shared memory busy
        self.target_ctas, self.decode_target_ctas = 2 * int(sms), int(sms)
        self.key = ("attention_items", self.group, self.num_kv_heads, self.head_dim, int(sms),
                    tuple(sorted(self.decode_clusters.items())), self.tensor_core, self.decode_tensor_core)

    def capacity(self, max_tokens: int, max_entries: int) -> int:
        chunk_tiles = -(-max_tokens * self.group // kernels.CHUNK_TILE_ROWS) + max_entries
        decode_tiles = max_entries * -(-self.group // kernels.DECODE_TILE_ROWS)
        return 4 * (chunk_tiles + decode_tiles + 2 * self.target_ctas)

    def plan(self, shape: StepShape) -> dict:
        lengths = np.asarray(shape.lengths, dtype=np.int64)
        starts = np.asarray(shape.starts, dtype=np.int64)
        rows = lengths * self.group
        is_decode = (lengths == 1) | (rows <= kernels.DECODE_TILE_ROWS)
        tensor_core = self.tensor_core and kernels.attention_tc_takes(self.head_dim, shape.page_size)
        for chunk_rows in ((kernels.CHUNK_TILE_ROWS_TC, kernels.CHUNK_TILE_ROWS) if tensor_core else (kernels.CHUNK_TILE_ROWS,)):
            tile_rows = np.where(is_decode, kernels.DECODE_TILE_ROWS, chunk_rows)
            tiles = -(-rows // tile_rows)
            ctas = int(tiles.sum()) * self.num_kv_heads
            target = self.decode_target_ctas if shape.decode_only else self.target_ctas
            splits = max(1, min(MAX_SPLITS, target // max(ctas, 1)))
            if not shape.decode_only:
                longest = int((starts + lengths).max())
                splits = max(1, min(splits, longest // MIN_KEYS_PER_SPLIT))
            elif tensor_core and self.decode_tensor_core:
                # ... and no more key ranges than the longest context has blocks of keys, rounded down to a power
                # of two: a step's launch constants then change at a handful of context lengths only (the runner
                # keeps a captured graph per set of constants)
                blocks = max(1, -(-int((starts + lengths).max()) // kernels.DECODE_TC_KEYS))
                # On long contexts the padding rows of a decode bucket do not count: their clusters come last in the
                # grid, see one key each, and the round they add (a few microseconds) costs less than the real rows
                # gain from more CTAs (measured at batch 5 of a bucket of 8: 5 % slower at 1,024 tokens, 10 % faster at 32,000).
                counted = ctas
                if blocks >= PADDING_FREE_BLOCKS:
                    real = len(lengths) - int(shape.padding)
                    counted = max(1, int(tiles[:real].sum()) * self.num_kv_heads)
                splits = min(cluster_splits(counted, self.decode_clusters), 1 << (blocks.bit_length() - 1))
            if splits == 1 or chunk_rows == kernels.CHUNK_TILE_ROWS or bool(is_decode.all()):
                break
            # The tcgen05 chunk kernel does not split key ranges, but it is several times faster per
            # key than the mma.sync tiles: it runs unsplit unless it would leave most of the GPU
            # idle on a long context (a few dozen prompt tokens behind thousands of cached ones).
            chunk_ctas = int(tiles[~is_decode].sum()) * self.num_kv_heads
            if chunk_ctas >= TC_CHUNK_MIN_CTAS or longest <= TC_CHUNK_SHORT_CONTEXT:
                splits = 1
                break
        # Single tokens beside prompt portions that the tcgen05 kernel takes unsplit: their tiles get key ranges of
        # their own (merged inside that kernel's clusters), or a request far into its context would be walked by one
        # CTA per kv head while the step waits.
        decode_splits = splits
        if (tensor_core and self.decode_tensor_core and not shape.decode_only and splits == 1 and chunk_rows == kernels.CHUNK_TILE_ROWS_TC
                and bool(is_decode.any()) and not bool(is_decode.all())):
            decode_ctas = int(tiles[is_decode].sum()) * self.num_kv_heads
            blocks = max(1, -(-int((starts + lengths)[is_decode].max()) // kernels.DECODE_TC_KEYS))
            decode_splits = min(cluster_splits(decode_ctas, self.decode_clusters), 1 << (blocks.bit_length() - 1))
        entry = np.repeat(np.arange(len(lengths), dtype=np.int64), tiles)
        first = np.concatenate(([0], np.cumsum(tiles)[:-1]))
        tile_index = np.arange(int(tiles.sum()), dtype=np.int64) - np.repeat(first, tiles)
        row0 = tile_index * np.repeat(tile_rows, tiles)
        decode_tile = np.repeat(is_decode, tiles)
        # keys a tile has to walk: the tiles with the most go first, so that the last wave is short
        keys = np.repeat(starts, tiles) + (row0 + np.repeat(tile_rows, tiles)) // self.group

        def items(mask: np.ndarray, ranges: int) -> np.ndarray:
            order = np.flatnonzero(mask)
            order = order[np.argsort(-keys[order], kind="stable")]
            count = len(order)
            out = np.zeros((count * ranges, 4), dtype=np.int32)
            out[:, 0] = np.repeat(entry[order], ranges)
            out[:, 1] = np.repeat(row0[order], ranges)
            out[:, 2] = np.tile(np.arange(ranges, dtype=np.int32), count)
            return out

        decode_rows = int(np.minimum(rows[is_decode], kernels.DECODE_TILE_ROWS).max()) if is_decode.any() else 0
        return {"chunk_items": items(~decode_tile, splits), "decode_items": items(decode_tile, decode_splits),
                "splits": splits, "decode_splits": int(decode_splits), "decode_rows": decode_rows,
                "chunk_rows": int(chunk_rows)}


@MIXERS.register("gqa_attention")
class GQAAttention(Mixer):
    rides_norms = True

    def __init__(
        self,
        *,
        hidden_size: int,
        num_heads: int,
        num_kv_heads: int,
        head_dim: int,
        position: PartSpec,
        qk_norm: bool = False,
        qk_norm_eps: float = 1e-6,
        window: int = 0,
        scale: float | None = None,
        shares_cache: bool = False,
        qkv_bias: bool = False,
        value_dim: int | None = None,
        gate: str | None = None,
        names: dict[str, str] | None = None,
        conv_width: int = 0,
        unit_after_rotation: bool = False,
        softcap: float = 0.0,
        sink: bool = False,
        value_mix: str | None = None,
        qk_norm_over: str = "head",
        cache_window: int | None = None,
        dtype,
        device,
    ) -> None:
        super().__init__(dtype=dtype, device=device)
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads ({num_heads}) must be divisible by num_kv_heads ({num_kv_heads})")
        # true sizes of a query/key head and of a value head, and the one size both are laid out in
        self.qk_dim = int(head_dim)
        self.v_dim = int(value_dim) if value_dim is not None else self.qk_dim
        padded = -(-max(self.qk_dim, self.v_dim) // 16) * 16
        if min(self.qk_dim, self.v_dim) < 1 or padded > 256:
            raise ValueError(f"head sizes ({head_dim}, {value_dim}) must lie between 1 and 256")
        if gate not in (None, "sigmoid"):
            raise ValueError(f"unknown output gate {gate!r}")
        if qkv_bias and (padded != self.qk_dim or padded != self.v_dim):
            raise ValueError("padded head sizes are not combined with a bias")
        if qk_norm_over not in ("head", "row"):
            raise ValueError(f"qk_norm_over must be 'head' or 'row', got {qk_norm_over!r}")
        self.row_norm = bool(qk_norm) and qk_norm_over == "row"
        self.gate = gate
        # Options of mixers whose q, k and v pass a short convolution: they take the float32 path between the
        # projection and the cache (convolution, rotation, a weightless norm after it, blended values).
        self.conv_width = int(conv_width)
        self.unit_after_rotation = bool(unit_after_rotation)
        self.softcap, self.has_sink = float(softcap), bool(sink)
        if value_mix not in (None, "first", "later"):
            raise ValueError(f"value_mix must be 'first', 'later' or None, got {value_mix!r}")
        self.value_mix = value_mix
        self.float_prelude = self.conv_width > 0 or self.unit_after_rotation or value_mix is not None
        if self.float_prelude and (qk_norm or qkv_bias or shares_cache):
            raise ValueError("the convolution path has no weighted q/k norm, bias or shared cache")
        if self.row_norm and qkv_bias:
            raise ValueError("the norm over the whole projection is not combined with a bias")
        if not 0 <= self.conv_width <= 16 or self.softcap < 0:
            raise ValueError("conv_width must lie between 0 and 16, softcap must not be negative")
        self.names = {name: name for name in (
            "q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight", "q_proj.bias", "k_proj.bias",
            "v_proj.bias", "q_norm.weight", "k_norm.weight", "g_proj.weight", "q_conv", "k_conv", "v_conv", "sink",
            "value_mix")}
        self.names.update(names or {})
        self.hidden = int(hidden_size)
        self.hq, self.hkv, self.d = int(num_heads), int(num_kv_heads), padded
        self.qk_norm, self.eps = bool(qk_norm), float(qk_norm_eps)
        self.window = int(window)
        # what the pages must keep: the layer's own window, unless a reader of its cache needs more (0 = everything)
        self.cache_window = self.window if cache_window is None else int(cache_window)
        if self.cache_window < 0 or (self.cache_window and (self.window == 0 or self.cache_window < self.window)):
            raise ValueError(f"cache_window ({cache_window}) must cover the layer's own window ({window})")
        self.scale = float(scale) if scale is not None else self.qk_dim**-0.5
        self.shares_cache = bool(shares_cache)
        device = torch.device(device)
        sms = torch.cuda.get_device_properties(device).multi_processor_count if device.type == "cuda" else DEFAULT_SMS
        clusters = None
        if device.type == "cuda" and dtype == torch.bfloat16:
            clusters = kernels.attention_decode_clusters(self.d, device) or None
        plain_scores = not self.softcap and not self.has_sink
        self._items = AttentionItems(self.hq // self.hkv, self.hkv, self.d, sms, clusters if plain_scores else None,
                                     decode_tensor_core=plain_scores)
        self.position = POSITION_ENCODINGS.build(position, dtype=dtype, device=device)
        self.rotary_dim = int(position.params.get("rotary_dim", getattr(self.position, "rotary_dim", self.d)))

        kv_rows = 0 if self.shares_cache else 2 * self.hkv * self.d
        # With the norm over the whole projection the gate's rows lie behind q, k and v in ONE matrix: one product
        # reads the mixer's input once for all four, and the kernels behind it take rows wider than they use.
        self.gate_rides = bool(self.gate) and self.row_norm
        self.qkv_rows = self.hq * self.d + kv_rows
        self.qkv = self.new_storage((self.qkv_rows + (self.hq * self.d if self.gate_rides else 0), self.hidden), MATRIX)
        self.o = self.new_storage((self.hidden, self.hq * self.d), MATRIX)
        self.qkv_bias = self.new_storage((self.qkv_rows,), VECTOR) if qkv_bias else None
        # a norm over the whole projection has a weight per laid-out entry (zero in a head's padding)
        norm_rows = (self.hq * self.d, self.hkv * self.d) if self.row_norm else (self.d, self.d)
        self.q_norm = self.new_storage((norm_rows[0],), VECTOR) if self.qk_norm else None
        self.k_norm = self.new_storage((norm_rows[1],), VECTOR) if self.qk_norm and not self.shares_cache else None
        self.g = None
        if self.gate:
            self.g = self.qkv[self.qkv_rows :] if self.gate_rides else self.new_storage((self.hq * self.d, self.hidden), MATRIX)
        self.taps = self.new_storage((self.qkv_rows, self.conv_width), VECTOR) if self.conv_width > 0 else None
        self.sink = self.new_storage((self.hq,), VECTOR) if self.has_sink else None
        self.mix = self.new_storage((1,), VECTOR) if self.value_mix else None
        self.inv_freq = None
        if (self.float_prelude or self.row_norm) and self.rotary_dim > 0:
            if not hasattr(self.position, "inv_freq"):
                raise ValueError("this path computes its angles from frequencies: position kind 'rotary_frequencies'")
            self.inv_freq = self.position.inv_freq

    # -- needs ----------------------------------------------------------------- #
    def cache_need(self) -> CacheNeed | None:
        kind = "window" if self.cache_window > 0 else "full"
        return CacheNeed(kind, self.hkv, self.d, self.cache_window)

    def state_need(self) -> StateNeed | None:
        """The convolution's last ``conv_width - 1`` inputs (projected q, k, v) per request, float32."""
        if self.conv_width > 1:
            return StateNeed(((self.conv_width - 1) * self.qkv_rows,), torch.float32)
        return None

    def step_planner(self) -> StepPlanner | None:
        if self.dtype != torch.bfloat16:
            return None      # the float32 path runs the one-warp-per-row kernel: no work list
        return self._items

    # -- weights --------------------------------------------------------------- #
    def tensor_specs(self) -> dict[str, TensorSpec]:
        specs = {
            "q_proj.weight": TensorSpec((self.hq * self.qk_dim, self.hidden)),
            "o_proj.weight": TensorSpec((self.hidden, self.hq * self.v_dim)),
        }
        if not self.shares_cache:
            specs["k_proj.weight"] = TensorSpec((self.hkv * self.qk_dim, self.hidden))
            specs["v_proj.weight"] = TensorSpec((self.hkv * self.v_dim, self.hidden))
        if self.qkv_bias is not None:
            for name in ("q_proj", "k_proj", "v_proj")[: 1 if self.shares_cache else 3]:
                specs[f"{name}.bias"] = TensorSpec((specs[f"{name}.weight"].shape[0],), VECTOR)
        if self.qk_norm:
            q_count, k_count = (self.hq * self.qk_dim, self.hkv * self.qk_dim) if self.row_norm else (self.qk_dim, self.qk_dim)
            specs["q_norm.weight"] = TensorSpec((q_count,), VECTOR, init="ones_normal")
            if not self.shares_cache:
                specs["k_norm.weight"] = TensorSpec((k_count,), VECTOR, init="ones_normal")
        if self.gate:
            specs["g_proj.weight"] = TensorSpec((self.hq * self.v_dim, self.hidden))
        if self.conv_width > 0:
            specs["q_conv"] = TensorSpec((self.hq * self.qk_dim, self.conv_width), VECTOR)
            specs["k_conv"] = TensorSpec((self.hkv * self.qk_dim, self.conv_width), VECTOR)
            specs["v_conv"] = TensorSpec((self.hkv * self.v_dim, self.conv_width), VECTOR)
        if self.has_sink:
            specs["sink"] = TensorSpec((self.hq,), VECTOR)
        if self.value_mix:
            specs["value_mix"] = TensorSpec((), VECTOR)      # one number; the first such layer has it and does not use it
        return {self.names[name]: spec for name, spec in specs.items()}

    def _heads(self, rows: torch.Tensor, heads: int) -> torch.Tensor:
        """``rows [heads * d, n]`` as ``[heads, d, n]``: a head's true rows come first, padding after."""
        return rows.view(heads, self.d, rows.shape[1])

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        q_rows, kv_rows = self.hq * self.d, self.hkv * self.d
        name = {theirs: ours for ours, theirs in self.names.items()}.get(name, "")
        if name == "q_proj.weight":
            self._heads(self.qkv[:q_rows], self.hq)[:, : self.qk_dim].copy_(tensor.view(self.hq, self.qk_dim, -1))
        elif name == "k_proj.weight":
            self._heads(self.qkv[q_rows : q_rows + kv_rows], self.hkv)[:, : self.qk_dim].copy_(
                tensor.view(self.hkv, self.qk_dim, -1))
        elif name == "v_proj.weight":
            self._heads(self.qkv[q_rows + kv_rows : self.qkv_rows], self.hkv)[:, : self.v_dim].copy_(
                tensor.view(self.hkv, self.v_dim, -1))
        elif name == "o_proj.weight":
            self.o.view(self.hidden, self.hq, self.d)[:, :, : self.v_dim].copy_(
                tensor.view(self.hidden, self.hq, self.v_dim))
        elif name == "g_proj.weight":
            self._heads(self.g, self.hq)[:, : self.v_dim].copy_(tensor.view(self.hq, self.v_dim, -1))
        elif name == "q_proj.bias":
            self.qkv_bias[:q_rows].copy_(tensor.to(torch.float32))
        elif name == "k_proj.bias":
            self.qkv_bias[q_rows : q_rows + kv_rows].copy_(tensor.to(torch.float32))
        elif name == "v_proj.bias":
            self.qkv_bias[q_rows + kv_rows :].copy_(tensor.to(torch.float32))
        elif name == "q_conv":
            self._heads(self.taps[:q_rows], self.hq)[:, : self.qk_dim].copy_(tensor.to(torch.float32).view(self.hq, self.qk_dim, -1))
        elif name == "k_conv":
            self._heads(self.taps[q_rows : q_rows + kv_rows], self.hkv)[:, : self.qk_dim].copy_(
                tensor.to(torch.float32).view(self.hkv, self.qk_dim, -1))
        elif name == "v_conv":
            self._heads(self.taps[q_rows + kv_rows :], self.hkv)[:, : self.v_dim].copy_(
                tensor.to(torch.float32).view(self.hkv, self.v_dim, -1))
        elif name == "sink":
            self.sink.copy_(tensor.to(torch.float32))
        elif name == "value_mix":
            self.mix.copy_(tensor.to(torch.float32).reshape(1))
        elif name == "q_norm.weight" and self.row_norm:
            self.q_norm.view(self.hq, self.d)[:, : self.qk_dim].copy_(tensor.to(torch.float32).view(self.hq, self.qk_dim))
        elif name == "k_norm.weight" and self.row_norm:
            self.k_norm.view(self.hkv, self.d)[:, : self.qk_dim].copy_(tensor.to(torch.float32).view(self.hkv, self.qk_dim))
        elif name == "q_norm.weight":
            self.q_norm[: self.qk_dim].copy_(tensor.to(torch.float32))
        elif name == "k_norm.weight":
            self.k_norm[: self.qk_dim].copy_(tensor.to(torch.float32))
        else:
            raise KeyError(name)

    def parameter_bytes(self) -> int:
        total = (self.qkv.numel() + self.o.numel() + (0 if self.g is None or self.gate_rides else self.g.numel())) * self.qkv.element_size()
        for vector in (self.q_norm, self.k_norm, self.qkv_bias, self.taps, self.sink, self.mix):
            if vector is not None:
                total += vector.numel() * 4
        return total

    def workspace_elements_per_token(self) -> int:
        gate = 2 * self.hq * self.d if self.gate else 0
        return self.qkv.shape[0] + 2 * self.hq * self.d + self.hidden + gate      # qkv, q, attended, projected

    def uses_libraries(self) -> set[str]:
        found = {"recurrent"} if self.float_prelude else set()
        if self.dtype == torch.bfloat16:
            from ..ops.build import attention_library
            found |= {"gemm", attention_library(self.d)}
        return found

    # -- forward --------------------------------------------------------------- #
    def forward(self, x, batch, cache, then_norm=None):
        if cache.group is None or cache.pages is None:
            raise ValueError("attention needs a cache group; the engine did not give this layer one")
        if cache.writes == self.shares_cache:
            raise ValueError("the layer's cache role in the run order does not match shares_cache")
        group = batch.groups[cache.group]
        rows = x.shape[0]
        qkv = batch.workspace.get("attn_qkv", rows, self.qkv.shape[0], x.dtype)
        gemm.linear(x, self.qkv, qkv, batch.fault, bias=self.qkv_bias, defer=batch.defer_products)
        q = batch.workspace.get("attn_q", rows, self.hq * self.d, x.dtype)
        if self.float_prelude:
            self._float_prelude(qkv, q, batch, cache, group)
        elif self.row_norm:
            kernels.row_norm_rope_write(
                qkv, q, num_heads=self.hq, num_kv_heads=self.hkv, head_dim=self.d, q_weight=self.q_norm,
                k_weight=self.k_norm, q_count=self.hq * self.qk_dim, k_count=self.hkv * self.qk_dim,
                inv_freq=self.inv_freq, positions=batch.positions, eps=self.eps, fault=batch.fault,
                kv_dest=group.kv_dest if cache.writes else None, cache=cache.pages if cache.writes else None,
                page_size=group.page_size)
        else:
            self._norm_rope_write(qkv, q, batch, cache, group)
        attended = batch.workspace.get("attn_out", rows, self.hq * self.d, x.dtype)
        self.attend(q, cache.pages, attended, batch, group)
        if self.gate:
            if self.gate_rides:
                gate = qkv[:, self.qkv_rows :]          # the first product brought it along
            else:
                gate = batch.workspace.get("attn_gate", rows, self.hq * self.d, x.dtype)
                gemm.linear(x, self.g, gate, batch.fault)
            gated = batch.workspace.get("attn_gated", rows, self.hq * self.d, x.dtype)
            attended = kernels.sigmoid_gate(attended, gate, gated)
        out = batch.workspace.get("attn_proj", rows, self.hidden, x.dtype)
        return gemm.linear(attended, self.o, out, batch.fault, then_norm=then_norm, defer=batch.defer_products)

    def _float_prelude(self, qkv, q, batch, cache, group) -> None:
        """Projection -> short convolution (float32, the slot's tail before the step's rows) -> rotation ->
        weightless norm -> blended values -> q out, k and v into the pages."""
        rows, width = qkv.shape
        wide = batch.workspace.get("attn_conv", rows, width, torch.float32)
        if self.conv_width > 0:
            tail = cache.state
            if self.conv_width > 1 and (tail is None or tail.shape[1] != (self.conv_width - 1) * width):
                raise ValueError("the engine did not give this mixer the state row it asked for")
            if tail is None:
                tail = batch.workspace.get("attn_no_tail", 1, 0, torch.float32, min_rows=1)
            kernels.causal_conv_silu(qkv, self.taps, None, tail, wide, batch, act=False)
        else:
            kernels.activate_rows(qkv, wide, act=False)
        first, mode = None, 0
        if self.value_mix:
            # what the first blending layer's values were for this step's tokens: left there by it, read by the later ones
            first = batch.workspace.get("attn_first_values", rows, self.hkv * self.d, torch.float32)
            mode = 1 if self.value_mix == "first" else 2
        kernels.rope_unit_write(
            wide, q, num_heads=self.hq, num_kv_heads=self.hkv, head_dim=self.d, inv_freq=self.inv_freq,
            positions=batch.positions, kv_dest=group.kv_dest, cache=cache.pages, page_size=group.page_size,
            norm_size=self.qk_dim, unit=self.unit_after_rotation, eps=self.eps, fault=batch.fault,
            first=first, first_mode=mode, mix=self.mix,
        )

    def _norm_rope_write(self, qkv, q, batch, cache, group) -> None:
        cos, sin = self.position.tables()
        kernels.qk_norm_rope_write(
            qkv, q,
            num_heads=self.hq, num_kv_heads=self.hkv, head_dim=self.d, rotary_dim=self.rotary_dim,
            cos=cos, sin=sin, positions=batch.positions, eps=self.eps, fault=batch.fault,
            q_weight=self.q_norm, k_weight=self.k_norm,
            kv_dest=group.kv_dest if cache.writes else None,
            cache=cache.pages if cache.writes else None,
            page_size=group.page_size, norm_size=self.qk_dim,
        )

    def attend(self, q, pages, out, batch, group) -> None:
        if q.dtype == torch.bfloat16:
            plan = batch.extras[self._items.key]
            splits = plan["splits"]
            part_out = part_lse = None
            if splits > 1:
                rows = q.shape[0] * self.hq * splits
                part_out = batch.workspace.get("attn_part_out", rows, self.d, torch.float32, min_rows=rows)
                part_lse = batch.workspace.get("attn_part_lse", rows, 1, torch.float32, min_rows=rows)
            kernels.attention_mma(
                q, pages, out,
                chunk_items=plan["chunk_items"], decode_items=plan["decode_items"], splits=splits,
                part_out=part_out, part_lse=part_lse,
                cu_seqlens=batch.cu_seqlens, entry_start=batch.entry_start, entry_slot=batch.entry_slot,
                block_table=group.block_table, num_heads=self.hq, num_kv_heads=self.hkv, head_dim=self.d,
                window=self.window, scale=self.scale, fault=batch.fault, decode_rows=plan.get("decode_rows", 0),
                chunk_rows=plan.get("chunk_rows", kernels.CHUNK_TILE_ROWS),
                decode_splits=plan.get("decode_splits", 0), softcap=self.softcap, sink=self.sink,
            )
            return
        kernels.attention_generic(
            q, pages, out,
            positions=batch.positions, token_slot=batch.token_slot, block_table=group.block_table,
            num_heads=self.hq, num_kv_heads=self.hkv, head_dim=self.d,
            window=self.window, scale=self.scale, fault=batch.fault, softcap=self.softcap, sink=self.sink,
        )
