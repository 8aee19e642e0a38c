"""Arrangements of a layer's parts: the pre-norm residual block, and the block with norms on the outputs.

``h' = h + Mixer(Norm(h)); h'' = h' + FeedForward(Norm(h'))`` with each add deferred into
the next norm, so a pair ``(x, residual)`` is threaded through the stack
(``rapid_llm/models/base.py:231-266,372-375``): ``residual`` is ``None`` entering the first
layer; the norm kernel forms ``x + residual`` in float32, stores it back and norms it.

Where the parts on both sides of a norm can take it along (``rides_norms``: the product before
it adds to the residual and applies the norm's weight, the product after it applies the row's
scale), the norm is offered to them and no norm kernel runs; the parts decide step by step
whether they accept (small steps in bfloat16 do).

``outnorm`` (:class:`OutputNormBlock`): ``h' = h + Norm(Mixer(h)); h'' = h' + Norm(FeedForward(h'))``.  The
sublayers read the stream itself; the stream is the float32 ``residual`` and ``x`` its rounding.

``sandwich`` (:class:`SandwichBlock`): a norm on both sides of each sublayer,
``h' = h + NormB(Mixer(NormA(h))); h'' = h' + NormD(FeedForward(NormC(h')))``, the stream float32 in ``residual``.

``postnorm`` (:class:`PostNormBlock`): the norm behind the sum, ``h' = Norm(alpha h + Mixer(h));
h'' = Norm(alpha h' + FeedForward(h'))``; the stream is the norm's own result, float32 in ``residual``.
"""

from __future__ import annotations

import torch

from ..config.model_spec import LayerSpec
from ..ops import gemm, kernels
from ..ops.gemm import ScaledRows
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, TensorSpec
from .norm import ADD, FIRST


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    """``names`` maps the roles to their checkpoint sub-prefixes."""

    NAMES = {
        "mixer_norm": "input_layernorm.",
        "mixer": "self_attn.",
        "feed_forward_norm": "post_attention_layernorm.",
        "feed_forward": "mlp.",
    }

    def __init__(self, *, layer: LayerSpec, dtype, device, names: dict[str, str] | None = None) -> None:
        super().__init__(dtype=dtype, device=device)
        self.names = dict(self.NAMES)
        self.names.update(names or layer.names or {})
        self.mixer_norm = NORMS.build(layer.norm, dtype=dtype, device=device)
        self.mixer = MIXERS.build(layer.mixer, dtype=dtype, device=device)
        # a layer without a feed-forward is the mixer's half alone: x + Mixer(Norm(x))
        self.feed_forward_norm = self.feed_forward = None
        if layer.feed_forward is not None:
            self.feed_forward_norm = NORMS.build(layer.norm, dtype=dtype, device=device)
            self.feed_forward = FEED_FORWARDS.build(layer.feed_forward, dtype=dtype, device=device)

    def _children(self):
        children = [(self.names["mixer_norm"], self.mixer_norm), (self.names["mixer"], self.mixer)]
        if self.feed_forward is not None:
            children += [(self.names["feed_forward_norm"], self.feed_forward_norm),
                         (self.names["feed_forward"], self.feed_forward)]
        return tuple(children)

    def cache_need(self):
        return self.mixer.cache_need()

    def state_need(self):
        return self.mixer.state_need()

    def step_planners(self):
        planner = self.mixer.step_planner()
        return [] if planner is None else [planner]

    def uses_libraries(self) -> set[str]:
        found: set[str] = set()
        for _, part in self._children():
            found |= part.uses_libraries()
        return found

    def tensor_specs(self) -> dict[str, TensorSpec]:
        specs = {}
        for prefix, part in self._children():
            for name, spec in part.tensor_specs().items():
                specs[prefix + name] = spec
        return specs

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        for prefix, part in self._children():
            if name.startswith(prefix):
                part.load_tensor(name[len(prefix):], tensor)
                return
        raise KeyError(name)

    def finalize(self, loaded: set[str]) -> None:
        for prefix, part in self._children():
            part.finalize({name[len(prefix):] for name in loaded if name.startswith(prefix)})

    def parameter_bytes(self) -> int:
        return sum(part.parameter_bytes() for _, part in self._children())

    def workspace_elements_per_token(self) -> int:
        return sum(part.workspace_elements_per_token() for _, part in self._children())

    def leading_norm(self):
        return self.mixer_norm if self.mixer.rides_norms else None

    def forward(self, x, residual, batch, cache, then_norm=None, addend=None):
        """``(x, residual)`` in, ``(x, residual)`` out; ``residual`` is ``None`` for the first layer."""
        if not self.mixer_norm.reads_deferred:
            gemm.flush()        # a norm that is no kernel of ops.kernels reads finished results only
        extra = {} if addend is None else {"addend": addend}
        if isinstance(x, ScaledRows):
            if addend is not None:
                raise ValueError("a norm that rode on the product before it cannot take an addend")
            normed = x          # the block before took this block's first norm along
        elif residual is None:
            residual = batch.workspace.get("residual", x.shape[0], x.shape[1], torch.float32)
            normed = self.mixer_norm.forward(x, residual, batch, mode=FIRST, write_residual=True, **extra)
        else:
            normed = self.mixer_norm.forward(x, residual, batch, mode=ADD, write_residual=True, **extra)
        if self.feed_forward is None:
            if self.mixer.rides_norms:
                offer = then_norm.following(residual, batch) if then_norm is not None else None
                return self.mixer.forward(normed, batch, cache, then_norm=offer), residual
            return self.mixer.forward(normed, batch, cache), residual
        if self.mixer.rides_norms:
            offer = self.feed_forward_norm.following(residual, batch) if self.feed_forward.rides_norms else None
            mixed = self.mixer.forward(normed, batch, cache, then_norm=offer)
        else:
            mixed = self.mixer.forward(normed, batch, cache)
        if isinstance(mixed, ScaledRows):
            normed = mixed
        else:
            if not self.feed_forward_norm.reads_deferred:
                gemm.flush()
            normed = self.feed_forward_norm.forward(mixed, residual, batch, mode=ADD, write_residual=True)
        if self.feed_forward.rides_norms:
            offer = then_norm.following(residual, batch) if then_norm is not None else None
            return self.feed_forward.forward(normed, batch, then_norm=offer), residual
        return self.feed_forward.forward(normed, batch), residual


@BLOCKS.register("outnorm")
class OutputNormBlock(PreNormBlock):
    """Norms on the sublayers' outputs: ``h <- h + Norm(Mixer(h)); h <- h + Norm(FeedForward(h))``.

    The sublayers read the stream itself.  The stream lives in ``residual`` (float32) and every norm adds
    its result there (one kernel: norm, add, store, and the sum's rounding to the engine's dtype, which is
    what the next sublayer reads); ``x`` is that rounding.  No norm stands in front of a product, so none
    rides on one."""

    stream_in_residual = True

    def leading_norm(self):
        return None

    def forward(self, x, residual, batch, cache, then_norm=None, addend=None):
        if addend is not None or isinstance(x, ScaledRows):
            raise ValueError("this arrangement takes plain rows and no addend")
        if residual is None:       # the embedding did not open the stream: it starts as x
            residual = batch.workspace.get("residual", x.shape[0], x.shape[1], torch.float32)
            kernels.to_float(x, residual)
        mixed = self.mixer.forward(x, batch, cache)
        gemm.flush()
        x = self.mixer_norm.join(mixed, residual, batch)
        if self.feed_forward is not None:
            wide = self.feed_forward.forward(x, batch)
            gemm.flush()
            x = self.feed_forward_norm.join(wide, residual, batch)
        return x, residual


class NormedStream:
    """Rows that are already the leading norm's result of the stream: what a :class:`SandwichBlock` hands the next
    one when the norm on its last sublayer's output took that block's first norm along."""

    def __init__(self, rows: torch.Tensor) -> None:
        self.rows = rows


class _LeadingOffer:
    """A :class:`SandwichBlock`'s first norm as the block before it sees it: only another sandwich block takes it
    along (``norm``); as a norm that rides on a product it declines."""

    def __init__(self, norm) -> None:
        self.norm = norm

    def following(self, residual, batch):
        return None


@BLOCKS.register("sandwich")
class SandwichBlock(PreNormBlock):
    """A norm in front of and behind each sublayer: ``h <- h + NormB(Mixer(NormA(h)))``, then
    ``h <- h + NormD(FeedForward(NormC(h)))``.  The stream lives in ``residual`` (float32, opened by the embedding
    or from ``x``); the norm behind a sublayer adds its result there and, in the same kernel, forms the norm in front
    of the next sublayer (of this block, or of the next block if that is a sandwich block too)."""

    stream_in_residual = True
    NAMES = {"mixer_norm": "norm1", "mixer_out_norm": "norm1b", "mixer": "mix.", "feed_forward_norm": "norm2",
             "feed_forward_out_norm": "norm2b", "feed_forward": "mlp."}

    def __init__(self, *, layer: LayerSpec, dtype, device, names: dict[str, str] | None = None) -> None:
        super().__init__(layer=layer, dtype=dtype, device=device, names=names)
        self.mixer_out_norm = NORMS.build(layer.norm, dtype=dtype, device=device)
        self.feed_forward_out_norm = None
        if self.feed_forward is not None:
            self.feed_forward_out_norm = NORMS.build(layer.norm, dtype=dtype, device=device)
        for norm in (self.mixer_norm, self.mixer_out_norm, self.feed_forward_norm, self.feed_forward_out_norm):
            if norm is not None and not hasattr(norm, "join_then"):
                raise ValueError("the sandwich arrangement needs norms that can join the stream (kind 'rmsnorm')")

    def _children(self):
        children = [(self.names["mixer_norm"], self.mixer_norm), (self.names["mixer_out_norm"], self.mixer_out_norm),
                    (self.names["mixer"], self.mixer)]
        if self.feed_forward is not None:
            children += [(self.names["feed_forward_norm"], self.feed_forward_norm),
                         (self.names["feed_forward_out_norm"], self.feed_forward_out_norm),
                         (self.names["feed_forward"], self.feed_forward)]
        # the longest prefix first: "norm1b" must not be taken for "norm1" followed by "b"
        return tuple(sorted(children, key=lambda child: -len(child[0])))

    def leading_norm(self):
        return _LeadingOffer(self.mixer_norm)

    def _close(self, y, norm, residual, batch, then_norm):
        """The norm behind a sublayer; with ``then_norm`` (an RMS norm) that norm of the new stream comes back."""
        gemm.flush()
        if then_norm is not None:
            return NormedStream(norm.join_then(y, residual, then_norm, batch))
        return norm.join(y, residual, batch)

    def forward(self, x, residual, batch, cache, then_norm=None, addend=None):
        if addend is not None or isinstance(x, ScaledRows):
            raise ValueError("this arrangement takes plain rows and no addend")
        after = then_norm.norm if isinstance(then_norm, _LeadingOffer) else None
        if isinstance(x, NormedStream):
            normed = x.rows
        else:
            if residual is None:       # the embedding did not open the stream: it starts as x
                residual = batch.workspace.get("residual", x.shape[0], x.shape[1], torch.float32)
                kernels.to_float(x, residual)
            normed = self.mixer_norm.of_stream(residual, batch)
        mixed = self.mixer.forward(normed, batch, cache)
        if self.feed_forward is None:
            return self._close(mixed, self.mixer_out_norm, residual, batch, after), residual
        normed = self._close(mixed, self.mixer_out_norm, residual, batch, self.feed_forward_norm).rows
        wide = self.feed_forward.forward(normed, batch)
        return self._close(wide, self.feed_forward_out_norm, residual, batch, after), residual


class ClosingNorm:
    """The norm behind a sum, ``stream <- norm(alpha * stream + y)``, as a :class:`PostNormBlock` offers it to a
    feed-forward whose last kernel can take it along (class flag ``closes_sums``)."""

    def __init__(self, norm, residual: torch.Tensor, alpha: float) -> None:
        self.norm, self.residual, self.alpha = norm, residual, alpha


@BLOCKS.register("postnorm")
class PostNormBlock(PreNormBlock):
    """The norm behind the sum: ``h <- Norm1(alpha * h + Mixer(h)); h <- Norm2(alpha * h + FeedForward(h))``.

    The sublayers read the stream itself.  The stream lives in ``residual`` (float32): one kernel forms
    ``alpha * stream + y`` for a sublayer's result ``y``, norms it, stores the norm as the stream's new value and
    writes its rounding to the engine's dtype, which is what the next sublayer reads; ``x`` is that rounding.
    ``alpha`` comes from the layer's ``arrangement_params`` (default 1).  The norm kind must offer ``post_join``
    (``layernorm``)."""

    stream_in_residual = True
    NAMES = {"mixer_norm": "norm1", "mixer": "mix.", "feed_forward_norm": "norm2", "feed_forward": "mlp."}

    def __init__(self, *, layer: LayerSpec, dtype, device, names: dict[str, str] | None = None) -> None:
        super().__init__(layer=layer, dtype=dtype, device=device, names=names)
        self.alpha = float((layer.arrangement_params or {}).get("alpha", 1.0))
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if norm is not None and not hasattr(norm, "post_join"):
                raise ValueError("the postnorm arrangement needs norms that can close a sum (kind 'layernorm')")
        self._closes = (self.feed_forward is not None and getattr(self.feed_forward, "closes_sums", False)
                        and getattr(self.feed_forward, "shared", None) is None and getattr(self.feed_forward_norm, "gain", 1.0) == 1.0)

    def leading_norm(self):
        return None

    def forward(self, x, residual, batch, cache, then_norm=None, addend=None):
        if addend is not None or isinstance(x, ScaledRows):
            raise ValueError("this arrangement takes plain rows and no addend")
        if residual is None:       # the embedding did not open the stream: it starts as x
            residual = batch.workspace.get("residual", x.shape[0], x.shape[1], torch.float32)
            kernels.to_float(x, residual)
        mixed = self.mixer.forward(x, batch, cache)
        gemm.flush()
        x = self.mixer_norm.post_join(mixed, residual, self.alpha, batch)
        if self.feed_forward is not None:
            if self._closes:      # the feed-forward's last kernel takes the sum with the stream and its norm along
                x = self.feed_forward.forward(x, batch, closing=ClosingNorm(self.feed_forward_norm, residual, self.alpha))
            else:
                wide = self.feed_forward.forward(x, batch)
                gemm.flush()
                x = self.feed_forward_norm.post_join(wide, residual, self.alpha, batch)
        return x, residual
