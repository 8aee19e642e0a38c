"""Norms with the residual add folded in: RMSNorm, and the layer norm with a mean and a bias.

``y = r * rsqrt(mean(r^2) + eps) * w`` with ``r = x`` or ``r = x + residual``; the weight
multiplies as ``w`` (with ``unit_offset`` the checkpoint stores ``w - 1``, a weight around zero, and one is added
when it is loaded).  Formula and the fused residual are the reference's
(``rapid_llm/kernels/ops/layernorm/skip_rmsnorm.py:41-48,51-85``; CPU twin
``rapid_llm/kernels/backend/cpu.py:18-29``); here the residual stream stays float32.
"""

from __future__ import annotations

import torch

from ..ops import gemm, kernels
from .base import NORMS, VECTOR, Norm, TensorSpec

FIRST, ADD, PLAIN = 0, 1, 2


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    reads_deferred = True       # it launches through ops.kernels, which runs queued products first

    def __init__(self, *, size: int, eps: float, dtype, device, name: str = "weight", unit_offset: bool = False) -> None:
        super().__init__(dtype=dtype, device=device)
        self.size = int(size)
        self.eps = float(eps)
        self.name = name          # the tensor's name after the part's prefix (may be empty)
        self.unit_offset = bool(unit_offset)
        self.weight = self.new_storage((self.size,), VECTOR)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.size,), VECTOR, init="normal" if self.unit_offset else "ones_normal")}

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        if name != self.name:
            raise KeyError(name)
        self.weight.copy_(tensor.to(torch.float32))
        if self.unit_offset:
            self.weight.add_(1.0)        # float32: the sum of one and a 16-bit number is exact enough to be the weight

    def parameter_bytes(self) -> int:
        return self.weight.numel() * 4

    def workspace_elements_per_token(self) -> int:
        return self.size

    def following(self, residual: torch.Tensor, batch) -> gemm.FollowingNorm | None:
        """This norm of ``residual + (a product's result)``, as an offer to that product."""
        if self.dtype != torch.bfloat16 or residual is None:
            return None
        return gemm.FollowingNorm(residual, self.weight, self.eps, batch.workspace)

    def join(self, y, residual, batch, name="stream_rows"):
        """The norm on a sublayer's output: ``residual += norm(y)`` in float32; returns the new stream in the
        engine's dtype (what the next sublayer reads)."""
        out = batch.workspace.get(name, y.shape[0], self.size, y.dtype)
        return kernels.join_rmsnorm(y, residual, self.weight, out, self.eps)

    def join_then(self, y, residual, next_norm: "RMSNorm", batch, name="normed"):
        """:meth:`join`, and ``next_norm`` of the new stream in the same pass: returns that norm's result."""
        out = batch.workspace.get(name, y.shape[0], self.size, y.dtype)
        return kernels.join_then_rmsnorm(y, residual, self.weight, next_norm.weight, out, self.eps)

    def of_stream(self, residual, batch, *, row_index=None, name="normed"):
        """The norm of the float32 stream itself (rows picked by ``row_index``), in the engine's dtype."""
        rows = residual.shape[0] if row_index is None else row_index.numel()
        out = batch.workspace.get(name, rows, self.size, self.dtype, min_rows=None if row_index is None else 64)
        return kernels.stream_rmsnorm(residual, self.weight, out, self.eps, row_index)

    def forward(self, x, residual, batch, *, mode, write_residual, row_index=None, name="normed", addend=None):
        """Norm of ``x`` (``FIRST``/``PLAIN``) or of ``x + residual`` (``ADD``).

        With ``write_residual`` the float32 sum is stored into ``residual``.  ``row_index``
        selects input rows (the rows whose logits are wanted, for the final norm).  ``addend``
        (:class:`~rapid_llm_b200.parts.base.StreamAddend`) is added to the sum before it is stored.
        """
        rows = x.shape[0] if row_index is None else row_index.numel()
        out = batch.workspace.get(name, rows, self.size, x.dtype, min_rows=None if row_index is None else 64)
        return kernels.add_rmsnorm(
            x, residual, self.weight, out, self.eps,
            mode=mode, write_residual=write_residual, row_index=row_index,
            extra_rows=None if addend is None else addend.rows,
            extra_vector=None if addend is None else addend.vector,
        )


@NORMS.register("layernorm")
class LayerNorm(Norm):
    """``n = (r - mean r) / sqrt(var r + eps) * weight + bias``, the variance being the mean of the squared deviations;
    float32 statistics, float32 weight and bias.  ``bias_suffix`` names the bias after the weight's own name
    (``None``: no bias).  ``gain`` multiplies what the norm hands on (not what it stores in the stream): a model
    whose head scales its logits by a constant gives that constant to its last norm, since
    ``(W n) * gain = W (n * gain)`` and the product's input is rounded once either way.

    Beside the interface of every norm (``forward`` with the modes of :mod:`parts.norm`) it has the two forms an
    arrangement with the norm BEHIND the sum needs: :meth:`post_join` (``stream <- norm(alpha * stream + y)``) and
    :meth:`of_stream`."""

    reads_deferred = True

    def __init__(self, *, size: int, eps: float, dtype, device, name: str = "weight", bias_suffix: str | None = ".b",
                 gain: float = 1.0) -> None:
        super().__init__(dtype=dtype, device=device)
        self.size, self.eps, self.gain = int(size), float(eps), float(gain)
        self.name = name
        self.bias_name = None if bias_suffix is None else name + bias_suffix
        self.weight = self.new_storage((self.size,), VECTOR)
        self.bias = None if self.bias_name is None else self.new_storage((self.size,), VECTOR)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        specs = {self.name: TensorSpec((self.size,), VECTOR, init="ones_normal")}
        if self.bias_name is not None:
            specs[self.bias_name] = TensorSpec((self.size,), VECTOR)
        return specs

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        if name == self.name:
            self.weight.copy_(tensor.to(torch.float32))
        elif name == self.bias_name:
            self.bias.copy_(tensor.to(torch.float32))
        else:
            raise KeyError(name)

    def parameter_bytes(self) -> int:
        return self.weight.numel() * 4 * (1 if self.bias is None else 2)

    def workspace_elements_per_token(self) -> int:
        return self.size

    def post_join(self, y, residual, alpha: float, batch, name="stream_rows"):
        """``residual <- norm(alpha * residual + y)`` in float32, in place; returns the new stream in the engine's
        dtype (what the next sublayer reads)."""
        out = batch.workspace.get(name, y.shape[0], self.size, y.dtype)
        return kernels.layernorm(y, residual, self.weight, self.bias, out, self.eps, residual_scale=alpha,
                                 store=kernels.LAYERNORM_STORE_NORM, gain=self.gain)

    def of_stream(self, residual, batch, *, row_index=None, name="normed"):
        """The norm of the float32 stream itself (rows picked by ``row_index``), in the engine's dtype."""
        rows = residual.shape[0] if row_index is None else row_index.numel()
        out = batch.workspace.get(name, rows, self.size, self.dtype, min_rows=None if row_index is None else 64)
        return kernels.layernorm(None, residual, self.weight, self.bias, out, self.eps, row_index=row_index, gain=self.gain)

    def forward(self, x, residual, batch, *, mode, write_residual, row_index=None, name="normed", addend=None):
        if addend is not None:
            raise ValueError("this norm takes no addend")
        rows = x.shape[0] if row_index is None else row_index.numel()
        out = batch.workspace.get(name, rows, self.size, x.dtype, min_rows=None if row_index is None else 64)
        if mode == ADD:
            store = kernels.LAYERNORM_STORE_SUM if write_residual else kernels.LAYERNORM_KEEP
            return kernels.layernorm(x, residual, self.weight, self.bias, out, self.eps, store=store, row_index=row_index,
                                     gain=self.gain)
        if mode == FIRST and write_residual:
            kernels.to_float(x, residual)
        return kernels.layernorm(x, None, self.weight, self.bias, out, self.eps, row_index=row_index, gain=self.gain)
