"""RMSNorm fused with the residual sum (reference ``src/llmserve/model.py:14-23``)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import Norm, ResidualStream, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """params: ``eps``; ``offset`` (default 0): the stored weight is an offset from this number, y = x_hat *
    (offset + w); ``weight_name`` (default "weight"): the tensor's name after the part's prefix.

    y = (x * rsqrt(mean(x^2) + eps)) * weight, where x is the float32 residual after the pending branch output has
    been added to it.  When the stream keeps several copies of the residual, or scales what a branch adds
    (``ResidualStream``), the same kernel launch mixes the copies, adds the scaled output and reads x as the
    weighted sum of the copies."""

    graph_safe = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        self.eps = float(params["eps"])
        offset = float(params.get("offset", 0.0))
        weight = weights[params.get("weight_name", "weight")].to(torch.float32)
        self.weight = (weight + offset if offset else weight).contiguous()

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        kind = "bias" if float(params.get("offset", 0.0)) else "norm"   # an offset weight is drawn around zero
        return {params.get("weight_name", "weight"): TensorSpec((hidden_size,), kind)}

    def forward(self, stream: ResidualStream, rows: torch.Tensor | None = None) -> torch.Tensor:
        hidden = self.weight.shape[0]
        n_rows = stream.residual.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n_rows, hidden), dtype=self.ctx.dtype, device=stream.residual.device)
        if stream.plain:
            ops.add_rmsnorm(stream.residual, stream.delta, self.weight, self.eps, out, rows=rows,
                            write_residual=rows is None)
        else:
            ops.streams_update_rmsnorm(stream.residual, stream.copies, stream.delta, stream.delta_scale,
                                       stream.delta_mult, stream.mix, stream.write, stream.read, self.weight,
                                       self.eps, out, rows=rows, write_back=rows is None)
        if rows is None:
            stream.delta = None
        return out


@register_norm("rmsnorm_after_sum")
class RMSNormAfterSum(Norm):
    """params: ``eps``, ``residual_mult`` (alpha), ``weight_name`` (default "weight").

    The norm of a layer that normalises after the sum: x <- (alpha x + y + b) / sqrt(mean((alpha x + y + b)^2) + eps) * w,
    where y is the pending branch output and b the bias that came with it (and c_t x_t, when the branch left a factor
    per row on its own input, ``stream.delta_row_scale``).  The result replaces the float32 residual
    and, rounded, ``stream.hidden``, which the next branch reads; the rounded rows are returned."""

    graph_safe = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        self.eps = float(params["eps"])
        self.alpha = float(params.get("residual_mult", 1.0))
        self.weight = weights[params.get("weight_name", "weight")].to(torch.float32).contiguous()

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        return {params.get("weight_name", "weight"): TensorSpec((hidden_size,), "norm")}

    def forward(self, stream: ResidualStream, rows: torch.Tensor | None = None) -> torch.Tensor:
        if rows is not None or not stream.plain:
            raise ops.KernelError("rmsnorm_after_sum: the norm runs over all rows of one copy of the residual")
        copy = stream.hidden if stream.hidden is not stream.residual else None
        ops.scaled_add_rmsnorm(stream.residual, stream.delta, stream.delta_bias, stream.delta_row_scale, self.alpha,
                               self.weight, self.eps, copy)
        stream.delta = stream.delta_bias = stream.delta_row_scale = None
        return stream.hidden


@register_norm("dynamic_tanh")
class DynamicTanh(Norm):
    """params: ``weight_name`` (default "weight"), ``bias_name`` (default: the weight's name + ".b"), ``alpha_name``
    (default: the weight's name + ".alpha").

    A norm without statistics: y = tanh(alpha x) * w + b with a learned scalar alpha, elementwise, in float32.
    As a layer's norm it adds the pending branch output to the float32 residual first; when the stream says that
    the output passes a norm of its own before it is added (``stream.delta_norm``, a norm of this kind: a layer that
    norms before and after each branch), the same launch applies that too:
        residual += after(delta);   returns before(residual)."""

    graph_safe = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        weight, bias, alpha = self._names(params)
        self.weight = weights[weight].to(torch.float32).contiguous()
        self.bias = weights[bias].to(torch.float32).contiguous()
        self.alpha = weights[alpha].to(torch.float32).reshape(1).contiguous()

    @staticmethod
    def _names(params) -> tuple[str, str, str]:
        weight = params.get("weight_name", "weight")
        return weight, params.get("bias_name", weight + ".b"), params.get("alpha_name", weight + ".alpha")

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        weight, bias, alpha = cls._names(params)
        return {weight: TensorSpec((hidden_size,), "norm"), bias: TensorSpec((hidden_size,), "bias"),
                alpha: TensorSpec((), "norm")}

    @property
    def triple(self):
        return self.alpha, self.weight, self.bias

    def forward(self, stream: ResidualStream, rows: torch.Tensor | None = None) -> torch.Tensor:
        if not stream.plain:
            raise ops.KernelError("dynamic_tanh: one copy of the residual, branch outputs added as they are")
        after = stream.delta_norm
        if after is not None and not isinstance(after, DynamicTanh):
            raise ops.KernelError("dynamic_tanh: the norm of a branch's output must be of the same kind")
        hidden = self.weight.shape[0]
        n_rows = stream.residual.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n_rows, hidden), dtype=self.ctx.dtype, device=stream.residual.device)
        ops.tanh_norm(stream.residual, stream.delta, after.triple if after is not None and stream.delta is not None else None,
                      self.triple, out, rows=rows, write_residual=rows is None)
        if rows is None:
            stream.delta = stream.delta_norm = None
        return out
