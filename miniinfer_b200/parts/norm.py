"""RMSNorm and layer norm, each with the residual add in front of it (one kernel).

Formula of the reference: ``w * x * rsqrt(mean(x^2) + eps)`` in float32
(miniinfer/layers/layernorm.py:27-32), fused with the residual add as in its Triton kernel
(kernels/triton/rms_norm.py:66-108).  The residual stream here is float32.
"""

from __future__ import annotations

from typing import Dict, Optional, Tuple, Union

import torch

from ..kernels import ops
from .base import Norm, ParamSpec, whole


Delta = Union[None, torch.Tensor, Tuple[Optional[torch.Tensor], ...]]


def split_delta(delta: Delta) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
  """What is pending for the residual stream as (first, second): a block whose mixer and feed-forward read the same
  normalised rows leaves two outputs to be added, the usual block one."""
  if delta is None or isinstance(delta, torch.Tensor):
    return delta, None
  parts = [d for d in delta if d is not None]
  if len(parts) > 2:
    raise ValueError("at most two outputs can be pending for the residual stream")
  return (parts + [None, None])[0], (parts + [None, None])[1]


class RMSNorm(Norm):
  """``(offset + w) * x / sqrt(mean(x^2) + eps)`` in float32, the residual add (of one or two pending outputs) in front
  of it in the same kernel.  ``offset``: 0 for a weight stored as it is applied, 1 for a weight stored around zero (the
  sum is made once, in float32, when the weights are bound).  ``gain``: a constant the normed rows are multiplied with (a
  model's logit scale on its final norm), folded into the applied weight the same way.  ``weight_name``: the file tensor
  (default ``<name>.weight``).

  ``add_scaled`` is the norm for blocks that norm a sublayer's OUTPUT: ``resid += mult * norm(y)``."""

  def __init__(self, name: str, dim: int, eps: float, offset: float = 0.0, weight_name: Optional[str] = None, gain: float = 1.0):
    super().__init__(name)
    self.dim = dim
    self.eps = float(eps)
    self.offset = float(offset)
    self.gain = float(gain)
    self.weight_name = weight_name or f"{name}.weight"

  def param_specs(self) -> Dict[str, ParamSpec]:
    return {"weight": ParamSpec((self.dim,), "vector", [whole(self.weight_name, (self.dim,))],
                                init="ones_noise" if self.offset == 0.0 else "normal")}

  def bind(self, params) -> None:
    super().bind(params)
    if (self.offset != 0.0 or self.gain != 1.0) and "weight" in params:
      self.weight = (params["weight"] + self.offset) * self.gain          # the stored tensor stays as the file has it

  def add_scaled(self, resid: torch.Tensor, y: torch.Tensor, mult: float, ctx, copy: bool = False,
                 keep: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """``resid += mult * norm(y)`` in float32, in place.  ``copy``: the new rows are also returned in the compute dtype (the
    residual rows themselves when that is float32).  ``keep``: per-request state rows that receive, for the last new token of
    every item, the residual row as it was before the addition."""
    out = None
    if copy:
      out = resid if ctx.dtype == torch.float32 else ctx.ws.buffer("resid_rows", (resid.shape[0], self.dim), ctx.dtype)
    ops.norm_scaled_add(resid, y, self.weight, self.eps, mult, ctx, copy=out if out is not resid else None, keep=keep)
    return out

  def as_rms(self):
    return self.weight, self.eps

  def add_norm(self, resid: torch.Tensor, delta: Delta, ctx) -> torch.Tensor:
    first, second = split_delta(delta)
    out = ctx.ws.buffer("normed", (resid.shape[0], self.dim), ctx.dtype)
    if second is not None:
      ops.add_rmsnorm_pair(out, None, resid, first, second, self.weight, None, self.eps, None, True)
    else:
      ops.add_rmsnorm(out, resid, first, self.weight, self.eps, None, True)
    return out

  def add_norm_pair(self, resid: torch.Tensor, delta: Delta, other: "RMSNorm", ctx) -> Tuple[torch.Tensor, torch.Tensor]:
    """What ``add_norm`` does, and the rows normalised with ``other``'s weight as well: two norms of the same rows share
    the root mean square (``other`` must be an RMSNorm of the same size and eps)."""
    if not isinstance(other, RMSNorm) or other.dim != self.dim or other.eps != self.eps:
      raise ValueError(f"{self.name}: a pair of norms must be two RMS norms of one size and eps")
    first, second = split_delta(delta)
    out = ctx.ws.buffer("normed", (resid.shape[0], self.dim), ctx.dtype)
    out2 = ctx.ws.buffer("normed_second", (resid.shape[0], self.dim), ctx.dtype)
    ops.add_rmsnorm_pair(out, out2, resid, first, second, self.weight, other.weight, self.eps, None, True)
    return out, out2

  def norm_rows(self, resid: torch.Tensor, delta: Delta, rows: torch.Tensor, ctx) -> torch.Tensor:
    first, second = split_delta(delta)
    out = ctx.ws.buffer("normed_rows", (rows.shape[0], self.dim), ctx.dtype)
    if second is not None:
      ops.add_rmsnorm_pair(out, None, resid, first, second, self.weight, None, self.eps, rows, False)
    else:
      ops.add_rmsnorm(out, resid, first, self.weight, self.eps, rows, False)
    return out


class LayerNorm(Norm):
  """``(x - mean) / sqrt(var + eps) * weight + bias`` in float32, the variance being the mean of the squared
  deviations; the residual add (of one or two pending outputs) in front of it, in one kernel.  ``bias_name``: the file
  tensor of the bias (default ``<name>.bias``; the weight is ``<name>.weight`` or, with ``bare_names``, ``<name>``)."""

  def __init__(self, name: str, dim: int, eps: float, weight_name: Optional[str] = None, bias_name: Optional[str] = None):
    super().__init__(name)
    self.dim = dim
    self.eps = float(eps)
    self.weight_name = weight_name or f"{name}.weight"
    self.bias_name = bias_name or f"{name}.bias"

  def param_specs(self) -> Dict[str, ParamSpec]:
    return {"weight": ParamSpec((self.dim,), "vector", [whole(self.weight_name, (self.dim,))], init="ones_noise"),
            "bias": ParamSpec((self.dim,), "vector", [whole(self.bias_name, (self.dim,))])}

  def validate(self, dtype: torch.dtype) -> None:
    if self.dim > 12000:
      raise ValueError(f"{self.name}: rows of {self.dim} values are more than the layer-norm kernel keeps in shared memory (12000)")

  def add_norm(self, resid: torch.Tensor, delta: Delta, ctx) -> torch.Tensor:
    first, second = split_delta(delta)
    out = ctx.ws.buffer("normed", (resid.shape[0], self.dim), ctx.dtype)
    ops.add_layernorm(out, resid, first, second, self.weight, self.bias, self.eps, None, True)
    return out

  def norm_rows(self, resid: torch.Tensor, delta: Delta, rows: torch.Tensor, ctx) -> torch.Tensor:
    first, second = split_delta(delta)
    out = ctx.ws.buffer("normed_rows", (rows.shape[0], self.dim), ctx.dtype)
    ops.add_layernorm(out, resid, first, second, self.weight, self.bias, self.eps, rows, False)
    return out
