"""Hyper-connections: a residual stream made of ``S`` streams.

The rows of the stream tensor are ``[token, S * width]`` float32, stream after stream; the embedding fills every stream
with the same row.  A sublayer ``f`` (a mixer or a feed-forward behind its norm) with vectors ``in [S]``, ``out [S]`` and a
matrix ``mix [S, S]`` (indexed [from, to]) reads and writes all streams:

    ``u = sum_s in[s] x_s;   y = f(norm(u));   x_t <- sum_s mix[s, t] x_s + out[t] y``  (all ``t`` at once, from the old streams)

and what leaves the model is the sum of the streams.  One kernel (``ops.hyper_connection``) writes the update of the
sublayer before and reads for the sublayer after - ``u`` and its RMS norm included when the norm is a plain RMS norm - so
the update of a sublayer is left pending (``PendingUpdate``) for whoever reads the streams next: the next sublayer, the
next block, or the final ``StreamSumNorm``.  Everything here is float32 whatever the compute dtype.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import Block, FeedForward, Mixer, Norm, ParamSpec, Part, whole

MAX_STREAMS = 8


@dataclass
class PendingUpdate:
  """A sublayer's output ``y [tokens, width]`` that is not yet in the streams, with the ``mix`` and ``out`` it enters by."""

  y: torch.Tensor
  mix: torch.Tensor
  out: torch.Tensor


def _pending(pending) -> Optional[PendingUpdate]:
  if pending is None or isinstance(pending, PendingUpdate):
    return pending
  raise TypeError("a stream tensor takes the pending update of a hyper-connection sublayer, not a plain residual addition")


class HyperConnectionBlock(Block):
  """A pre-norm layer over ``streams`` residual streams: the mixer behind ``mixer_norm`` and, if there is one, the
  feed-forward behind ``ffn_norm``, each with hyper-connection weights of its own.  File tensors: ``<name>.hc1.{in,out,mix}``
  for the mixer and ``<name>.hc2.{in,out,mix}`` for the feed-forward."""

  def __init__(self, name: str, streams: int, width: int, mixer_norm: Norm, mixer: Mixer, ffn_norm: Optional[Norm],
               ffn: Optional[FeedForward]):
    super().__init__(name)
    if streams < 1:
      raise ValueError(f"{name}: streams must be positive, got {streams}")
    self.streams, self.width = streams, width
    self.mixer_norm, self.mixer = mixer_norm, mixer
    self.ffn = ffn
    self.ffn_norm = ffn_norm if ffn is not None else None
    if ffn is not None and ffn_norm is None:
      raise ValueError(f"{name}: a feed-forward needs its norm")

  def sub_parts(self) -> List[Part]:
    return [self.mixer_norm, self.mixer] + ([self.ffn_norm, self.ffn] if self.ffn is not None else [])

  def mixer_part(self) -> Optional[Mixer]:
    return self.mixer

  def param_specs(self) -> Dict[str, ParamSpec]:
    S, n = self.streams, self.name
    specs = {}
    for q in ("1", "2") if self.ffn is not None else ("1",):
      specs[f"hc{q}_in"] = ParamSpec((S,), "vector", [whole(f"{n}.hc{q}.in", (S,))], init="mean_noise")
      specs[f"hc{q}_out"] = ParamSpec((S,), "vector", [whole(f"{n}.hc{q}.out", (S,))], init="ones_noise")
      specs[f"hc{q}_mix"] = ParamSpec((S, S), "vector", [whole(f"{n}.hc{q}.mix", (S, S))], init="identity_noise")
    return specs

  def validate(self, dtype: torch.dtype) -> None:
    if self.streams > MAX_STREAMS:
      raise ValueError(f"{self.name}: the hyper-connection kernel takes up to {MAX_STREAMS} streams, got {self.streams}")

  def _read(self, streams: torch.Tensor, pending, in_w: torch.Tensor, norm: Norm, ctx) -> torch.Tensor:
    """Brings the streams up to date with ``pending`` and returns the normalised input of the next sublayer."""
    p = _pending(pending)
    T = streams.shape[0]
    rms = norm.as_rms()
    if rms is not None:
      x = ctx.ws.buffer("normed", (T, self.width), ctx.dtype)
      ops.hyper_connection(x, streams, p.y if p else None, p.mix if p else None, p.out if p else None, in_w, rms[0], rms[1], None, True)
      return x
    u = ctx.ws.buffer("hyper_read", (T, self.width), torch.float32)
    ops.hyper_connection(u, streams, p.y if p else None, p.mix if p else None, p.out if p else None, in_w, None, 1.0, None, True)
    return norm.add_norm(u, None, ctx)

  def forward(self, resid: torch.Tensor, pending, ctx, cache):
    if resid.shape[1] != self.streams * self.width:
      raise RuntimeError(f"{self.name}: the stream tensor has rows of {resid.shape[1]} values, {self.streams} x {self.width} expected")
    x = self._read(resid, pending, self.hc1_in, self.mixer_norm, ctx)
    pending = PendingUpdate(self.mixer.forward(x, ctx, cache), self.hc1_mix, self.hc1_out)
    if self.ffn is None:
      return pending
    x = self._read(resid, pending, self.hc2_in, self.ffn_norm, ctx)
    return PendingUpdate(self.ffn.forward(x, ctx), self.hc2_mix, self.hc2_out)


class StreamSumNorm(Norm):
  """The norm that ends a model of ``streams`` residual streams: the pending update is applied, the streams are summed,
  and the sum is RMS-normed, ``w * x / sqrt(mean(x^2) + eps)``, in one kernel."""

  def __init__(self, name: str, dim: int, eps: float, streams: int, weight_name: Optional[str] = None):
    super().__init__(name)
    self.dim, self.eps, self.streams = dim, float(eps), streams
    self.weight_name = weight_name or f"{name}.weight"

  def param_specs(self) -> Dict[str, ParamSpec]:
    return {"weight": ParamSpec((self.dim,), "vector", [whole(self.weight_name, (self.dim,))], init="ones_noise")}

  def validate(self, dtype: torch.dtype) -> None:
    if self.streams > MAX_STREAMS:
      raise ValueError(f"{self.name}: the hyper-connection kernel takes up to {MAX_STREAMS} streams, got {self.streams}")

  def add_norm(self, resid: torch.Tensor, delta, ctx) -> torch.Tensor:
    p = _pending(delta)
    out = ctx.ws.buffer("normed", (resid.shape[0], self.dim), ctx.dtype)
    ops.hyper_connection(out, resid, p.y if p else None, p.mix if p else None, p.out if p else None, None, self.weight, self.eps, None, True)
    return out

  def norm_rows(self, resid: torch.Tensor, delta, rows: torch.Tensor, ctx) -> torch.Tensor:
    p = _pending(delta)
    out = ctx.ws.buffer("normed_rows", (rows.shape[0], self.dim), ctx.dtype)
    ops.hyper_connection(out, resid, p.y if p else None, p.mix if p else None, p.out if p else None, None, self.weight, self.eps, rows, False)
    return out
