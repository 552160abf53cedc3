"""The arrangement of the parts of a layer.

``PreNormBlock`` is the reference's wiring (miniinfer/models/fused_qwen3.py:175-196): the residual
is carried beside the hidden state; each norm first adds the previous part's output into the
residual and then normalises it.  The block returns its feed-forward output as the pending
addition for whoever comes next (the next block's first norm, or the final norm).
"""

from __future__ import annotations

from typing import List, Optional

import torch

from ..cache.manager import LayerCache
from ..cache.specs import CompositeSpec, FixedStateSpec
from ..kernels import ops
from .base import Block, FeedForward, Mixer, Norm, ParamSpec, Part, whole


class PreNormBlock(Block):
  """``ffn`` (and its norm) may be None: a layer of a mixer alone, whose output is left pending."""

  def __init__(self, name: str, mixer_norm: Norm, mixer: Mixer, ffn_norm: Optional[Norm], ffn: Optional[FeedForward]):
    super().__init__(name)
    if ffn is not None and ffn_norm is None:
      raise ValueError(f"{name}: a feed-forward needs its norm")
    self.mixer_norm = mixer_norm
    self.mixer = mixer
    self.ffn_norm = ffn_norm if ffn is not None else None
    self.ffn = ffn

  def sub_parts(self) -> List[Part]:
    return [self.mixer_norm, self.mixer] + ([self.ffn_norm, self.ffn] if self.ffn is not None else [])

  def mixer_part(self) -> Optional[Mixer]:
    return self.mixer

  def forward(self, resid: torch.Tensor, pending: Optional[torch.Tensor], ctx, cache) -> Optional[torch.Tensor]:
    # A part may offer to work on the residual stream itself - its norm in its first kernel, the add of its
    # output in its last (for a step of few rows: fewer launches).  Then nothing is pending behind it.
    if pending is None and self.mixer.takes_residual(self.mixer_norm, ctx):
      self.mixer.forward_on_residual(resid, self.mixer_norm, ctx, cache)
      a = None
    else:
      x = self.mixer_norm.add_norm(resid, pending, ctx)
      a = self.mixer.forward(x, ctx, cache)
    if self.ffn is None:
      return a
    if a is None and self.ffn.takes_residual(self.ffn_norm, ctx):
      self.ffn.forward_on_residual(resid, self.ffn_norm, ctx)
      return None
    x = self.ffn_norm.add_norm(resid, a, ctx)
    return self.ffn.forward(x, ctx)


class ParallelBlock(Block):
  """Mixer and feed-forward side by side on the same residual rows: ``x <- x + (mixer(norm(x)) + ff(ffn_norm(x)))``.
  With one norm (``ffn_norm`` None) both read its output; with two, each has a norm of its own on the same rows, and the
  two are computed together (``Norm.add_norm_pair``: one root mean square, two weights).  The two outputs are left pending
  as a pair and added, in float32, by the norm that comes next.  ``ffn`` may be None (a layer without a feed-forward)."""

  def __init__(self, name: str, norm: Norm, mixer: Mixer, ffn: Optional[FeedForward], ffn_norm: Optional[Norm] = None):
    super().__init__(name)
    self.norm = norm
    self.mixer = mixer
    self.ffn = ffn
    self.ffn_norm = ffn_norm if ffn is not None else None

  def sub_parts(self) -> List[Part]:
    return [self.norm, self.mixer] + ([self.ffn_norm] if self.ffn_norm is not None else []) + ([self.ffn] if self.ffn is not None else [])

  def mixer_part(self) -> Optional[Mixer]:
    return self.mixer

  def forward(self, resid: torch.Tensor, pending, ctx, cache):
    if self.ffn_norm is not None:
      x, x_ffn = self.norm.add_norm_pair(resid, pending, self.ffn_norm, ctx)
    else:
      x = x_ffn = self.norm.add_norm(resid, pending, ctx)
    a = self.mixer.forward(x, ctx, cache)
    if self.ffn is None:
      return a
    return (a, self.ffn.forward(x_ffn, ctx))


class OutputNormBlock(Block):
  """A layer whose sublayers read the residual stream as it is and whose norms stand on the sublayers' outputs:

      ``x <- x + mult * norm1(mixer(h))``, then ``x <- x + mult * norm2(ff(x))``,   ``h = x`` or, with ``token_shift``,
      ``h[t] = x[t] + (x[t - 1] - x[t]) * shift``  (element by element; ``x[t - 1]`` is zero for a request's first token)

  The residual stream is float32; a sublayer gets its rows rounded once to the compute dtype.  With ``token_shift`` the block
  keeps, for every request, the residual row its mixer last read (``width`` float32 values beside what the mixer itself keeps),
  so that the first token of a later portion finds its predecessor; ``shift`` is the file tensor ``<name>.shift``.  The norms must be RMS norms
  (``RMSNorm.add_scaled``).  ``ffn`` may be None.  Nothing is left pending behind the block."""

  def __init__(self, name: str, width: int, mixer_norm: Norm, mixer: Mixer, ffn_norm: Optional[Norm], ffn: Optional[FeedForward],
               mult: float = 1.0, token_shift: bool = False, shift_name: Optional[str] = None):
    super().__init__(name)
    if ffn is not None and ffn_norm is None:
      raise ValueError(f"{name}: a feed-forward needs its norm")
    for n in (mixer_norm, ffn_norm):
      if n is not None and not hasattr(n, "add_scaled"):
        raise ValueError(f"{name}: the norm of a sublayer's output must offer add_scaled (an RMS norm), got {type(n).__name__}")
    self.width = width
    self.mixer_norm, self.mixer = mixer_norm, mixer
    self.ffn = ffn
    self.ffn_norm = ffn_norm if ffn is not None else None
    self.mult = float(mult)
    self.token_shift = bool(token_shift)
    self.shift_name = shift_name or f"{name}.shift"

  def sub_parts(self) -> List[Part]:
    return [self.mixer_norm, self.mixer] + ([self.ffn_norm, self.ffn] if self.ffn is not None else [])

  def mixer_part(self) -> Optional[Mixer]:
    return self.mixer

  def param_specs(self):
    if not self.token_shift:
      return {}
    return {"shift": ParamSpec((self.width,), "vector", [whole(self.shift_name, (self.width,))], init="half_noise")}

  def cache_spec(self):
    inner = self.mixer.cache_spec()
    if not self.token_shift:
      return inner
    mine = FixedStateSpec((self.width,), "float32")
    if inner is None:
      return mine
    return CompositeSpec((mine,) + (tuple(inner.members) if isinstance(inner, CompositeSpec) else (inner,)))

  def _split_cache(self, cache):
    """(the rows of the token shift's state or None, the mixer's cache)."""
    if not self.token_shift:
      return None, cache
    if cache.kind == "state":
      return cache.tensor, LayerCache(kind="none", writes=False)
    if cache.kind != "composite" or cache.members[0].kind != "state":
      raise RuntimeError(f"{self.name}: a block with a token shift needs its state beside the mixer's cache, got {cache.kind!r}")
    rest = cache.members[1:]
    if len(rest) == 1:
      return cache.members[0].tensor, rest[0]
    return cache.members[0].tensor, LayerCache("composite", writes=cache.writes, members=list(rest))

  def forward(self, resid: torch.Tensor, pending, ctx, cache):
    if pending is not None:      # what a block of another kind left behind joins the stream first
      self.mixer_norm.add_norm(resid, pending, ctx)
    shift_rows, mixer_cache = self._split_cache(cache)
    if self.token_shift or ctx.dtype != torch.float32:
      h = ctx.ws.buffer("shifted", resid.shape, ctx.dtype)
      ops.token_shift(h, resid, self.shift if self.token_shift else None, shift_rows, ctx)
    else:
      h = resid
    a = self.mixer.forward(h, ctx, mixer_cache)
    # the mixer has read the rows: the last one of every request becomes the shift's state as the addition replaces it
    x = self.mixer_norm.add_scaled(resid, a, self.mult, ctx, copy=self.ffn is not None, keep=shift_rows)
    if self.ffn is not None:
      f = self.ffn.forward(x, ctx)
      self.ffn_norm.add_scaled(resid, f, self.mult, ctx)
    return None
