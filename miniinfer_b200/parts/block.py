"""The arrangement of the parts of a layer.

``PreNormBlock`` is the reference's wiring (miniinfer/models/fused_qwen3.py:175-196): the residual
is carried beside the hidden state; each norm first adds the previous part's output into the
residual and then normalises it.  The block returns its feed-forward output as the pending
addition for whoever comes next (the next block's first norm, or the final norm).
"""

from __future__ import annotations

from typing import List, Optional

import torch

from .base import Block, FeedForward, Mixer, Norm, Part


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
