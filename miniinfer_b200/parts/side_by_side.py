"""Two mixers side by side on the same input, as one mixer part: each output is divided by its root mean square over the
model width and multiplied by a weight of its own, and the mixer's output is ``scale`` times their sum (0.5: their mean).

    ``out = scale * (w_left * left(h) / rms(left(h)) + w_right * right(h) / rms(right(h)))``,  ``rms(x) = sqrt(mean(x^2) + eps)``

With ``normed=False`` the outputs are summed as they are, each times a constant: ``out = left_scale * left(h) + right_scale *
right(h)`` (no weights, no norms).

What the pair keeps for a request is what its members keep, handed over member by member (``CompositeSpec``): one may hold
pages of keys and the other a recurrent state.  File tensors: the members' under ``<name>.left.*`` / ``<name>.right.*``, the
two weights ``<name>.left.out`` and ``<name>.right.out``.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache.specs import CacheSpec, CompositeSpec
from ..kernels import ops
from .base import Mixer, ParamSpec, Part, whole


class SideBySideMixer(Mixer):
  def __init__(self, name: str, hidden_size: int, left: Mixer, right: Mixer, norm_eps: float, scale: float = 0.5,
               weight_names: Optional[Dict[str, str]] = None, normed: bool = True, left_scale: float = 1.0, right_scale: float = 1.0):
    super().__init__(name)
    self.normed = bool(normed)
    self.left_scale, self.right_scale = float(left_scale), float(right_scale)
    self.hidden_size = hidden_size
    self.left, self.right = left, right
    self.norm_eps = float(norm_eps)
    self.scale = float(scale)
    self.weight_names = {"left": f"{name}.left.out", "right": f"{name}.right.out"}
    self.weight_names.update(weight_names or {})
    left.out_buffer, right.out_buffer = "mixer_out_left", "mixer_out_right"

  def sub_parts(self) -> List[Part]:
    return [self.left, self.right]

  def cache_spec(self) -> Optional[CacheSpec]:
    members = (self.left.cache_spec(), self.right.cache_spec())
    if any(m is None or isinstance(m, CompositeSpec) for m in members):
      raise ValueError(f"{self.name}: both members must keep pages or a state of their own")
    return CompositeSpec(members)

  def param_specs(self) -> Dict[str, ParamSpec]:
    W = self.hidden_size
    if not self.normed:
      return {}
    return {"left_out": ParamSpec((W,), "vector", [whole(self.weight_names["left"], (W,))], init="ones_noise"),
            "right_out": ParamSpec((W,), "vector", [whole(self.weight_names["right"], (W,))], init="ones_noise")}

  def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
    if cache.kind != "composite" or len(cache.members) != 2:
      raise RuntimeError(f"{self.name}: two mixers side by side need the caches of both, got {cache.kind!r}")
    a = self.left.forward(x, ctx, cache.members[0])
    b = self.right.forward(x, ctx, cache.members[1])
    out = ctx.ws.buffer(self.out_buffer, (x.shape[0], self.hidden_size), ctx.dtype)
    if self.normed:
      ops.rms_pair_sum(out, a, b, self.left_out, self.right_out, self.norm_eps, self.scale)
    else:
      ops.scaled_pair_sum(out, a, b, self.left_scale, self.right_scale)
    return out
