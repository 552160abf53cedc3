"""Rotary position encoding as a part: it owns theta, the rotated width and the angle table.

The table is made exactly as the reference makes it, in float32 on the host
(miniinfer/layers/position_encoding.py:29-45): ``inv = 1 / theta^(2j/dim)``, ``angle = pos * inv``,
a row holds ``cos`` of all angles and then ``sin``.  The rotation itself happens inside the mixer's
fused QKV kernel, in float32 (the reference rotates in the model's dtype, position_encoding.py:105-106).
"""

from __future__ import annotations

from typing import Optional

import torch

from .base import PositionEncoding


class RotaryEncoding(PositionEncoding):
  def __init__(self, name: str, rotary_dim: int, theta: float, max_position_embeddings: int):
    super().__init__(name)
    if rotary_dim <= 0 or rotary_dim % 2:
      raise ValueError(f"rotary_dim must be positive and even, got {rotary_dim}")
    self.rotary_dim = rotary_dim
    self.theta = float(theta)
    self.max_position_embeddings = max_position_embeddings
    self._table: Optional[torch.Tensor] = None

  def build_table(self, positions: int) -> torch.Tensor:
    inv_freq = 1.0 / (self.theta ** (torch.arange(0, self.rotary_dim, 2, dtype=torch.float) / self.rotary_dim))
    t = torch.arange(positions, dtype=torch.float)
    freqs = torch.einsum("i,j -> ij", t, inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1).contiguous()

  def prepare(self, device, max_positions: int) -> None:
    n = min(max_positions, self.max_position_embeddings)
    self._table = self.build_table(n).to(device)

  def rotary_table(self) -> Optional[torch.Tensor]:
    if self._table is None:
      raise RuntimeError("RotaryEncoding.prepare was not called")
    return self._table

  def max_positions(self) -> Optional[int]:
    return self.max_position_embeddings


class ScaledRotaryEncoding(RotaryEncoding):
  """Rotary angles whose frequencies are stretched for contexts longer than the ``original`` one (YaRN): with
  ``f_i = theta^(-2i/dims)`` and ``turns(t) = dims * ln(original / (2 pi t)) / (2 ln theta)`` - the index of the frequency
  that makes ``t`` turns over the original context - frequencies below index ``lo = max(floor(turns(fast)), 0)`` stay,
  those above ``hi = min(ceil(turns(slow)), dims - 1)`` are divided by ``factor``, those between are blended linearly
  (``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``, ``f_i <- f_i / factor * ramp_i + f_i * (1 - ramp_i)``), and cos
  and sin are multiplied by ``0.1 ln(factor) + 1``.  Angles are made in float64 and rounded once.  Without ``scaling``
  this is the plain table."""

  def __init__(self, name: str, rotary_dim: int, theta: float, max_position_embeddings: int, scaling: Optional[dict] = None):
    super().__init__(name, rotary_dim, theta, max_position_embeddings)
    if scaling is not None:
      for key in ("factor", "original", "fast", "slow"):
        if not isinstance(scaling.get(key), (int, float)) or not scaling[key] > 0:
          raise ValueError(f"{name}: scaling.{key} must be a positive number, got {scaling.get(key)!r}")
    self.scaling = dict(scaling) if scaling is not None else None

  def frequencies(self):
    """(frequencies [dims / 2] in float64, the factor on cos and sin)."""
    import math
    dims = self.rotary_dim
    i = torch.arange(0, dims // 2, dtype=torch.float64)
    f = self.theta ** (-2.0 * i / dims)
    s = self.scaling
    if s is None:
      return f, 1.0

    def turns(t):
      return dims * math.log(s["original"] / (2 * math.pi * t)) / (2 * math.log(self.theta))

    lo = max(math.floor(turns(s["fast"])), 0)
    hi = min(math.ceil(turns(s["slow"])), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / s["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(s["factor"]) + 1.0

  def build_table(self, positions: int) -> torch.Tensor:
    f, m = self.frequencies()
    angles = torch.arange(positions, dtype=torch.float64)[:, None] * f[None, :]
    return torch.cat((angles.cos() * m, angles.sin() * m), dim=-1).float().contiguous()


class BandScaledRotaryEncoding(RotaryEncoding):
  """Rotary angles whose low frequencies are divided by ``factor`` and whose high frequencies stay, by wavelength
  (the scaling of Llama 3.1): with ``f_i = theta^(-2i/dims)`` and wavelength ``l_i = 2 pi / f_i``, ``f_i`` stays where
  ``l_i < original / high``, becomes ``f_i / factor`` where ``l_i > original / low``, and between the two
  ``(1 - s) f_i / factor + s f_i`` with ``s = (original / l_i - low) / (high - low)``.  cos and sin are not scaled.  Angles
  are made in float64 and rounded once.  Without ``scaling`` this is the plain table."""

  def __init__(self, name: str, rotary_dim: int, theta: float, max_position_embeddings: int, scaling: Optional[dict] = None):
    super().__init__(name, rotary_dim, theta, max_position_embeddings)
    if scaling is not None:
      for key in ("factor", "low", "high", "original"):
        if not isinstance(scaling.get(key), (int, float)) or not scaling[key] > 0:
          raise ValueError(f"{name}: scaling.{key} must be a positive number, got {scaling.get(key)!r}")
      if not scaling["high"] > scaling["low"]:
        raise ValueError(f"{name}: scaling.high must be more than scaling.low")
    self.scaling = dict(scaling) if scaling is not None else None

  def frequencies(self) -> torch.Tensor:
    """Frequencies [dims / 2] in float64."""
    import math
    dims = self.rotary_dim
    f = self.theta ** (-2.0 * torch.arange(0, dims // 2, dtype=torch.float64) / dims)
    s = self.scaling
    if s is None:
      return f
    turns = s["original"] * f / (2 * math.pi)          # original / wavelength
    blend = ((turns - s["low"]) / (s["high"] - s["low"])).clamp(0.0, 1.0)
    return (1.0 - blend) * f / s["factor"] + blend * f

  def build_table(self, positions: int) -> torch.Tensor:
    angles = torch.arange(positions, dtype=torch.float64)[:, None] * self.frequencies()[None, :]
    return torch.cat((angles.cos(), angles.sin()), dim=-1).float().contiguous()
