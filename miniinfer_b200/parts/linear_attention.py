"""Linear attention with a decaying matrix state, as a mixer part: gated linear attention (a learned decay per token and
key channel) and retention (one fixed decay a head) are two settings of it.

For the normalised rows ``h`` of a step, with ``H`` heads, query/key size ``dim`` and value size ``vdim``:

  * one fused product gives ``q``, ``k`` (``H x dim``), ``v`` and the gate's logits (``H x vdim``) and, with ``decay="channel"``,
    the low-rank input ``W_a1 h`` of the decays;
  * with ``rotary`` the first ``rotary_dim`` values of every query and key head are rotated by the token's position (value i
    with value i + rotary_dim / 2); then ``q <- q_scale * q`` and ``k <- k_scale * k``;
  * ``decay="channel"``: ``alpha = sigmoid(z)^(1 / tau)`` with ``z = W_a2 (W_a1 h) + b`` laid out ``H x dim``, made as
    ``exp(logsigmoid(z) / tau)``;  ``decay="head"``: ``alpha`` is the constant ``head_decay[h]`` for every channel of head h;
  * per head ``S_t = diag(alpha_t) S_(t-1) + k_t v_t^T`` and ``o_t = S_t^T q_t`` (the read-out sees the token's own write);
  * ``o <- o / sqrt(mean(o^2) + eps)`` over ``vdim``, times a weight ``[vdim]`` shared by the heads if ``norm_weight``;
  * the heads, side by side, are multiplied with ``silu`` (or ``sigmoid``) of the gate's logits and projected by ``W_o``.

What a request keeps is ``S`` of every head as one float32 row (``FixedStateSpec``), zero at admission.  Angles, decays and
their logarithms, the state, the sums over it and the norm are float32 whatever the compute dtype.  File tensors (after
``<name>.``): ``q``, ``k``, ``v``, ``g``, ``o`` and, as the options ask, ``norm``, ``a1``, ``a2``, ``a2.b``.
"""

from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from ..cache.specs import CacheSpec, FixedStateSpec
from ..kernels import ops
from .base import Mixer, ParamSpec, Piece, PositionEncoding, whole
from .recurrent import _state_rows


class LinearAttentionMixer(Mixer):
  def __init__(self, name: str, hidden_size: int, num_heads: int, dim: int, vdim: int, norm_eps: float, decay: str = "channel",
               decay_rank: Optional[int] = None, tau: float = 1.0, head_decay: Optional[Sequence[float]] = None,
               rotary: Optional[PositionEncoding] = None, q_scale: float = 1.0, k_scale: float = 1.0, norm_weight: bool = True,
               gate: str = "silu", tensors: Optional[Dict[str, str]] = None):
    super().__init__(name)
    for what, v in (("heads", num_heads), ("dim", dim), ("vdim", vdim)):
      if v <= 0:
        raise ValueError(f"{name}: {what} must be positive, got {v}")
    if decay not in ("channel", "head"):
      raise ValueError(f"{name}: decay must be 'channel' or 'head', got {decay!r}")
    if decay == "channel":
      if decay_rank is None or decay_rank <= 0 or not tau > 0:
        raise ValueError(f"{name}: decays per channel need the rank of their projection and a positive tau (got {decay_rank}, {tau})")
    else:
      if head_decay is None or len(head_decay) != num_heads or not all(0.0 <= float(d) <= 1.0 for d in head_decay):
        raise ValueError(f"{name}: decays per head need one factor in 0..1 for each of the {num_heads} heads, got {head_decay!r}")
    if gate not in ("silu", "sigmoid"):
      raise ValueError(f"{name}: gate must be 'silu' or 'sigmoid', got {gate!r}")
    self.hidden_size, self.num_heads, self.dim, self.vdim = hidden_size, num_heads, dim, vdim
    self.norm_eps = float(norm_eps)
    self.decay = decay
    self.decay_rank = int(decay_rank) if decay == "channel" else 0
    self.tau = float(tau)
    self.head_decay_values = [float(d) for d in head_decay] if decay == "head" else None
    self.position = rotary
    self.q_scale, self.k_scale = float(q_scale), float(k_scale)
    self.norm_weight = bool(norm_weight)
    self.gate = gate
    t = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "a1": "a1", "a2": "a2", "a2_bias": "a2.b"}
    t.update(tensors or {})
    self.tensors = t
    H = num_heads
    # rows of the fused projection: the decays' low-rank input first (the product behind it reads it in place)
    self.a1_off = 0
    self.q_off = self.decay_rank
    self.k_off = self.q_off + H * dim
    self.v_off = self.k_off + H * dim
    self.g_off = self.v_off + H * vdim
    self.proj_width = self.g_off + H * vdim
    self._head_decay: Optional[torch.Tensor] = None

  def cache_spec(self) -> Optional[CacheSpec]:
    return FixedStateSpec((self.num_heads * self.dim * self.vdim,), "float32")

  def param_specs(self) -> Dict[str, ParamSpec]:
    W, H, D, Dv, n, t, r = self.hidden_size, self.num_heads, self.dim, self.vdim, self.name, self.tensors, self.decay_rank
    pieces = [Piece(f"{n}.{t['q']}", self.q_off, (H * D, W)), Piece(f"{n}.{t['k']}", self.k_off, (H * D, W)),
              Piece(f"{n}.{t['v']}", self.v_off, (H * Dv, W)), Piece(f"{n}.{t['g']}", self.g_off, (H * Dv, W))]
    if self.decay == "channel":
      pieces.append(Piece(f"{n}.{t['a1']}", self.a1_off, (r, W)))
    specs = {"proj": ParamSpec((self.proj_width, W), "matrix", [pieces]),
             "w_o": ParamSpec((W, H * Dv), "matrix", [whole(f"{n}.{t['o']}", (W, H * Dv))])}
    if self.decay == "channel":
      specs["a2"] = ParamSpec((H * D, r), "matrix", [whole(f"{n}.{t['a2']}", (H * D, r))])
      specs["a2_bias"] = ParamSpec((H * D,), "vector", [whole(f"{n}.{t['a2_bias']}", (H * D,))], init="decay_bias")
    if self.norm_weight:
      specs["norm"] = ParamSpec((Dv,), "vector", [whole(f"{n}.{t['norm']}", (Dv,))], init="ones_noise")
    return specs

  def validate(self, dtype: torch.dtype) -> None:
    if self.dim > 4096:
      raise ValueError(f"{self.name}: the linear-attention kernel keeps up to 4096 key channels a head, got dim={self.dim}")
    rotary = getattr(self.position, "rotary_dim", None)
    if rotary is not None and rotary > self.dim:
      raise ValueError(f"{self.name}: the rotary encoding covers {rotary} values, more than dim={self.dim}")
    if dtype == torch.bfloat16 and self.hidden_size % 8:
      raise ValueError(f"{self.name}: width={self.hidden_size} must be a multiple of 8 in bfloat16 (rows are read 16 bytes at a time)")

  def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
    T = x.shape[0]
    H, D, Dv = self.num_heads, self.dim, self.vdim
    state = _state_rows(cache, self.name)
    proj = ctx.ws.buffer("linear_attention_proj", (T, self.proj_width), ctx.dtype)
    ops.linear(proj, x, self.proj)
    logits = None
    if self.decay == "channel":
      logits = ctx.ws.buffer("linear_attention_decay", (T, H * D), torch.float32)
      ops.linear(logits, proj[:, self.a1_off:self.a1_off + self.decay_rank], self.a2)
    elif self._head_decay is None or self._head_decay.device != x.device:
      # constants of the model: rounded to float32 once, as the recurrence holds them
      self._head_decay = torch.tensor(self.head_decay_values, dtype=torch.float64).to(torch.float32).to(x.device)
    heads = ctx.ws.buffer("linear_attention_heads", (T, H * Dv), ctx.dtype)
    ops.linear_attention(heads, proj[:, self.q_off:self.q_off + H * D], proj[:, self.k_off:self.k_off + H * D],
                         proj[:, self.v_off:self.v_off + H * Dv], proj[:, self.g_off:self.g_off + H * Dv], state, ctx, H, D, Dv,
                         self.norm_eps, decay_logits=logits, decay_bias=self.a2_bias if logits is not None else None, tau=self.tau,
                         head_decay=self._head_decay if logits is None else None,
                         rope=self.position.rotary_table() if self.position is not None else None, q_scale=self.q_scale,
                         k_scale=self.k_scale, norm_weight=self.norm if self.norm_weight else None, gate_silu=self.gate == "silu",
                         workspace=ctx.ws)
    out = ctx.ws.buffer(self.out_buffer, (T, self.hidden_size), ctx.dtype)
    ops.linear(out, heads, self.w_o)
    return out
