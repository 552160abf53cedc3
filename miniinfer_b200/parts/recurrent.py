"""Mixers that carry a state from token to token: the selective scan and the gated delta rule, each behind a short
causal convolution.  What such a mixer keeps for a request is one float32 row (``FixedStateSpec``): the convolution's
last ``taps - 1`` inputs, then the recurrent state.  The state manager hands out a zeroed row when a request is admitted;
the kernels walk an item's new tokens from the stored state and leave the state after its last token, on the device,
so steps of these mixers are replayed from CUDA graphs like steps of attention.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.specs import CacheSpec, FixedStateSpec
from ..kernels import ops
from .base import Mixer, ParamSpec, Piece, whole


def _state_rows(cache, name: str) -> torch.Tensor:
  if cache.kind != "state":
    raise RuntimeError(f"{name}: a recurrent mixer needs a per-request state, got a cache of kind {cache.kind!r}")
  return cache.tensor


class SelectiveScanMixer(Mixer):
  """Selective state-space mixer.  With ``inner`` channels, ``state`` values a channel and a step-size rank ``dt_rank``:

    ``[u | z] = W_in h``;  ``u <- silu(conv(u) + conv_bias)`` (causal, per channel, ``taps`` taps);
    ``[r | B | C] = W_x u`` (``dt_rank``, ``state``, ``state`` values);  ``dt = softplus(W_dt r + dt_bias)``;  ``A = -exp(A_log)``;
    ``S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c u_c B_n``;  ``y_c = sum_n S[c, n] C_n + D_c u_c``;  out = ``W_o (y * silu(z))``.

  The step size, the decays and the state are float32.  File tensors (after ``<name>.``): ``in``, ``conv``, ``conv.b``, ``x``,
  ``dt``, ``dt.b``, ``A_log``, ``D``, ``o``."""

  def __init__(self, name: str, hidden_size: int, inner: int, state: int, dt_rank: int, taps: int,
               tensors: Optional[Dict[str, str]] = None):
    super().__init__(name)
    for what, v in (("inner", inner), ("state", state), ("dt_rank", dt_rank), ("taps", taps)):
      if v <= 0:
        raise ValueError(f"{name}: {what} must be positive, got {v}")
    self.hidden_size, self.inner, self.state, self.dt_rank, self.taps = hidden_size, inner, state, dt_rank, taps
    t = {"in": "in", "conv": "conv", "conv_b": "conv.b", "x": "x", "dt": "dt", "dt_b": "dt.b", "A_log": "A_log", "D": "D", "o": "o"}
    t.update(tensors or {})
    self.tensors = t
    self.conv_floats = (taps - 1) * inner

  def cache_spec(self) -> Optional[CacheSpec]:
    return FixedStateSpec((self.conv_floats + self.inner * self.state,), "float32")

  def param_specs(self) -> Dict[str, ParamSpec]:
    W, I, N, R, K, n, t = self.hidden_size, self.inner, self.state, self.dt_rank, self.taps, self.name, self.tensors
    return {
      "w_in": ParamSpec((2 * I, W), "matrix", [whole(f"{n}.{t['in']}", (2 * I, W))]),
      "conv": ParamSpec((I, K), "vector", [whole(f"{n}.{t['conv']}", (I, K))], init="half_noise"),
      "conv_b": ParamSpec((I,), "vector", [whole(f"{n}.{t['conv_b']}", (I,))]),
      "w_x": ParamSpec((R + 2 * N, I), "matrix", [whole(f"{n}.{t['x']}", (R + 2 * N, I))]),
      "w_dt": ParamSpec((I, R), "matrix", [whole(f"{n}.{t['dt']}", (I, R))]),
      "dt_b": ParamSpec((I,), "vector", [whole(f"{n}.{t['dt_b']}", (I,))]),
      "A_log": ParamSpec((I, N), "vector", [whole(f"{n}.{t['A_log']}", (I, N))]),
      "D": ParamSpec((I,), "vector", [whole(f"{n}.{t['D']}", (I,))], init="ones_noise"),
      "w_o": ParamSpec((W, I), "matrix", [whole(f"{n}.{t['o']}", (W, I))]),
    }

  def bind(self, params) -> None:
    super().bind(params)
    if "w_x" in params:      # the step-size rows and the B / C rows as two matrices: two products with packed outputs
      self.w_x_dt, self.w_x_bc = params["w_x"][:self.dt_rank], params["w_x"][self.dt_rank:]

  def validate(self, dtype: torch.dtype) -> None:
    if self.state > 128 or self.taps > 16:
      raise ValueError(f"{self.name}: the scan kernel takes up to 128 state values a channel and the convolution up to 16 taps "
                       f"(got state={self.state}, conv={self.taps})")

  def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
    T = x.shape[0]
    I, N, R = self.inner, self.state, self.dt_rank
    state = _state_rows(cache, self.name)
    xz = ctx.ws.buffer("scan_xz", (T, 2 * I), ctx.dtype)
    ops.linear(xz, x, self.w_in)
    u = ctx.ws.buffer("scan_u", (T, I), ctx.dtype)
    ops.causal_conv(u, xz[:, :I], self.conv, self.conv_b, state[:, :max(self.conv_floats, 1)], ctx, silu=True)
    low = ctx.ws.buffer("scan_dt_low", (T, R), ctx.dtype)
    ops.linear(low, u, self.w_x_dt)
    bc = ctx.ws.buffer("scan_bc", (T, 2 * N), ctx.dtype)
    ops.linear(bc, u, self.w_x_bc)
    dt = ctx.ws.buffer("scan_dt", (T, I), ctx.dtype)
    ops.linear(dt, low, self.w_dt)
    y = ctx.ws.buffer("scan_y", (T, I), ctx.dtype)
    ops.selective_scan(y, u, dt, bc, 0, N, xz[:, I:], self.dt_b, self.A_log, self.D, state[:, self.conv_floats:], ctx, workspace=ctx.ws)
    out = ctx.ws.buffer(self.out_buffer, (T, self.hidden_size), ctx.dtype)
    ops.linear(out, y, self.w_o)
    return out


class GatedDeltaMixer(Mixer):
  """Gated delta rule.  With ``H`` heads of ``vdim`` values, ``G`` query/key heads of ``dim`` values (head h reads q/k head
  ``h // (H / G)``):

    ``q, k, v = silu(conv(W_q h)), silu(conv(W_k h)), silu(conv(W_v h))`` (causal, per channel, no bias);
    q and k become unit vectors per head, ``x / sqrt(sum x^2 + 1e-6)``, q also times ``dim^-1/2``;
    ``beta = sigmoid(W_b h)`` a head;  ``g = exp(-exp(A_log_h) softplus(W_a2 (W_a1 h) + dt_bias))`` a head and key channel;
    per head ``S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q`` (the read-out sees the token's own write);
    ``o <- o / sqrt(mean(o^2) + eps) * norm * sigmoid(W_g2 (W_g1 h))``; out = ``W_o o``.

  Decays, gates of the recurrence, unit norms and the state are float32.  One fused product gives q, k, v, beta's logits and
  the two low-rank inputs; one convolution runs over the q, k and v channels together.  File tensors (after ``<name>.``):
  ``q``, ``q.conv``, ``k``, ``k.conv``, ``v``, ``v.conv``, ``b``, ``A_log``, ``norm``, ``a1``, ``a2``, ``dt_bias``, ``g1``, ``g2``, ``o``."""

  def __init__(self, name: str, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, taps: int,
               decay_rank: int, gate_rank: int, norm_eps: float, tensors: Optional[Dict[str, str]] = None):
    super().__init__(name)
    if num_heads <= 0 or num_kv_heads <= 0 or num_heads % num_kv_heads:
      raise ValueError(f"{name}: heads={num_heads} must be a multiple of kv_heads={num_kv_heads}")
    for what, v in (("dim", dim), ("vdim", vdim), ("taps", taps), ("decay_rank", decay_rank), ("gate_rank", gate_rank)):
      if v <= 0:
        raise ValueError(f"{name}: {what} must be positive, got {v}")
    self.hidden_size, self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.taps = hidden_size, num_heads, num_kv_heads, dim, vdim, taps
    self.decay_rank, self.gate_rank, self.norm_eps = decay_rank, gate_rank, float(norm_eps)
    t = {"q": "q", "k": "k", "v": "v", "b": "b", "a1": "a1", "a2": "a2", "g1": "g1", "g2": "g2", "o": "o", "A_log": "A_log",
         "dt_bias": "dt_bias", "norm": "norm", "conv": "conv"}
    t.update(tensors or {})
    self.tensors = t
    H, G = num_heads, num_kv_heads
    # rows of the fused projection: the two low-rank inputs first (so that they start on 16-byte boundaries and the
    # products behind them can read them in place), then what the convolution runs over, then beta's logits
    self.a1_off, self.g1_off = 0, decay_rank
    self.conv_off = decay_rank + gate_rank
    self.q_off, self.k_off, self.v_off = 0, G * dim, 2 * G * dim      # within the convolved channels
    self.channels = 2 * G * dim + H * vdim
    self.b_off = self.conv_off + self.channels
    self.proj_width = self.b_off + H
    self.conv_floats = (taps - 1) * self.channels

  def cache_spec(self) -> Optional[CacheSpec]:
    return FixedStateSpec((self.conv_floats + self.num_heads * self.dim * self.vdim,), "float32")

  def param_specs(self) -> Dict[str, ParamSpec]:
    W, H, G, D, Dv, K, n, t = self.hidden_size, self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.taps, self.name, self.tensors
    c = t["conv"]
    return {
      "proj": ParamSpec((self.proj_width, W), "matrix", [[
        Piece(f"{n}.{t['q']}", self.conv_off + self.q_off, (G * D, W)), Piece(f"{n}.{t['k']}", self.conv_off + self.k_off, (G * D, W)),
        Piece(f"{n}.{t['v']}", self.conv_off + self.v_off, (H * Dv, W)), Piece(f"{n}.{t['b']}", self.b_off, (H, W)),
        Piece(f"{n}.{t['a1']}", self.a1_off, (self.decay_rank, W)), Piece(f"{n}.{t['g1']}", self.g1_off, (self.gate_rank, W))]]),
      "conv": ParamSpec((self.channels, K), "vector", [[
        Piece(f"{n}.{t['q']}.{c}", self.q_off, (G * D, K)), Piece(f"{n}.{t['k']}.{c}", self.k_off, (G * D, K)),
        Piece(f"{n}.{t['v']}.{c}", self.v_off, (H * Dv, K))]], init="half_noise"),
      "a2": ParamSpec((H * D, self.decay_rank), "matrix", [whole(f"{n}.{t['a2']}", (H * D, self.decay_rank))]),
      "g2": ParamSpec((H * Dv, self.gate_rank), "matrix", [whole(f"{n}.{t['g2']}", (H * Dv, self.gate_rank))]),
      "dt_bias": ParamSpec((H * D,), "vector", [whole(f"{n}.{t['dt_bias']}", (H * D,))]),
      "A_log": ParamSpec((H,), "vector", [whole(f"{n}.{t['A_log']}", (H,))]),
      "norm": ParamSpec((Dv,), "vector", [whole(f"{n}.{t['norm']}", (Dv,))], init="ones_noise"),
      "w_o": ParamSpec((W, H * Dv), "matrix", [whole(f"{n}.{t['o']}", (W, H * Dv))]),
    }

  def validate(self, dtype: torch.dtype) -> None:
    if self.taps > 16:
      raise ValueError(f"{self.name}: the convolution takes up to 16 taps, got {self.taps}")
    if self.dim > 4096:
      raise ValueError(f"{self.name}: the delta-rule kernel keeps up to 4096 key channels a head, got dim={self.dim}")

  def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
    T = x.shape[0]
    H, G, D, Dv = self.num_heads, self.num_kv_heads, self.dim, self.vdim
    state = _state_rows(cache, self.name)
    proj = ctx.ws.buffer("delta_proj", (T, self.proj_width), ctx.dtype)
    ops.linear(proj, x, self.proj)
    qkv = ctx.ws.buffer("delta_qkv", (T, self.channels), ctx.dtype)
    ops.causal_conv(qkv, proj[:, self.conv_off:self.conv_off + self.channels], self.conv, None, state[:, :max(self.conv_floats, 1)], ctx, silu=True)
    decay = ctx.ws.buffer("delta_decay", (T, H * D), ctx.dtype)
    ops.linear(decay, proj[:, self.a1_off:self.a1_off + self.decay_rank], self.a2)
    gate = ctx.ws.buffer("delta_gate", (T, H * Dv), ctx.dtype)
    ops.linear(gate, proj[:, self.g1_off:self.g1_off + self.gate_rank], self.g2)
    heads = ctx.ws.buffer("delta_heads", (T, H * Dv), ctx.dtype)
    ops.gated_delta(heads, qkv[:, self.q_off:self.q_off + G * D], qkv[:, self.k_off:self.k_off + G * D], qkv[:, self.v_off:],
                    decay, proj[:, self.b_off:self.b_off + H], gate, self.dt_bias, self.A_log, self.norm, self.norm_eps,
                    state[:, self.conv_floats:], ctx, H, G, D, Dv, workspace=ctx.ws)
    out = ctx.ws.buffer(self.out_buffer, (T, self.hidden_size), ctx.dtype)
    ops.linear(out, heads, self.w_o)
    return out


class RglruMixer(Mixer):
  """A recurrent block around a real-gated linear recurrent unit.  Two branches of ``channels`` values:

    ``y = gelu_tanh(W_y h + b_y)``;   ``u = conv(W_x h + b_x) + conv_bias`` (causal, per channel, ``taps`` taps, no activation);
    u in ``blocks`` equal parts, in each part ``b``:  ``r = sigmoid(Ra[b] u_b + ra_bias[b])``,  ``i = sigmoid(Ri[b] u_b + ri_bias[b])``;
    ``log a = -rate * r * softplus(lam)``,  ``S <- a S + sqrt(1 - a^2) * i * u``  per channel, from zero;   out = ``W_o (S * y)``.

  ``rate`` is the design's constant 8.  Gates, decays and the state are float32.  What the mixer keeps for a request: the
  convolution's last ``taps - 1`` inputs (with their bias), then ``S``.  One fused product gives both branches; the two gate
  matrices of a part are stacked, so one batched product gives both logits.  File tensors (after ``<name>.``): ``y``, ``y.b``,
  ``x``, ``x.b``, ``conv``, ``conv.b``, ``ra``, ``ra.b``, ``ri``, ``ri.b``, ``lam``, ``o``."""

  def __init__(self, name: str, hidden_size: int, channels: int, blocks: int, taps: int, tensors: Optional[Dict[str, str]] = None):
    super().__init__(name)
    if channels <= 0 or blocks <= 0 or taps <= 0 or channels % blocks:
      raise ValueError(f"{name}: {channels} channels must split into {blocks} equal parts, and the convolution needs taps (got {taps})")
    self.hidden_size, self.channels, self.blocks, self.taps = hidden_size, channels, blocks, taps
    self.part = channels // blocks
    t = {"y": "y", "y_b": "y.b", "x": "x", "x_b": "x.b", "conv": "conv", "conv_b": "conv.b", "ra": "ra", "ra_b": "ra.b", "ri": "ri",
         "ri_b": "ri.b", "lam": "lam", "o": "o"}
    t.update(tensors or {})
    self.tensors = t
    self.conv_floats = (taps - 1) * channels

  def cache_spec(self) -> Optional[CacheSpec]:
    return FixedStateSpec((self.conv_floats + self.channels,), "float32")

  def param_specs(self) -> Dict[str, ParamSpec]:
    W, C, B, P, K, n, t = self.hidden_size, self.channels, self.blocks, self.part, self.taps, self.name, self.tensors
    # rows b * 2P .. of the stacked gate matrix: part b's Ra, then its Ri
    gates = [p for b in range(B) for p in (Piece(f"{n}.{t['ra']}", 2 * P * b, (P, P), part=b, of=B),
                                           Piece(f"{n}.{t['ri']}", 2 * P * b + P, (P, P), part=b, of=B))]
    return {
      "w_in": ParamSpec((2 * C, W), "matrix", [[Piece(f"{n}.{t['x']}", 0, (C, W)), Piece(f"{n}.{t['y']}", C, (C, W))]]),
      "x_b": ParamSpec((C,), "vector", [whole(f"{n}.{t['x_b']}", (C,))], init="half_noise"),
      "y_b": ParamSpec((C,), "vector", [whole(f"{n}.{t['y_b']}", (C,))], init="half_noise"),
      "conv": ParamSpec((C, K), "vector", [whole(f"{n}.{t['conv']}", (C, K))], init="half_noise"),
      "conv_b": ParamSpec((C,), "vector", [whole(f"{n}.{t['conv_b']}", (C,))]),
      "gates": ParamSpec((2 * C, P), "matrix", [gates], init="fan_in"),
      "ra_b": ParamSpec((B, P), "vector", [whole(f"{n}.{t['ra_b']}", (B, P))]),
      "ri_b": ParamSpec((B, P), "vector", [whole(f"{n}.{t['ri_b']}", (B, P))]),
      "lam": ParamSpec((C,), "vector", [whole(f"{n}.{t['lam']}", (C,))]),
      "w_o": ParamSpec((W, C), "matrix", [whole(f"{n}.{t['o']}", (W, C))]),
    }

  def bind(self, params) -> None:
    super().bind(params)
    for k in ("ra_b", "ri_b"):      # one bias a channel, the parts one after the other
      if k in params:
        setattr(self, k, params[k].reshape(-1))

  def validate(self, dtype: torch.dtype) -> None:
    if self.taps > 16:
      raise ValueError(f"{self.name}: the convolution takes up to 16 taps, got {self.taps}")
    if dtype == torch.bfloat16 and (self.hidden_size % 8 or self.channels % 8):
      raise ValueError(f"{self.name}: width={self.hidden_size} and channels={self.channels} must be multiples of 8 in bfloat16 "
                       f"(rows are read 16 bytes at a time)")

  def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
    T = x.shape[0]
    C, B, P = self.channels, self.blocks, self.part
    state = _state_rows(cache, self.name)
    proj = ctx.ws.buffer("rglru_proj", (T, 2 * C), ctx.dtype)
    ops.linear(proj, x, self.w_in)
    u = ctx.ws.buffer("rglru_u", (T, C), ctx.dtype)
    ops.causal_conv(u, proj[:, :C], self.conv, self.conv_b, state[:, :max(self.conv_floats, 1)], ctx, silu=False, in_bias=self.x_b)
    if T > ops.SKINNY_BEST_M and ctx.dtype == torch.bfloat16 and P % 8 == 0:
      # many rows: the parts' products on the tensor cores, each leaving its part's logits side by side
      gates = ctx.ws.buffer("rglru_gates", (B, T, 2 * P), torch.float32)
      ops.linear_parts(gates, u, self.gates.view(B, 2 * P, P))
    else:
      gates = ctx.ws.buffer("rglru_gates", (T, 2 * C), torch.float32)
      ops.linear_batched(gates.view(T, B, 2 * P), u.view(T, B, P), self.gates.view(B, 2 * P, P))
    s = ctx.ws.buffer("rglru_s", (T, C), ctx.dtype)
    ops.rglru_recurrence(s, u, gates, proj[:, C:], self.ra_b, self.ri_b, self.y_b, self.lam, state[:, self.conv_floats:], ctx, B, workspace=ctx.ws)
    out = ctx.ws.buffer(self.out_buffer, (T, self.hidden_size), ctx.dtype)
    ops.linear(out, s, self.w_o)
    return out


class MinGruMixer(Mixer):
  """A gated recurrence whose gates read only the current token (minGRU), over ``channels`` channels:

    ``z = sigmoid(W_z h + b_z)``;  ``x = W_x h + b_x``;  the candidate ``c = x + 1/2`` where ``x >= 0`` and ``sigmoid(x)`` below;
    ``S <- (1 - z) S + z c``  per channel, from zero;   out = ``W_o (S * silu(W_g h))``.

  The gate, the candidate and the state are float32; the state is all the mixer keeps for a request.  One fused product gives
  z's logits, x and g.  File tensors (after ``<name>.``): ``z``, ``z.b``, ``x``, ``x.b``, ``g``, ``o``."""

  def __init__(self, name: str, hidden_size: int, channels: int, tensors: Optional[Dict[str, str]] = None):
    super().__init__(name)
    if channels <= 0:
      raise ValueError(f"{name}: channels must be positive, got {channels}")
    self.hidden_size, self.channels = hidden_size, channels
    t = {"z": "z", "z_b": "z.b", "x": "x", "x_b": "x.b", "g": "g", "o": "o"}
    t.update(tensors or {})
    self.tensors = t

  def cache_spec(self) -> Optional[CacheSpec]:
    return FixedStateSpec((self.channels,), "float32")

  def param_specs(self) -> Dict[str, ParamSpec]:
    W, C, n, t = self.hidden_size, self.channels, self.name, self.tensors
    return {
      "w_in": ParamSpec((3 * C, W), "matrix", [[Piece(f"{n}.{t['z']}", 0, (C, W)), Piece(f"{n}.{t['x']}", C, (C, W)),
                                                Piece(f"{n}.{t['g']}", 2 * C, (C, W))]]),
      "z_b": ParamSpec((C,), "vector", [whole(f"{n}.{t['z_b']}", (C,))], init="half_noise"),
      "x_b": ParamSpec((C,), "vector", [whole(f"{n}.{t['x_b']}", (C,))], init="half_noise"),
      "w_o": ParamSpec((W, C), "matrix", [whole(f"{n}.{t['o']}", (W, C))]),
    }

  def validate(self, dtype: torch.dtype) -> None:
    if dtype == torch.bfloat16 and (self.hidden_size % 8 or self.channels % 8):
      raise ValueError(f"{self.name}: width={self.hidden_size} and channels={self.channels} must be multiples of 8 in bfloat16 "
                       f"(rows are read 16 bytes at a time)")

  def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
    T = x.shape[0]
    C = self.channels
    state = _state_rows(cache, self.name)
    proj = ctx.ws.buffer("mingru_proj", (T, 3 * C), ctx.dtype)
    ops.linear(proj, x, self.w_in)
    s = ctx.ws.buffer("mingru_s", (T, C), ctx.dtype)
    ops.mingru_recurrence(s, proj, self.z_b, self.x_b, state, ctx, workspace=ctx.ws)
    out = ctx.ws.buffer(self.out_buffer, (T, self.hidden_size), ctx.dtype)
    ops.linear(out, s, self.w_o)
    return out
