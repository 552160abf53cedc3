"""Dense SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))`` with gate and up in one matrix
(miniinfer/models/fused_qwen3.py:111-138; order gate, up: miniinfer/loader/weight.py:87-93).
"""

from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..kernels import ops
from .base import FeedForward, ParamSpec, Piece, whole


class SwiGLUFeedForward(FeedForward):
  """``tensors``: the file names of the gate, up and down matrices after ``<name>.`` (default: ``gate_proj.weight``,
  ``up_proj.weight``, ``down_proj.weight``, with ``gate_up_proj.weight`` accepted for the fused pair)."""

  def __init__(self, name: str, hidden_size: int, intermediate_size: int, tensors: Optional[Tuple[str, str, str]] = None):
    super().__init__(name)
    self.hidden_size = hidden_size
    self.intermediate_size = intermediate_size
    self.tensors = tensors

  def param_specs(self) -> Dict[str, ParamSpec]:
    H, I = self.hidden_size, self.intermediate_size
    if self.tensors is not None:
      g, u, d = (f"{self.name}.{t}" for t in self.tensors)
      return {"gate_up": ParamSpec((2 * I, H), "matrix", [[Piece(g, 0, (I, H)), Piece(u, I, (I, H))]]),
              "down": ParamSpec((H, I), "matrix", [whole(d, (H, I))])}
    return {
      "gate_up": ParamSpec((2 * I, H), "matrix", [
        [Piece(f"{self.name}.gate_proj.weight", 0, (I, H)), Piece(f"{self.name}.up_proj.weight", I, (I, H))],
        whole(f"{self.name}.gate_up_proj.weight", (2 * I, H)),
      ]),
      "down": ParamSpec((H, I), "matrix", [whole(f"{self.name}.down_proj.weight", (H, I))]),
    }

  def validate(self, dtype: torch.dtype) -> None:
    if dtype == torch.bfloat16:
      for what, k in (("hidden_size", self.hidden_size), ("intermediate_size", self.intermediate_size)):
        if k % 8:
          raise ValueError(f"{self.name}: {what}={k} must be a multiple of 8 in bfloat16 (rows are read 16 bytes at a time)")

  def takes_residual(self, norm, ctx) -> bool:
    return norm.as_rms() is not None and ops.fuses_few_rows(ctx.num_tokens, ctx.dtype)

  def forward_on_residual(self, resid: torch.Tensor, norm, ctx) -> None:
    """Two kernels: norm + gate-and-up product + SwiGLU, then the down product + residual add."""
    weight, eps = norm.as_rms()
    act = ctx.ws.buffer("ffn_act", (resid.shape[0], self.intermediate_size), ctx.dtype)
    ops.linear_swiglu_normed(act, resid, weight, eps, self.gate_up)
    ops.linear_add(resid, act, self.down)

  def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
    T = x.shape[0]
    act = ctx.ws.buffer("ffn_act", (T, self.intermediate_size), ctx.dtype)
    ops.linear_swiglu(act, x, self.gate_up, ctx.ws)
    out = ctx.ws.buffer("ffn_out", (T, self.hidden_size), ctx.dtype)
    ops.linear(out, act, self.down)
    return out


class ActivatedFeedForward(FeedForward):
  """Dense feed-forward of two matrices with an activation between them: ``down(act(up(x)))``.  ``activation``:
  ``relu_squared`` (``max(z, 0)^2``).  ``tensors``: the file names of the up and down matrices after ``<name>.``."""

  ACTIVATIONS = ("relu_squared",)

  def __init__(self, name: str, hidden_size: int, intermediate_size: int, activation: str = "relu_squared",
               tensors: Tuple[str, str] = ("up", "down")):
    super().__init__(name)
    if activation not in self.ACTIVATIONS:
      raise ValueError(f"{name}: activation {activation!r} is not known ({', '.join(self.ACTIVATIONS)})")
    self.hidden_size = hidden_size
    self.intermediate_size = intermediate_size
    self.activation = activation
    self.tensors = tuple(tensors)

  def param_specs(self) -> Dict[str, ParamSpec]:
    H, I = self.hidden_size, self.intermediate_size
    u, d = (f"{self.name}.{t}" for t in self.tensors)
    return {"up": ParamSpec((I, H), "matrix", [whole(u, (I, H))]), "down": ParamSpec((H, I), "matrix", [whole(d, (H, I))])}

  def validate(self, dtype: torch.dtype) -> None:
    if dtype == torch.bfloat16:
      for what, k in (("hidden_size", self.hidden_size), ("intermediate_size", self.intermediate_size)):
        if k % 8:
          raise ValueError(f"{self.name}: {what}={k} must be a multiple of 8 in bfloat16 (rows are read 16 bytes at a time)")

  def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
    T = x.shape[0]
    act = ctx.ws.buffer("ffn_act", (T, self.intermediate_size), ctx.dtype)
    ops.linear_relu_squared(act, x, self.up, ctx.ws)
    out = ctx.ws.buffer("ffn_out", (T, self.hidden_size), ctx.dtype)
    ops.linear(out, act, self.down)
    return out


class RoutedExpertsFeedForward(FeedForward):
  """A mixture of ``num_experts`` small gated feed-forward layers of which each token uses ``top``.

  Router logits ``z = W_router h`` accumulated in float32 by the engine's matrix product (in bfloat16 mode both operands
  are bfloat16, whose products are exact in float32).  ``router_weights="sigmoid_share"``: scores ``s = sigmoid(z)`` in float32;
  the experts of the ``top`` largest ``s + correction`` are chosen; their weights are their ``s`` (without the correction)
  divided by the sum of those ``s`` (+ 1e-20).  ``router_weights="softmax_chosen"``: the ``top`` largest logits are chosen, the
  weights are the softmax over the chosen logits alone, and there is no correction.  The output is the weighted sum of the
  chosen experts' outputs.

  An expert is ``down(act(gate x) * up x)`` with ``activation="silu"`` or ``activation="clamped"`` and its ``limit``:
  ``g = min(gate x, limit)``, ``u = clamp(up x, -limit, limit)``, ``g * sigmoid(1.702 g) * (u + 1)``.

  ``shared_size``: an expert of that size more (``shared_limit`` its limit, same form) that every token runs through; its
  output is added to the sum, times ``sigmoid(w_sg . h)`` - one number a token - if ``shared_gate``.  The gate's row rides as
  the last row of the router's matrix, so its logit comes out of the router's product.

  The experts' matrices are stacked: ``gate_up [E, 2 ff, H]`` (an expert's gate rows, then its up rows), ``down [E, H, ff]``.
  File tensors: ``<name>.router``, ``<name>.correction``, ``<name>.e<i>.gate`` / ``.up`` / ``.down``,
  ``<name>.shared.gate`` / ``.up`` / ``.down`` / ``.sg``."""

  def __init__(self, name: str, hidden_size: int, expert_size: int, num_experts: int, top: int, router_weights: str = "sigmoid_share",
               activation: str = "silu", limit: float = 0.0, shared_size: Optional[int] = None, shared_limit: Optional[float] = None,
               shared_gate: bool = False):
    super().__init__(name)
    if not (1 <= top <= num_experts):
      raise ValueError(f"{name}: top={top} must lie in 1..experts={num_experts}")
    if router_weights not in ("sigmoid_share", "softmax_chosen"):
      raise ValueError(f"{name}: router_weights={router_weights!r} is not known (sigmoid_share, softmax_chosen)")
    if activation not in ops.GLU_KINDS or (activation == "clamped" and not limit > 0):
      raise ValueError(f"{name}: activation={activation!r} is not known ({', '.join(ops.GLU_KINDS)}) or its limit {limit!r} is not positive")
    if shared_size is None and shared_gate:
      raise ValueError(f"{name}: a gate for a shared expert that is not there")
    if shared_size is not None and shared_size <= 0:
      raise ValueError(f"{name}: shared_size must be positive, got {shared_size}")
    self.hidden_size = hidden_size
    self.expert_size = expert_size
    self.num_experts = num_experts
    self.top = top
    self.router_weights = router_weights
    self.activation, self.limit = activation, float(limit)
    self.shared_size = shared_size
    self.shared_limit = float(shared_limit) if shared_limit is not None else float(limit)
    self.shared_gate = bool(shared_gate)
    if shared_size is not None and activation == "clamped" and not self.shared_limit > 0:
      raise ValueError(f"{name}: the shared expert's limit must be positive, got {shared_limit!r}")

  def param_specs(self) -> Dict[str, ParamSpec]:
    H, F, E, n = self.hidden_size, self.expert_size, self.num_experts, self.name
    gate_up = [p for e in range(E) for p in (Piece(f"{n}.e{e}.gate", 2 * F * e, (F, H)), Piece(f"{n}.e{e}.up", 2 * F * e + F, (F, H)))]
    down = [Piece(f"{n}.e{e}.down", H * e, (H, F)) for e in range(E)]
    router = [Piece(f"{n}.router", 0, (E, H))] + ([Piece(f"{n}.shared.sg", E, (1, H))] if self.shared_gate else [])
    specs = {
      "router": ParamSpec((E + (1 if self.shared_gate else 0), H), "matrix", [router], init="fan_in"),
      "gate_up": ParamSpec((2 * F * E, H), "matrix", [gate_up]),
      "down": ParamSpec((H * E, F), "matrix", [down]),
    }
    if self.router_weights == "sigmoid_share":
      specs["correction"] = ParamSpec((E,), "vector", [whole(f"{n}.correction", (E,))])
    if self.shared_size is not None:
      S = self.shared_size
      specs["shared_gate_up"] = ParamSpec((2 * S, H), "matrix", [[Piece(f"{n}.shared.gate", 0, (S, H)), Piece(f"{n}.shared.up", S, (S, H))]])
      specs["shared_down"] = ParamSpec((H, S), "matrix", [whole(f"{n}.shared.down", (H, S))])
    return specs

  def validate(self, dtype: torch.dtype) -> None:
    if self.num_experts > 256 or self.top > 32:
      raise ValueError(f"{self.name}: the routing kernel takes up to 256 experts and top up to 32")
    if dtype == torch.bfloat16:
      for what, k in (("hidden_size", self.hidden_size), ("expert_size", self.expert_size), ("shared_size", self.shared_size or 8)):
        if k % 8:
          raise ValueError(f"{self.name}: {what}={k} must be a multiple of 8 in bfloat16 (rows are read 16 bytes at a time)")

  def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
    H, F, E = self.hidden_size, self.expert_size, self.num_experts
    T = x.shape[0]
    shared = None
    if self.shared_size is not None:
      act = ctx.ws.buffer("ffn_act", (T, self.shared_size), ctx.dtype)
      ops.linear_glu(act, x, self.shared_gate_up, ctx.ws, self.activation, self.shared_limit)
      shared = ctx.ws.buffer("ffn_shared", (T, H), ctx.dtype)
      ops.linear(shared, act, self.shared_down)
    out = ctx.ws.buffer("ffn_out", (T, H), ctx.dtype)
    ops.routed_experts(out, x, self.router, self.correction if self.router_weights == "sigmoid_share" else None,
                       self.gate_up.view(E, 2 * F, H), self.down.view(E, H, F), self.top, ctx.ws, weights=self.router_weights,
                       glu=self.activation, limit=self.limit, shared=shared, shared_gated=self.shared_gate)
    return out
