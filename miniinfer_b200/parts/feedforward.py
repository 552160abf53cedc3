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
  """A mixture of ``num_experts`` small SwiGLU feed-forward layers of which each token uses ``top``.

  Router logits ``z = W_router h`` accumulated in float32 by the engine's matrix product (in bfloat16 mode both operands
  are bfloat16, whose products are exact in float32) and scores ``s = sigmoid(z)`` in float32.  The experts of the ``top`` largest ``s + correction`` are chosen;
  their weights are their ``s`` (without the correction) divided by the sum of those ``s`` (+ 1e-20); the output is
  the weighted sum of the chosen experts' outputs.  The experts' matrices are stacked: ``gate_up [E, 2 ff, H]`` (an
  expert's gate rows, then its up rows), ``down [E, H, ff]``.  File tensors: ``<name>.router``, ``<name>.correction``,
  ``<name>.e<i>.gate`` / ``.up`` / ``.down``."""

  def __init__(self, name: str, hidden_size: int, expert_size: int, num_experts: int, top: int):
    super().__init__(name)
    if not (1 <= top <= num_experts):
      raise ValueError(f"{name}: top={top} must lie in 1..experts={num_experts}")
    self.hidden_size = hidden_size
    self.expert_size = expert_size
    self.num_experts = num_experts
    self.top = top

  def param_specs(self) -> Dict[str, ParamSpec]:
    H, F, E, n = self.hidden_size, self.expert_size, self.num_experts, self.name
    gate_up = [p for e in range(E) for p in (Piece(f"{n}.e{e}.gate", 2 * F * e, (F, H)), Piece(f"{n}.e{e}.up", 2 * F * e + F, (F, H)))]
    down = [Piece(f"{n}.e{e}.down", H * e, (H, F)) for e in range(E)]
    return {
      "router": ParamSpec((E, H), "matrix", [whole(f"{n}.router", (E, H))], init="fan_in"),
      "correction": ParamSpec((E,), "vector", [whole(f"{n}.correction", (E,))]),
      "gate_up": ParamSpec((2 * F * E, H), "matrix", [gate_up]),
      "down": ParamSpec((H * E, F), "matrix", [down]),
    }

  def validate(self, dtype: torch.dtype) -> None:
    if self.num_experts > 256 or self.top > 32:
      raise ValueError(f"{self.name}: the routing kernel takes up to 256 experts and top up to 32")
    if dtype == torch.bfloat16:
      for what, k in (("hidden_size", self.hidden_size), ("expert_size", self.expert_size)):
        if k % 8:
          raise ValueError(f"{self.name}: {what}={k} must be a multiple of 8 in bfloat16 (rows are read 16 bytes at a time)")

  def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
    H, F, E = self.hidden_size, self.expert_size, self.num_experts
    out = ctx.ws.buffer("ffn_out", (x.shape[0], H), ctx.dtype)
    ops.routed_experts(out, x, self.router, self.correction, self.gate_up.view(E, 2 * F, H), self.down.view(E, H, F),
                       self.top, ctx.ws)
    return out
