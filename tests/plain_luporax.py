"""Plain implementation of the Luporax design: whole sequences, no cache, float64 on the CPU, one function per
mechanism, written from the design's equations and sharing nothing with the package.  It also makes the random
weights of the tests (``make_model``), with distributions under which every mechanism moves the logits.

Notation: ``T`` tokens, ``W`` width, ``H`` query heads, ``G`` key/value heads, ``D`` query/key size, ``Dv`` value size,
``C`` channels of a recurrence, ``E`` experts.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch

F64 = torch.float64


# ------------------------------------------------------------------------------------------ small mechanisms


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
  return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
  """RMS norm whose weight is stored around zero."""
  return rms_unit(x, eps) * (1.0 + w)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
  return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(x: torch.Tensor) -> torch.Tensor:
  return x * torch.sigmoid(x)


def token_shift(h: torch.Tensor, shift: torch.Tensor) -> torch.Tensor:
  """h [T, W]: every token moves toward the token before it (zeros before the first), by a factor per channel."""
  before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], 0)
  return h + (before - h) * shift


def rotate_half(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
  """x [T, heads, size]: the first rot.dims values of every head are rotated, value i with value i + dims / 2, by the
  angle position * base^(-2 i / dims); the rest stay."""
  dims, base = int(rot["dims"]), float(rot["base"])
  half = dims // 2
  f = base ** (-2.0 * torch.arange(half, dtype=F64) / dims)
  a = positions.to(F64)[:, None] * f[None, :]
  cos, sin = a.cos()[:, None, :], a.sin()[:, None, :]
  out = x.clone()
  u, v = x[..., :half], x[..., half:dims]
  out[..., :half] = u * cos - v * sin
  out[..., half:dims] = v * cos + u * sin
  return out


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
  """x [T, C], taps [C, K] (the last column weighs the current token), zeros before the start: -> [T, C]."""
  T, C = x.shape
  K = taps.shape[1]
  padded = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x], 0)
  out = torch.zeros_like(x)
  for j in range(K):
    out = out + padded[j:j + T] * taps[:, j]
  return out + bias


def diagonal_recurrence(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
  """S_t = a_t S_(t-1) + b_t element by element from S = 0: a, b [T, C] -> all S_t [T, C]."""
  S = torch.zeros(a.shape[1], dtype=a.dtype)
  out = []
  for t in range(a.shape[0]):
    S = a[t] * S + b[t]
    out.append(S)
  return torch.stack(out) if out else torch.zeros_like(a)


# ------------------------------------------------------------------------------------------ the mixers


def rglru(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
  """The recurrent block around a real-gated linear recurrent unit."""
  C, B = int(m["width"]), int(m["blocks"])
  y = gelu_tanh(h @ W[p + "y"].T + W[p + "y.b"])
  u = causal_conv(h @ W[p + "x"].T + W[p + "x.b"], W[p + "conv"], W[p + "conv.b"])
  ub = u.view(-1, B, C // B)
  r = torch.sigmoid(torch.einsum("boi,tbi->tbo", W[p + "ra"], ub) + W[p + "ra.b"]).reshape(-1, C)
  i = torch.sigmoid(torch.einsum("boi,tbi->tbo", W[p + "ri"], ub) + W[p + "ri.b"]).reshape(-1, C)
  log_a = -8.0 * r * torch.nn.functional.softplus(W[p + "lam"])
  a = torch.exp(log_a)
  S = diagonal_recurrence(a, torch.sqrt(1.0 - a * a) * i * u)
  return (S * y) @ W[p + "o"].T


def mingru(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
  """A gated recurrence whose gates read only the current token."""
  z = torch.sigmoid(h @ W[p + "z"].T + W[p + "z.b"])
  u = h @ W[p + "x"].T + W[p + "x.b"]
  candidate = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
  S = diagonal_recurrence(1.0 - z, z * candidate)
  return (S * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def sigmoid_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
  """Grouped-query attention whose weights are sigmoids of the capped scores, not normalised over the keys."""
  T = h.shape[0]
  H, G, D, Dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
  q = rms_unit(h @ W[p + "q"].T + W[p + "q.b"], eps) * W[p + "q.norm"]
  k = rms_unit(h @ W[p + "k"].T + W[p + "k.b"], eps) * W[p + "k.norm"]
  v = (h @ W[p + "v"].T + W[p + "v.b"]).view(T, G, Dv)
  pos = torch.arange(T)
  q = rotate_half(q.view(T, H, D), pos, m["rot"])
  k = rotate_half(k.view(T, G, D), pos, m["rot"])
  cap = m.get("softcap")
  visible = pos[:, None] >= pos[None, :]
  heads = []
  for i in range(H):
    g = i // (H // G)
    s = (q[:, i] @ k[:, g].T) * float(m["scale"])
    if cap:
      s = float(cap) * torch.tanh(s / float(cap))
    w = torch.sigmoid(s + W[p + "pb"][i]) * visible
    heads.append(w @ v[:, g])
  return torch.cat(heads, -1) @ W[p + "o"].T


def mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, layer: dict, eps: float) -> torch.Tensor:
  kind = layer["type"]
  if kind == "rglru":
    return rglru(h, W, p, layer["mixer"])
  if kind == "mingru":
    return mingru(h, W, p, layer["mixer"])
  if kind == "attention":
    return sigmoid_attention(h, W, p, layer["mixer"], eps)
  raise ValueError(kind)


# ------------------------------------------------------------------------------------------ the feed-forward


def expert(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, limit: float) -> torch.Tensor:
  g = torch.clamp(h @ W[p + "gate"].T, max=limit)
  u = torch.clamp(h @ W[p + "up"].T, -limit, limit)
  return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def mixture(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
  E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
  z = h @ W[p + "router"].T
  chosen = torch.topk(z, top, dim=-1)
  weights = torch.softmax(chosen.values, -1)
  out = torch.zeros_like(h)
  for e in range(E):
    y = expert(h, W, f"{p}e{e}.", float(mlp["expert"]["limit"]))
    share = (weights * (chosen.indices == e)).sum(-1, keepdim=True)
    out = out + share * y
  if mlp.get("shared") is not None:
    out = out + torch.sigmoid(h @ W[p + "shared.sg"].T) * expert(h, W, p + "shared.", float(mlp["shared"]["limit"]))
  return out


# ------------------------------------------------------------------------------------------ the model


def source_layer(cfg: dict, i: int) -> int:
  """The layer whose tensors layer ``i`` uses."""
  while cfg["layers"][i].get("weights_of") is not None:
    i = int(cfg["layers"][i]["weights_of"])
  return i


def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens, layers_out: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
  """Logits [T, vocab] of one sequence (float32); ``layers_out`` receives the residual stream after every layer."""
  W = {k: v.to(F64) for k, v in W.items()}
  eps, m = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
  x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
  for i, layer in enumerate(cfg["layers"]):
    p = f"l{source_layer(cfg, i)}."
    h = token_shift(x, W[p + "shift"])
    x = x + m * norm_one_plus(mixer(h, W, p + "mix.", layer, eps), W[p + "norm1"], eps)
    if layer.get("mlp") is not None:
      x = x + m * norm_one_plus(mixture(x, W, p + "mlp.", layer["mlp"]), W[p + "norm2"], eps)
    if layers_out is not None:
      layers_out.append(x.float().clone())
  return ((norm_one_plus(x, W["final.norm"], eps) @ W["embed"].T) * float(cfg["logit_scale"])).float()


def generate(cfg: dict, W: Dict[str, torch.Tensor], prompt: List[int], n: int) -> List[int]:
  ids = list(prompt)
  for _ in range(n):
    ids.append(int(forward(cfg, W, ids)[-1].argmax()))
  return ids[len(prompt):]
