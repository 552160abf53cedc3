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


# ------------------------------------------------------------------------------------------ weights for the tests


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
  """Name -> shape of every tensor of a model with this configuration (layers that run another's weights have none)."""
  Wd, V = cfg["width"], cfg["vocab"]
  out: Dict[str, tuple] = {"embed": (V, Wd), "final.norm": (Wd,)}
  for i, layer in enumerate(cfg["layers"]):
    if layer.get("weights_of") is not None:
      continue
    p, m, q = f"l{i}.", layer["mixer"], f"l{i}.mix."
    out.update({p + "norm1": (Wd,), p + "shift": (Wd,)})
    if layer["type"] == "attention":
      H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
      out.update({q + "q": (H * D, Wd), q + "q.b": (H * D,), q + "k": (G * D, Wd), q + "k.b": (G * D,), q + "v": (G * Dv, Wd),
                  q + "v.b": (G * Dv,), q + "q.norm": (H * D,), q + "k.norm": (G * D,), q + "pb": (H,), q + "o": (Wd, H * Dv)})
    elif layer["type"] == "rglru":
      C, B, K = m["width"], m["blocks"], m["conv"]
      out.update({q + "y": (C, Wd), q + "y.b": (C,), q + "x": (C, Wd), q + "x.b": (C,), q + "conv": (C, K), q + "conv.b": (C,),
                  q + "ra": (B, C // B, C // B), q + "ra.b": (B, C // B), q + "ri": (B, C // B, C // B), q + "ri.b": (B, C // B),
                  q + "lam": (C,), q + "o": (Wd, C)})
    else:
      C = m["width"]
      out.update({q + "z": (C, Wd), q + "z.b": (C,), q + "x": (C, Wd), q + "x.b": (C,), q + "g": (C, Wd), q + "o": (Wd, C)})
    mlp = layer.get("mlp")
    if mlp is not None:
      q, F = p + "mlp.", mlp["expert"]["ff"]
      out[p + "norm2"] = (Wd,)
      out[q + "router"] = (mlp["router"]["experts"], Wd)
      for e in range(mlp["router"]["experts"]):
        out.update({f"{q}e{e}.gate": (F, Wd), f"{q}e{e}.up": (F, Wd), f"{q}e{e}.down": (Wd, F)})
      if mlp.get("shared") is not None:
        S = mlp["shared"]["ff"]
        out.update({q + "shared.gate": (S, Wd), q + "shared.up": (S, Wd), q + "shared.down": (Wd, S), q + "shared.sg": (1, Wd)})
  return out


def make_model(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
  """Random weights, all exactly representable in bfloat16, under which every mechanism moves the logits: projections with
  a fan-in scale (the experts' gate and up rows larger, so that the clamps bite), norm weights around zero, biases of the
  size of the projections' outputs, shifts between 0 and 1, decays that keep a memory between a few and a few hundred
  tokens, routers whose largest logits stand apart."""
  g = torch.Generator().manual_seed(seed)
  W: Dict[str, torch.Tensor] = {}
  for name, shape in tensor_shapes(cfg).items():
    last = name.split(".")[-1]
    r = torch.randn(shape, generator=g)
    if name == "embed":
      t = r
    elif last in ("norm1", "norm2") or name == "final.norm":
      t = 0.3 * r
    elif last == "norm":
      t = 1.0 + 0.3 * r
    elif last == "shift":
      t = torch.rand(shape, generator=g)
    elif last == "lam":
      t = -3.5 + 1.2 * r
    elif last == "pb":
      t = -1.0 + 0.7 * r
    elif last == "b":
      t = 0.5 * r
    elif last == "conv":
      t = 0.5 * r
    elif last == "router":
      t = r * 4.0 / math.sqrt(shape[-1])
    elif last in ("ra", "ri"):
      t = r * 2.0 / math.sqrt(shape[-1])
    elif last in ("gate", "up"):
      t = r * 2.0 / math.sqrt(shape[-1])
    else:
      t = r * (1.5 if last in ("q", "k") else 1.0) / math.sqrt(shape[-1])
    W[name] = t.to(torch.bfloat16).float()
  return W


def write_model(cfg: dict, W: Dict[str, torch.Tensor], folder: str, dtype: torch.dtype = torch.bfloat16) -> str:
  from safetensors.torch import save_file
  os.makedirs(folder, exist_ok=True)
  with open(os.path.join(folder, "config.json"), "w") as f:
    json.dump(cfg, f)
  save_file({k: v.to(dtype).contiguous() for k, v in W.items()}, os.path.join(folder, "model.safetensors"))
  return folder


def make_model_dir(cfg: dict, folder: str, seed: int) -> str:
  return write_model(cfg, make_model(cfg, seed), folder)


def read_weights(model_dir: str) -> Dict[str, torch.Tensor]:
  from safetensors.torch import load_file
  return {k: v.float() for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}


def read_config(model_dir: str) -> dict:
  with open(os.path.join(model_dir, "config.json"), encoding="utf-8") as f:
    return json.load(f)


# ------------------------------------------------------------------------------------------ configurations


def moe(ff, limit, experts, top, shared=None) -> dict:
  d = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
  if shared is not None:
    d["shared"] = {"ff": shared[0], "limit": shared[1]}
  return d


def attention(heads, kv_heads, dim, vdim, rot_dims, base, scale, softcap, mlp, weights_of=None) -> dict:
  m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": {"dims": rot_dims, "base": base}, "scale": scale}
  if softcap is not None:
    m["softcap"] = softcap
  return _layer("attention", m, mlp, weights_of)


def rglru_layer(width, blocks, conv, mlp, weights_of=None) -> dict:
  return _layer("rglru", {"width": width, "blocks": blocks, "conv": conv}, mlp, weights_of)


def mingru_layer(width, mlp, weights_of=None) -> dict:
  return _layer("mingru", {"width": width}, mlp, weights_of)


def _layer(kind, mixer, mlp, weights_of) -> dict:
  d = {"type": kind, "mixer": mixer, "mlp": mlp}
  if weights_of is not None:
    d["weights_of"] = weights_of
  return d


# Three configurations that differ in every size, in the order of their layers and in what is there at all.  A: a rotation
# over a part of a head, one key/value head for four query heads, key and value sizes that differ and are no multiple of
# 16, three parts in the recurrent unit, a layer without a feed-forward, layers that run another's weights (one of them
# twice).  B: as many key/value heads as query heads, the whole head rotated, no cap on the scores, a recurrent unit of
# one part whose convolution has one tap, a router that takes all of its experts and one that takes one, a feed-forward
# without a shared expert, multipliers of 1.  C: heads of 64 (the tensor-core and tensor-copy kernels), pages of 64.  D: odd
# sizes - a width of 72, a vocabulary of 333, sixteen query heads on one key/value head, a cap of 5 that bites, a rotation
# of 8 of 32 values, a convolution of 7 taps over 5 parts of 8 channels, 40 experts of which a token takes 6, a multiplier
# above 1 and an eps of 1e-3.
_A_MLP = moe(24, 1.5, 5, 2, (16, 0.8))
_C_MLP = moe(64, 2.5, 8, 3, (96, 1.2))
CONFIGS = {
  "A": {"architecture": "Luporax", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 0.5, "logit_scale": 0.3, "layers": [
    mingru_layer(40, _A_MLP),
    attention(4, 1, 24, 16, 16, 10000.0, 0.3, 20.0, _A_MLP),
    rglru_layer(48, 3, 3, None),
    attention(4, 1, 24, 16, 16, 10000.0, 0.3, 20.0, _A_MLP, weights_of=1),
    rglru_layer(48, 3, 3, None, weights_of=2),
    attention(4, 1, 24, 16, 16, 10000.0, 0.3, 20.0, _A_MLP, weights_of=3)]},
  "B": {"architecture": "Luporax", "vocab": 200, "width": 32, "norm": {"eps": 1e-6}, "residual_mult": 1.0, "logit_scale": 1.0, "layers": [
    rglru_layer(32, 1, 1, moe(16, 3.0, 3, 3)),
    attention(2, 2, 16, 32, 16, 500.0, 0.25, None, moe(24, 1.0, 4, 1, (8, 2.0))),
    mingru_layer(16, None)]},
  "C": {"architecture": "Luporax", "vocab": 500, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 0.8, "logit_scale": 0.5, "layers": [
    attention(8, 2, 64, 64, 32, 20000.0, 0.125, 30.0, _C_MLP),
    rglru_layer(96, 2, 4, _C_MLP),
    mingru_layer(160, _C_MLP),
    attention(8, 2, 64, 64, 32, 20000.0, 0.125, 30.0, _C_MLP, weights_of=0)]},
  "D": {"architecture": "Luporax", "vocab": 333, "width": 72, "norm": {"eps": 1e-3}, "residual_mult": 1.3, "logit_scale": 0.07, "layers": [
    rglru_layer(40, 5, 7, moe(16, 0.5, 40, 6, (8, 3.0))),
    attention(16, 1, 32, 48, 8, 3000.0, 0.9, 5.0, moe(16, 0.5, 40, 6, (8, 3.0))),
    attention(16, 1, 32, 48, 8, 3000.0, 0.9, 5.0, moe(16, 0.5, 40, 6, (8, 3.0)), weights_of=1),
    mingru_layer(24, None)]},
}
