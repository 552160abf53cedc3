"""Plain implementation of the Famupel design: whole sequences, no cache, float32 on the CPU, one function per
mechanism, written from the design's equations and sharing nothing with the package.  It also makes the random
weights of the tests (``make_model``), with distributions under which every mechanism moves the logits.

Notation: ``T`` tokens, ``W`` width, ``H`` query heads, ``G`` key/value heads, ``D`` query/key size, ``Dv`` value size,
``S`` residual streams.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch


# ------------------------------------------------------------------------------------------ small mechanisms


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
  return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_plain(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
  return rms_unit(x, eps) * w


def silu(x: torch.Tensor) -> torch.Tensor:
  return x * torch.sigmoid(x)


def relu_squared_ff(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
  return (torch.relu(h @ up.T) ** 2) @ down.T


def rotary_frequencies(rot: dict) -> torch.Tensor:
  """Frequencies [dims / 2] in float64.  ``rot``: dims, base and, optionally, scaling {factor, low, high, original}: a
  frequency whose wavelength is shorter than original / high stays, one whose wavelength is longer than original / low
  is divided by factor, and between the two the divided and the plain frequency are blended linearly in
  original / wavelength."""
  dims, base = rot["dims"], float(rot["base"])
  f = base ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
  s = rot.get("scaling")
  if not s:
    return f
  out = f.clone()
  for i in range(dims // 2):
    wavelength = 2 * math.pi / float(f[i])
    if wavelength < s["original"] / s["high"]:
      continue
    if wavelength > s["original"] / s["low"]:
      out[i] = f[i] / s["factor"]
    else:
      t = (s["original"] / wavelength - s["low"]) / (s["high"] - s["low"])
      out[i] = (1 - t) * f[i] / s["factor"] + t * f[i]
  return out


def rotate_half(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
  """x [T, heads, size]: the first rot.dims values of every head are rotated, value i with value i + dims / 2."""
  dims = rot["dims"]
  a = positions.to(torch.float64)[:, None] * rotary_frequencies(rot)[None, :]
  cos, sin = a.cos().float()[:, None, :], a.sin().float()[:, None, :]
  out = x.clone()
  u, v = x[..., :dims // 2], x[..., dims // 2:dims]
  out[..., :dims // 2] = u * cos - v * sin
  out[..., dims // 2:dims] = v * cos + u * sin
  return out


def decayed_linear_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor) -> torch.Tensor:
  """q, k [T, H, D], v [T, H, Dv], decay [T, H, D] (a factor per key channel): S_t = diag(decay_t) S_(t-1) + k_t v_t^T,
  o_t = S_t^T q_t, from S = 0.  -> [T, H, Dv]."""
  T, H, D = q.shape
  S = torch.zeros(H, D, v.shape[-1], dtype=torch.float64)
  out = []
  for t in range(T):
    S = decay[t].double()[:, :, None] * S + k[t].double()[:, :, None] * v[t].double()[:, None, :]
    out.append(torch.einsum("hd,hde->he", q[t].double(), S))
  return torch.stack(out).float()


# ------------------------------------------------------------------------------------------ mixers


def gated_linear_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
  T = h.shape[0]
  H, D, Dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
  q = (h @ W[p + "q"].T).view(T, H, D) * D ** -0.5
  k = (h @ W[p + "k"].T).view(T, H, D)
  v = (h @ W[p + "v"].T).view(T, H, Dv)
  z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
  alpha = torch.exp(torch.nn.functional.logsigmoid(z) / tau).view(T, H, D)
  o = decayed_linear_attention(q, k, v, alpha)
  o = norm_plain(o, W[p + "norm"], eps).reshape(T, H * Dv)
  return (o * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def softmax_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
  T = h.shape[0]
  H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
  pos = torch.arange(T)
  q = h @ W[p + "q"].T + W[p + "q.b"]
  k = h @ W[p + "k"].T + W[p + "k.b"]
  v = (h @ W[p + "v"].T + W[p + "v.b"]).view(T, G, Dv)
  q = norm_plain(q, W[p + "q.norm"], eps).view(T, H, D)       # over the whole projection, before the heads are split
  k = norm_plain(k, W[p + "k.norm"], eps).view(T, G, D)
  q, k = rotate_half(q, pos, m["rot"]), rotate_half(k, pos, m["rot"])
  rep = H // G
  k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
  scores = torch.einsum("ihd,jhd->hij", q, k) * float(m["scale"])
  seen = pos[None, :] <= pos[:, None]
  scores = scores.masked_fill(~seen[None], float("-inf"))
  o = torch.einsum("hij,jhe->ihe", torch.softmax(scores, dim=-1), v).reshape(T, H * Dv)
  return (o * torch.sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T


def retention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
  T = h.shape[0]
  H, D, Dv = m["heads"], m["dim"], m["vdim"]
  pos = torch.arange(T)
  q = rotate_half((h @ W[p + "q"].T).view(T, H, D), pos, m["rot"])
  k = rotate_half((h @ W[p + "k"].T).view(T, H, D), pos, m["rot"]) * D ** -0.5
  v = (h @ W[p + "v"].T).view(T, H, Dv)
  decay = torch.tensor(m["decay"], dtype=torch.float64).float()[None, :, None].expand(T, H, D)
  o = rms_unit(decayed_linear_attention(q, k, v, decay), eps).reshape(T, H * Dv)
  return (o * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, layer: dict, eps: float) -> torch.Tensor:
  m = layer["mixer"]
  if layer["type"] == "gla":
    return gated_linear_attention(h, W, p, m, eps)
  if layer["type"] == "parallel":
    return float(m["left_scale"]) * softmax_attention(h, W, p + "left.", m["left"], eps) + \
      float(m["right_scale"]) * retention(h, W, p + "right.", m["right"], eps)
  raise ValueError(layer["type"])


# ------------------------------------------------------------------------------------------ the model


def hyper_sublayer(xs: torch.Tensor, W: Dict[str, torch.Tensor], p: str, fn) -> torch.Tensor:
  """xs [S, T, W]: the streams.  u = sum_s in[s] x_s; y = fn(u); x_t <- sum_s mix[s, t] x_s + out[t] y."""
  u = torch.einsum("s,stw->tw", W[p + "in"], xs)
  y = fn(u)
  return torch.einsum("st,sjw->tjw", W[p + "mix"], xs) + W[p + "out"][:, None, None] * y[None]


def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens, layers_out: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
  """Logits [T, vocab] of one sequence; ``layers_out`` receives the residual stream (the sum of the streams) after every layer."""
  W = {k: v.float() for k, v in W.items()}
  eps = float(cfg["norm"]["eps"])
  x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
  S = cfg.get("streams")
  xs = x[None].repeat(S, 1, 1) if S else None
  for i, layer in enumerate(cfg["layers"]):
    p = f"l{i}."
    subs = [("1", lambda u, p=p, layer=layer: mixer(norm_plain(u, W[p + "norm1"], eps), W, p + "mix.", layer, eps))]
    if layer.get("mlp") is not None:
      subs.append(("2", lambda u, p=p: relu_squared_ff(norm_plain(u, W[p + "norm2"], eps), W[p + "mlp.up"], W[p + "mlp.down"])))
    for q, fn in subs:
      if S:
        xs = hyper_sublayer(xs, W, f"{p}hc{q}.", fn)
      else:
        x = x + fn(x)
    if layers_out is not None:
      layers_out.append((xs.sum(0) if S else x).clone())
  if S:
    x = xs.sum(0)
  return norm_plain(x, W["final.norm"], eps) @ W["head"].T


# ------------------------------------------------------------------------------------------ weights for the tests


def tensor_shapes(cfg: dict, ranks: Optional[Dict[int, int]] = None) -> Dict[str, tuple]:
  """Name -> shape of every tensor of a model with this configuration (``ranks``: the low rank of a gla layer's decay)."""
  Wd, V, S = cfg["width"], cfg["vocab"], cfg.get("streams")
  out: Dict[str, tuple] = {"embed": (V, Wd), "final.norm": (Wd,), "head": (V, Wd)}
  for i, layer in enumerate(cfg["layers"]):
    p, m = f"l{i}.", layer["mixer"]
    out[p + "norm1"] = (Wd,)
    if layer["type"] == "gla":
      H, D, Dv, r = m["heads"], m["dim"], m["vdim"], (ranks or {}).get(i, 8)
      out.update({p + "mix.q": (H * D, Wd), p + "mix.k": (H * D, Wd), p + "mix.v": (H * Dv, Wd), p + "mix.g": (H * Dv, Wd),
                  p + "mix.o": (Wd, H * Dv), p + "mix.norm": (Dv,), p + "mix.a1": (r, Wd), p + "mix.a2": (H * D, r), p + "mix.a2.b": (H * D,)})
    else:
      l, r = m["left"], m["right"]
      H, G, D, Dv = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
      q = p + "mix.left."
      out.update({q + "q": (H * D, Wd), q + "q.b": (H * D,), q + "k": (G * D, Wd), q + "k.b": (G * D,), q + "v": (G * Dv, Wd),
                  q + "v.b": (G * Dv,), q + "q.norm": (H * D,), q + "k.norm": (G * D,), q + "g": (H * Dv, Wd), q + "o": (Wd, H * Dv)})
      H, D, Dv = r["heads"], r["dim"], r["vdim"]
      q = p + "mix.right."
      out.update({q + "q": (H * D, Wd), q + "k": (H * D, Wd), q + "v": (H * Dv, Wd), q + "g": (H * Dv, Wd), q + "o": (Wd, H * Dv)})
    subs = ["1"]
    if layer.get("mlp") is not None:
      out.update({p + "norm2": (Wd,), p + "mlp.up": (layer["mlp"]["ff"], Wd), p + "mlp.down": (Wd, layer["mlp"]["ff"])})
      subs.append("2")
    if S:
      for q in subs:
        out.update({f"{p}hc{q}.in": (S,), f"{p}hc{q}.out": (S,), f"{p}hc{q}.mix": (S, S)})
  return out


def make_model(cfg: dict, seed: int, ranks: Optional[Dict[int, int]] = None) -> Dict[str, torch.Tensor]:
  """Random weights, all exactly representable in bfloat16, under which every mechanism moves the logits: projections
  with a fan-in scale, norm weights around one, biases of the size of the projections' outputs, decay biases that keep
  the gated layers' memories between a few and a few hundred tokens, stream matrices near the identity with clear
  off-diagonal parts."""
  g = torch.Generator().manual_seed(seed)
  W: Dict[str, torch.Tensor] = {}
  S = cfg.get("streams")
  for name, shape in tensor_shapes(cfg, ranks).items():
    last = name.split(".")[-1]
    if name == "embed":
      t = torch.randn(shape, generator=g)
    elif last in ("norm", "norm1", "norm2") or name == "final.norm":
      t = 1.0 + 0.3 * torch.randn(shape, generator=g)
    elif name.endswith("a2.b"):
      t = 3.0 + 2.0 * torch.randn(shape, generator=g)
    elif last == "b":
      t = 0.5 * torch.randn(shape, generator=g)
    elif last == "in":
      t = 1.0 / S + 0.3 * torch.randn(shape, generator=g)
    elif last == "out":
      t = 1.0 + 0.3 * torch.randn(shape, generator=g)
    elif last == "mix":
      t = torch.eye(S) + 0.25 * torch.randn(shape, generator=g)
    else:
      t = torch.randn(shape, generator=g) * (1.5 if last in ("q", "k") else 1.0) / math.sqrt(shape[-1])
    W[name] = t.to(torch.bfloat16).float()
  return W


def write_model(cfg: dict, W: Dict[str, torch.Tensor], folder: str, dtype: torch.dtype = torch.bfloat16) -> str:
  from safetensors.torch import save_file
  os.makedirs(folder, exist_ok=True)
  with open(os.path.join(folder, "config.json"), "w") as f:
    json.dump(cfg, f)
  save_file({k: v.to(dtype).contiguous() for k, v in W.items()}, os.path.join(folder, "model.safetensors"))
  return folder


def make_model_dir(cfg: dict, folder: str, seed: int, ranks: Optional[Dict[int, int]] = None) -> str:
  return write_model(cfg, make_model(cfg, seed, ranks), folder)


def read_weights(model_dir: str) -> Dict[str, torch.Tensor]:
  from safetensors.torch import load_file
  return {k: v.float() for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}


def read_config(model_dir: str) -> dict:
  with open(os.path.join(model_dir, "config.json"), encoding="utf-8") as f:
    return json.load(f)


def generate(cfg: dict, W: Dict[str, torch.Tensor], prompt: List[int], n: int) -> List[int]:
  ids = list(prompt)
  for _ in range(n):
    ids.append(int(forward(cfg, W, ids)[-1].argmax()))
  return ids[len(prompt):]


# ------------------------------------------------------------------------------------------ configurations


def dense(ff) -> dict:
  return {"kind": "dense", "ff": ff}


def gla(heads, dim, vdim, tau, mlp) -> dict:
  return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "mlp": mlp}


def rot_of(dims, base, scaling=None) -> dict:
  r = {"dims": dims, "base": base}
  if scaling is not None:
    r["scaling"] = scaling
  return r


def pair(left: dict, right: dict, left_scale, right_scale, mlp) -> dict:
  return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}, "mlp": mlp}


def left_of(heads, kv_heads, dim, vdim, rot, scale) -> dict:
  return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rot, "scale": scale}


def right_of(heads, dim, vdim, rot, decay) -> dict:
  return {"heads": heads, "dim": dim, "vdim": vdim, "rot": rot, "decay": decay}


# Three configurations that differ in every size, in the order of their layers and in what is there at all: A has three
# streams, a layer without a feed-forward, grouped and ungrouped attention heads, rotations over a part of a head with
# all three bands of the frequency scaling, and odd sizes (a key size that is no multiple of 16, more value than key
# channels and the reverse); B has no streams (the usual residual sum), starts with a pair, and rotates whole heads
# without scaling; C has one stream (its hyper-connection weights still act), heads of 64 and 128 values for the
# tensor-core attention kernels, key sizes past 128 in the linear attention, and decays of 0 and 1.
CONFIGS = {
  "A": {"architecture": "Famupel", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "streams": 3, "layers": [
    gla(3, 20, 24, 8.0, dense(96)),
    pair(left_of(4, 1, 24, 16, rot_of(16, 10000.0, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}), 0.3),
         right_of(2, 24, 40, rot_of(8, 5000.0), [0.9, 0.996]), 0.7, 1.3, dense(80)),
    gla(1, 40, 16, 4.0, None),
    pair(left_of(2, 2, 16, 32, rot_of(8, 100.0), 0.25), right_of(3, 16, 8, rot_of(16, 300.0), [0.5, 0.97, 0.999]), 1.2, 0.6, None),
    gla(2, 16, 16, 1.0, dense(72))]},
  "B": {"architecture": "Famupel", "vocab": 512, "width": 96, "norm": {"eps": 1e-6}, "layers": [
    pair(left_of(6, 3, 32, 32, rot_of(32, 50000.0), 0.2), right_of(2, 48, 24, rot_of(48, 10000.0), [0.98, 0.9]), 1.0, 1.0, dense(128)),
    gla(4, 24, 8, 32.0, dense(64)),
    gla(2, 32, 48, 2.0, None)]},
  "C": {"architecture": "Famupel", "vocab": 333, "width": 128, "norm": {"eps": 1e-6}, "streams": 1, "layers": [
    gla(1, 160, 32, 16.0, dense(160)),
    pair(left_of(4, 2, 64, 128, rot_of(64, 500000.0, {"factor": 2.0, "low": 2.0, "high": 8.0, "original": 128}), 0.125),
         right_of(2, 64, 64, rot_of(32, 10000.0), [1.0, 0.0]), 0.5, 2.0, dense(96)),
    pair(left_of(2, 1, 128, 64, rot_of(32, 10000.0), 0.09), right_of(1, 136, 16, rot_of(136, 10000.0), [0.99]), 1.0, 1.0, dense(64))]},
}
RANKS = {"A": {0: 8, 2: 4, 4: 16}, "B": {1: 12, 2: 8}, "C": {0: 16}}
