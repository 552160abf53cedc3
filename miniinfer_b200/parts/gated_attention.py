"""Windowed grouped-query attention with unit-norm queries and keys, a sink in the softmax, values mixed across layers
and an output gate - and, optionally, rotated heads, weights on the head norms, values that are the keys as projected, and
first tokens that stay visible behind the window - as a mixer part over the paged cache.

For the normalised rows ``h`` of a step, with ``H`` query heads, ``G`` key/value heads (query head ``i`` reads
key/value head ``i // (H / G)``), query/key size ``dim`` and value size ``vdim``:

  * one fused product gives ``q``, ``k``, ``v`` and the gate's logits ``g``; with ``biases`` a bias each is added to ``q``,
    ``k`` and ``v`` (float32, file tensors ``q.b``, ``k.b``, ``v.b``);
  * every head of ``q`` and ``k`` is divided by its root mean square, ``x / sqrt(mean(x^2) + eps)`` (float32), and
    multiplied by a weight per dimension shared by all heads if ``norm_weights``; with ``norm_over="projection"`` the root
    mean square runs over the whole of ``q`` (of ``k``) before the heads are split, and the weights have the projection's size;
  * with ``rotary`` (a position encoding that has a table) the first ``rotary_dim`` values of every query and key head are
    then rotated by the token's position, value i with value i + rotary_dim / 2 or, ``rotary_interleaved``, 2i with 2i + 1;
    without it positions do not enter the scores;
  * ``values_from_keys``: there is no value projection; a head's value is its key as projected, before norm and rotation;
  * ``value_mix="mixed"``: ``v <- (1 - lambda) v + lambda v_src`` with ``lambda`` a learned scalar and ``v_src`` the
    values that the layer with ``value_mix="source"`` made for the same token in this step (handed on through
    ``ctx.shared[value_mix_key]``); what is cached is the mixed ``v`` and the normalised ``k``;
  * token ``i`` sees token ``j`` of its request if ``0 <= i - j < window`` (``window`` None: every earlier token) or, with
    ``keep_first``, if ``j < keep_first`` and ``j <= i``: the first tokens stay visible, at their true positions;
  * ``softmax`` over ``scale * q . k`` whose denominator also holds ``exp(sink)`` of the query head (``sinks``), a term
    with no key and no value;
  * ``softcap`` > 0: a scaled score ``s`` becomes ``softcap * tanh(s / softcap)`` before the weights are made;
  * ``weights="sigmoid"``: no softmax - the weight of a visible key is ``sigmoid(s + b)`` with ``b`` a learned number per
    query head (file tensor ``pb``), and the weights are not normalised over the keys (``sinks`` must be off);
  * the heads' outputs, side by side, are multiplied element by element with ``sigmoid(g)`` (``gated``), then projected.

Every option can be switched off, so other designs may take the parts they need.  The cache keeps keys and values in
rows of one size, ``max(dim, vdim)`` rounded up to a multiple of 16 and zero-filled: a zero tail adds nothing to a score,
and the kernels write only the first ``vdim`` values of an output head.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.specs import CacheSpec, PagedKVSpec
from ..kernels import ops
from .base import ParamSpec, Piece, PositionEncoding, whole
from .mixer import AttentionMixer


class GatedAttentionMixer(AttentionMixer):
  def __init__(self, name: str, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float,
               norm_eps: Optional[float], window: Optional[int] = None, sinks: bool = True, gated: bool = True,
               value_mix: Optional[str] = None, value_mix_key: str = "value_mix_source",
               tensors: Optional[Dict[str, str]] = None, rotary: Optional[PositionEncoding] = None,
               rotary_interleaved: bool = False, norm_weights: bool = False, values_from_keys: bool = False,
               keep_first: int = 0, biases: bool = False, norm_over: str = "head", softcap: float = 0.0, weights: str = "softmax"):
    super().__init__(name, hidden_size, num_heads, num_kv_heads, dim, scale, norm_eps, rotary, window)
    if values_from_keys and (vdim != dim or value_mix is not None):
      raise ValueError(f"{name}: values that are the keys have the keys' size ({dim}, got vdim={vdim}) and are not mixed")
    if keep_first < 0 or (keep_first and window is None):
      raise ValueError(f"{name}: keep_first={keep_first} needs a window and must not be negative")
    if norm_over not in ("head", "projection"):
      raise ValueError(f"{name}: norm_over must be 'head' or 'projection', got {norm_over!r}")
    if biases and (values_from_keys or value_mix is not None):
      raise ValueError(f"{name}: biases go with projected, unmixed values")
    if weights not in ("softmax", "sigmoid") or (weights == "sigmoid" and sinks):
      raise ValueError(f"{name}: weights must be 'softmax' or 'sigmoid' (got {weights!r}), and sigmoid weights take no sink")
    if not softcap >= 0:
      raise ValueError(f"{name}: softcap must not be negative, got {softcap!r}")
    self.softcap = float(softcap)
    self.sigmoid_weights = weights == "sigmoid"
    self.biases = bool(biases)
    self.norm_whole = norm_over == "projection"
    self.rotary_interleaved = bool(rotary_interleaved)
    self.norm_weights = bool(norm_weights)
    self.values_from_keys = bool(values_from_keys)
    self.keep_first = int(keep_first)
    if value_mix not in (None, "source", "mixed"):
      raise ValueError(f"{name}: value_mix must be None, 'source' or 'mixed', got {value_mix!r}")
    if dim <= 0 or vdim <= 0:
      raise ValueError(f"{name}: dim and vdim must be positive")
    self.dim = dim
    self.vdim = vdim
    self.cache_head_dim = -(-max(dim, vdim) // 16) * 16
    self.sinks = sinks
    self.gated = gated
    self.value_mix = value_mix
    self.value_mix_key = value_mix_key
    t = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "sink": "sink", "mix": "vmix", "q_norm": "q.norm", "k_norm": "k.norm",
         "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "score_bias": "pb"}
    t.update(tensors or {})
    self.tensors = t
    H, G = num_heads, num_kv_heads
    self.q_off = 0
    self.k_off = H * dim
    self.v_off = self.k_off if values_from_keys else self.k_off + G * dim
    self.g_off = self.k_off + G * dim + (0 if values_from_keys else G * vdim)
    self.proj_width = self.g_off + (H * vdim if gated else 0)

  def cache_spec(self) -> Optional[CacheSpec]:
    return PagedKVSpec(self.num_kv_heads, self.cache_head_dim, self.window, self.keep_first)

  def param_specs(self) -> Dict[str, ParamSpec]:
    Hd, H, G, D, Dv, n, t = self.hidden_size, self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.name, self.tensors
    pieces = [Piece(f"{n}.{t['q']}", self.q_off, (H * D, Hd)), Piece(f"{n}.{t['k']}", self.k_off, (G * D, Hd))]
    if not self.values_from_keys:
      pieces.append(Piece(f"{n}.{t['v']}", self.v_off, (G * Dv, Hd)))
    if self.gated:
      pieces.append(Piece(f"{n}.{t['g']}", self.g_off, (H * Dv, Hd)))
    specs = {"qkvg": ParamSpec((self.proj_width, Hd), "matrix", [pieces]),
             "o": ParamSpec((Hd, H * Dv), "matrix", [whole(f"{n}.{t['o']}", (Hd, H * Dv))])}
    if self.norm_weights:
      nq, nk = ((H * D,), (G * D,)) if self.norm_whole else ((D,), (D,))
      specs["q_norm"] = ParamSpec(nq, "vector", [whole(f"{n}.{t['q_norm']}", nq)], init="ones_noise")
      specs["k_norm"] = ParamSpec(nk, "vector", [whole(f"{n}.{t['k_norm']}", nk)], init="ones_noise")
    if self.biases:
      # one vector over the fused projection's query, key and value columns
      specs["bias"] = ParamSpec((self.g_off,), "vector", [[
        Piece(f"{n}.{t['q_bias']}", self.q_off, (H * D,)), Piece(f"{n}.{t['k_bias']}", self.k_off, (G * D,)),
        Piece(f"{n}.{t['v_bias']}", self.v_off, (G * Dv,))]], init="half_noise")
    if self.sinks:
      specs["sink"] = ParamSpec((H,), "vector", [whole(f"{n}.{t['sink']}", (H,))])
    if self.sigmoid_weights:
      specs["score_bias"] = ParamSpec((H,), "vector", [whole(f"{n}.{t['score_bias']}", (H,))])
    if self.value_mix is not None:
      # the layer whose values are the source carries the scalar too (unused), as its file does
      specs["mix"] = ParamSpec((), "vector", [whole(f"{n}.{t['mix']}", ())], init="half_noise")
    return specs

  def validate(self, dtype: torch.dtype) -> None:
    if self.cache_head_dim > 256:
      raise ValueError(f"{self.name}: head sizes up to 256 are supported, got dim={self.dim}, vdim={self.vdim}")
    rotary = getattr(self.position, "rotary_dim", None)
    if rotary is not None and rotary > self.dim:
      raise ValueError(f"{self.name}: the rotary encoding covers {rotary} values, more than dim={self.dim}")
    if dtype == torch.bfloat16 and self.gated:      # the gate's rows are read 16 bytes at a time
      for what, k in (("width", self.hidden_size), ("heads * vdim", self.num_heads * self.vdim),
                      ("the fused projection's rows", self.proj_width)):
        if k % 8:
          raise ValueError(f"{self.name}: {what}={k} must be a multiple of 8 in bfloat16 (rows are read 16 bytes at a time)")

  def takes_residual(self, norm, ctx) -> bool:
    return False

  def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
    T = x.shape[0]
    H, G, D, Dv, hdp = self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.cache_head_dim
    if cache.kind != "paged":
      raise RuntimeError(f"{self.name}: attention needs a paged cache, got {cache.kind!r}")
    proj = ctx.ws.buffer("qkvg", (T, self.proj_width), ctx.dtype)
    ops.linear(proj, x, self.qkvg)
    q_heads = ctx.ws.buffer("q_heads", (T, H * hdp), ctx.dtype)
    v_other, v_mode, mix = None, 0, None
    if self.value_mix == "source":
      v_other = ctx.ws.buffer(f"values:{self.value_mix_key}", (T, G * Dv), ctx.dtype)
      ctx.shared[self.value_mix_key] = v_other
      v_mode = 1
    elif self.value_mix == "mixed":
      v_other = ctx.shared.get(self.value_mix_key)
      if v_other is None or v_other.shape != (T, G * Dv):
        raise RuntimeError(f"{self.name}: no layer before this one has left its values under {self.value_mix_key!r}")
      v_mode, mix = 2, self.mix
    ops.qkv_norm_mix_store(proj, self.q_off, self.k_off, self.v_off, q_heads, H, G, D, Dv,
                           self.qk_norm_eps if self.qk_norm_eps is not None else 1.0, self.qk_norm_eps is not None,
                           self.q_norm if self.norm_weights else None, self.k_norm if self.norm_weights else None, mix, v_other, v_mode,
                           ctx.slot_mapping[cache.group] if cache.writes else None, cache.tensor if cache.writes else None,
                           rope=self.position.rotary_table() if self.position is not None else None, positions=ctx.positions,
                           interleaved=self.rotary_interleaved, bias=self.bias if self.biases else None, norm_whole=self.norm_whole)
    attn = ctx.ws.buffer("attn_out", (T, H * Dv), ctx.dtype)
    ops.attention(attn, q_heads, cache.tensor, ctx.block_tables[cache.group], self._batch(ctx), H, G, hdp, self.scale,
                  self.window, sink=self.sink if self.sinks else None, gate=proj if self.gated else None,
                  gate_offset=self.g_off, out_hd=Dv, keep_first=self.keep_first, softcap=self.softcap,
                  score_bias=self.score_bias if self.sigmoid_weights else None)
    out = ctx.ws.buffer(self.out_buffer, (T, self.hidden_size), ctx.dtype)
    ops.linear(out, attn, self.o)
    return out
