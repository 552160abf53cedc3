"""Famupel, put together from parts.

Per layer: a pre-norm layer of a mixer and a dense squared-ReLU feed-forward (``ActivatedFeedForward``; a layer may have
none), each behind a plain RMS norm.  With ``streams`` in the configuration the residual stream is that many streams, every
sublayer reads a weighted sum of them and writes back through a mixing matrix (``HyperConnectionBlock``), and the model
ends with the sum of the streams (``StreamSumNorm``); without it the layer is the usual ``PreNormBlock``.  The mixer is one of

  * ``gla`` - gated linear attention: a matrix state per head that decays by a learned factor per token and key channel
    (``LinearAttentionMixer`` with ``decay="channel"``; queries scaled by ``dim^-1/2``, a weight on the heads' norm);
  * ``parallel`` - grouped-query softmax attention over every earlier token with biased projections, one RMS norm over the
    whole of the queries (of the keys), rotary positions whose low frequencies are stretched band by band, and a sigmoid
    output gate (``GatedAttentionMixer`` with those options), beside a retention - the same linear attention with one fixed
    decay a head, rotated queries and keys, keys scaled by ``dim^-1/2`` and a norm without weight
    (``LinearAttentionMixer`` with ``decay="head"``) - the two summed with a constant each (``SideBySideMixer``, ``normed=False``).

Around the layers: an embedding, a final norm and an untied head.  Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.*``, ``l<i>.mlp.{up,down}``, ``l<i>.hc1.*``, ``l<i>.hc2.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.model_config import FamupelConfig
from ..config.registry import register_model
from ..parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, LMHead, TokenEmbedding, make
from .spec import ModelSpec


@register_model("Famupel", FamupelConfig)
def build_famupel(cfg: FamupelConfig) -> ModelSpec:
  W, eps, S = cfg.width, cfg.norm_eps, cfg.streams
  embedding = TokenEmbedding("embed", cfg.vocab, W, tensor="embed", copies=S if S is not None else 1)
  blocks, encodings, unused = [], [], []

  def rotary(name, rot):
    pe = make(POSITION_ENCODINGS, "band_scaled_rotary", name, rot.dims, rot.base, cfg.max_position_embeddings, scaling=rot.scaling)
    encodings.append(pe)
    return pe

  for i in range(len(cfg.layers)):
    p = f"l{i}"
    kind, m = cfg.type_of(i), cfg.mixer_of(i)
    if kind == "gla":
      mixer = make(MIXERS, "linear_attention", f"{p}.mix", W, m.heads, m.dim, m.vdim, eps, decay="channel", decay_rank=cfg.low_rank(i),
                   tau=m.tau, q_scale=m.dim ** -0.5, norm_weight=True, gate="silu")
    else:
      lc, rc, left_scale, right_scale = m
      left = make(MIXERS, "gated_attention", f"{p}.mix.left", W, lc.heads, lc.kv_heads, lc.dim, lc.vdim, lc.scale, eps, None,
                  sinks=False, gated=True, rotary=rotary(f"{p}.mix.left.rot", lc.rot), rotary_interleaved=False, norm_weights=True,
                  biases=True, norm_over="projection")
      right = make(MIXERS, "linear_attention", f"{p}.mix.right", W, rc.heads, rc.dim, rc.vdim, eps, decay="head", head_decay=rc.decay,
                   rotary=rotary(f"{p}.mix.right.rot", rc.rot), k_scale=rc.dim ** -0.5, norm_weight=False, gate="silu")
      mixer = make(MIXERS, "side_by_side", f"{p}.mix", W, left, right, eps, normed=False, left_scale=left_scale, right_scale=right_scale)
    ff = cfg.ff_of(i)
    ffn = make(FEED_FORWARDS, "activated", f"{p}.mlp", W, ff, activation="relu_squared", tensors=("up", "down")) if ff is not None else None
    norm1 = make(NORMS, "rmsnorm", f"{p}.norm1", W, eps, weight_name=f"{p}.norm1")
    norm2 = make(NORMS, "rmsnorm", f"{p}.norm2", W, eps, weight_name=f"{p}.norm2") if ffn is not None else None
    if ffn is None:      # a file may still hold what the absent feed-forward's sublayer would read
      unused += [f"{p}.norm2"] + [f"{p}.hc2.{t}" for t in ("in", "out", "mix")]
    if S is not None:
      blocks.append(make(BLOCKS, "hyper_connection", p, S, W, norm1, mixer, norm2, ffn))
    else:
      blocks.append(make(BLOCKS, "pre_norm", p, norm1, mixer, norm2, ffn))
  if S is not None:
    final_norm = make(NORMS, "stream_sum_rmsnorm", "final.norm", W, eps, S, weight_name="final.norm")
  else:
    final_norm = make(NORMS, "rmsnorm", "final.norm", W, eps, weight_name="final.norm")
  lm_head = LMHead("head", cfg.vocab, W, tensor="head")
  return ModelSpec(config=cfg, embedding=embedding, blocks=blocks, final_norm=final_norm, lm_head=lm_head,
                   position_encodings=encodings, aliases={}, unused=unused, init_std=cfg.initializer_range)
