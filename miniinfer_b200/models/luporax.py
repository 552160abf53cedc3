"""Luporax, put together from parts.

Per layer an ``OutputNormBlock``: the sublayers read the residual stream itself - the mixer through a token shift toward the
token before - and ``residual_mult`` times the RMS norm of each sublayer's output (weights stored around zero) is added to the
stream.  The mixer is one of

  * ``attention`` - grouped-query attention over every earlier token with biased projections, one RMS norm over the whole
    of the queries (of the keys), rotate-half rotation of the first ``rot.dims`` values of a head, scores capped by a tanh,
    and weights that are sigmoids of the score plus a number per head, not normalised over the keys
    (``GatedAttentionMixer`` with those options);
  * ``rglru`` - a real-gated linear recurrent unit behind a short convolution, beside a gelu branch (``RglruMixer``);
  * ``mingru`` - a minimal gated recurrence with a silu read-out gate (``MinGruMixer``).

The feed-forward is a mixture of clamped gated experts chosen by their largest router logits, weighted by the softmax over
the chosen logits, plus a shared expert under a sigmoid gate (``RoutedExpertsFeedForward`` with those options), or absent.  A
layer that names another's weights runs that layer's block again: the run list names the block twice, and every run has a
cache and state of its own.  Around the layers: an embedding, a final norm that carries the logit scale, and the embedding
table as the head.  Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.shift``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``.
"""

from __future__ import annotations

from ..config.model_config import LuporaxConfig
from ..config.registry import register_model
from ..parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, LMHead, TokenEmbedding, make
from .spec import LayerRun, ModelSpec


@register_model("Luporax", LuporaxConfig)
def build_luporax(cfg: LuporaxConfig) -> ModelSpec:
  W, eps, mult = cfg.width, cfg.norm_eps, float(cfg.residual_mult)
  embedding = TokenEmbedding("embed", cfg.vocab, W, tensor="embed")
  blocks, encodings, block_of = [], [], {}
  for i in range(len(cfg.layers)):
    if cfg.weights_layer(i) != i:
      continue
    p = f"l{i}"
    kind, m = cfg.type_of(i), cfg.mixer_of(i)
    if kind == "attention":
      rotary = make(POSITION_ENCODINGS, "band_scaled_rotary", f"{p}.mix.rot", m.rot.dims, m.rot.base, cfg.max_position_embeddings)
      encodings.append(rotary)
      mixer = make(MIXERS, "gated_attention", f"{p}.mix", W, m.heads, m.kv_heads, m.dim, m.vdim, m.scale, eps, None, sinks=False,
                   gated=False, rotary=rotary, rotary_interleaved=False, norm_weights=True, biases=True, norm_over="projection",
                   softcap=m.softcap or 0.0, weights="sigmoid")
    elif kind == "rglru":
      mixer = make(MIXERS, "rglru", f"{p}.mix", W, m.width, m.blocks, m.conv)
    else:
      mixer = make(MIXERS, "mingru", f"{p}.mix", W, m.width)
    mlp = cfg.mlp_of(i)
    ffn = None
    if mlp is not None:
      ffn = make(FEED_FORWARDS, "routed_experts", f"{p}.mlp", W, mlp.ff, mlp.experts, mlp.top, router_weights="softmax_chosen",
                 activation="clamped", limit=mlp.limit, shared_size=mlp.shared.ff if mlp.shared else None,
                 shared_limit=mlp.shared.limit if mlp.shared else None, shared_gate=mlp.shared is not None)
    norm1 = make(NORMS, "rmsnorm", f"{p}.norm1", W, eps, offset=1.0, weight_name=f"{p}.norm1")
    norm2 = make(NORMS, "rmsnorm", f"{p}.norm2", W, eps, offset=1.0, weight_name=f"{p}.norm2") if ffn is not None else None
    block_of[i] = len(blocks)
    blocks.append(make(BLOCKS, "output_norm", p, W, norm1, mixer, norm2, ffn, mult=mult, token_shift=True, shift_name=f"{p}.shift"))
  final_norm = make(NORMS, "rmsnorm", "final.norm", W, eps, offset=1.0, weight_name="final.norm", gain=float(cfg.logit_scale))
  lm_head = LMHead("head", cfg.vocab, W, tied_to=embedding)
  unused = [f"l{i}.norm2" for i in block_of if cfg.mlp_of(i) is None]
  return ModelSpec(config=cfg, embedding=embedding, blocks=blocks, final_norm=final_norm, lm_head=lm_head,
                   position_encodings=encodings, run_list=[LayerRun(block_of[cfg.weights_layer(i)]) for i in range(len(cfg.layers))],
                   aliases={}, unused=unused, init_std=cfg.initializer_range)
