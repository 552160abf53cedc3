"""Typed model configurations, read from the architecture's own ``config.json`` keys.

The reference keeps every JSON key as an untyped attribute (miniinfer/config/model/base.py:29-31)
and gives defaults in the constructor (miniinfer/config/model/qwen3.py:16-35).  Here every key the
architecture defines is a typed field; keys that change the computation but are not implemented
raise an error that names the key instead of being ignored.
"""

from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
  """A configuration that cannot be run, with the key that is at fault."""


@dataclass
class ModelConfig:
  """What every architecture's configuration gives to the engine."""

  architectures: List[str] = field(default_factory=list)
  model_type: str = ""
  vocab_size: int = 0
  max_position_embeddings: int = 0
  bos_token_id: Optional[int] = None
  eos_token_id: Any = None          # int, list of ints or None
  torch_dtype: Optional[str] = None
  extra: Dict[str, Any] = field(default_factory=dict)

  @classmethod
  def from_dict(cls, d: Dict[str, Any]) -> "ModelConfig":
    names = {f.name for f in dataclasses.fields(cls)}
    known = {k: v for k, v in d.items() if k in names and k != "extra"}
    cfg = cls(**known)
    cfg.extra = {k: v for k, v in d.items() if k not in names}
    # "dtype" is the newer spelling of "torch_dtype" in config.json files.
    if cfg.torch_dtype is None and "dtype" in cfg.extra:
      cfg.torch_dtype = cfg.extra.pop("dtype")
    cfg.validate()
    return cfg

  @classmethod
  def from_json(cls, path: str) -> "ModelConfig":
    if os.path.isdir(path):
      path = os.path.join(path, "config.json")
    with open(path, encoding="utf-8") as f:
      return cls.from_dict(json.load(f))

  def to_dict(self) -> Dict[str, Any]:
    d = dataclasses.asdict(self)
    extra = d.pop("extra")
    d.update(extra)
    return {k: v for k, v in d.items() if v is not None}

  def eos_ids(self) -> List[int]:
    if self.eos_token_id is None:
      return []
    if isinstance(self.eos_token_id, (list, tuple)):
      return [int(x) for x in self.eos_token_id]
    return [int(self.eos_token_id)]

  def validate(self) -> None:  # pragma: no cover - overridden
    pass

  def read_tensor_shapes(self, shapes: Dict[str, tuple]) -> None:
    """For designs in which a size is given by a tensor's shape alone: called with the shapes of the weights file's tensors
    when a configuration is read from a model folder.  Default: nothing to learn."""


@dataclass
class Qwen3Config(ModelConfig):
  """Qwen3 dense decoder (defaults: miniinfer/config/model/qwen3.py:16-35)."""

  model_type: str = "qwen3"
  vocab_size: int = 151936
  hidden_size: int = 1024
  intermediate_size: int = 3072
  num_hidden_layers: int = 28
  num_attention_heads: int = 16
  num_key_value_heads: Optional[int] = 8
  head_dim: Optional[int] = 128
  hidden_act: str = "silu"
  max_position_embeddings: int = 40960
  initializer_range: float = 0.02
  rms_norm_eps: float = 1e-6
  rope_theta: float = 1000000.0
  rope_scaling: Optional[Dict[str, Any]] = None
  attention_bias: bool = False
  attention_dropout: float = 0.0
  tie_word_embeddings: bool = True
  use_cache: bool = True
  use_sliding_window: bool = False
  sliding_window: Optional[int] = None
  max_window_layers: Optional[int] = None
  layer_types: Optional[List[str]] = None

  def validate(self) -> None:
    if self.num_key_value_heads is None:            # qwen3.py:46-48
      self.num_key_value_heads = self.num_attention_heads
    if self.head_dim is None:                        # qwen3.py:75-79
      if self.hidden_size % self.num_attention_heads:
        raise ConfigError("head_dim is absent and hidden_size is not a multiple of num_attention_heads")
      self.head_dim = self.hidden_size // self.num_attention_heads
    for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
      v = getattr(self, key)
      if not isinstance(v, int) or v <= 0:
        raise ConfigError(f"{key} must be a positive integer, got {v!r}")
    if self.num_attention_heads % self.num_key_value_heads:
      raise ConfigError("num_attention_heads must be a multiple of num_key_value_heads "
                        f"({self.num_attention_heads} vs {self.num_key_value_heads})")
    if self.head_dim % 2:
      raise ConfigError(f"head_dim must be even for the rotary encoding, got {self.head_dim}")
    if self.hidden_act != "silu":                    # fused_qwen3.py:122-123
      raise ConfigError(f"hidden_act={self.hidden_act!r} is not supported (only 'silu')")
    if self.rope_scaling not in (None, {}):
      kind = self.rope_scaling.get("rope_type", self.rope_scaling.get("type"))
      if kind not in (None, "default"):
        raise ConfigError(f"rope_scaling={self.rope_scaling!r} is not supported")
    if self.attention_bias:
      raise ConfigError("attention_bias=true is not supported (the architecture has no QKV bias)")
    if not (self.rms_norm_eps > 0):
      raise ConfigError("rms_norm_eps must be positive")
    if self.use_sliding_window:
      if not self.sliding_window or self.sliding_window <= 0:
        raise ConfigError("use_sliding_window=true needs a positive sliding_window")
    if self.layer_types is not None:
      if len(self.layer_types) != self.num_hidden_layers:
        raise ConfigError("layer_types must have num_hidden_layers entries")
      for t in self.layer_types:
        if t not in ("full_attention", "sliding_attention"):
          raise ConfigError(f"layer_types entry {t!r} is not known")

  def window_of_layer(self, layer: int) -> Optional[int]:
    """The attention window of a layer, or None for all keys.  The reference carries these keys
    without reading them; their meaning here: ``layer_types`` decides if given, else the layers
    from ``max_window_layers`` on are windowed when ``use_sliding_window`` is set."""
    if not self.use_sliding_window or not self.sliding_window:
      return None
    if self.layer_types is not None:
      return int(self.sliding_window) if self.layer_types[layer] == "sliding_attention" else None
    first = self.max_window_layers if self.max_window_layers is not None else 0
    return int(self.sliding_window) if layer >= first else None


@dataclass
class RikanexMixerConfig:
  """The attention of one Rikanex layer (``layers[i].mixer``)."""

  heads: int
  kv_heads: int
  dim: int                      # query / key size of a head
  vdim: int                     # value size of a head
  scale: float                  # the scores' factor
  window: Optional[int]         # ``mask.size``: token i sees j with 0 <= i - j < window; None: every earlier token
  v_mix: bool                   # values mixed with those of the first layer that says so


@dataclass
class RikanexMlpConfig:
  """The feed-forward of one Rikanex layer (``layers[i].mlp``): ``kind`` dense (``ff``) or moe (``ff`` of an expert,
  ``experts``, ``top``)."""

  kind: str
  ff: int
  experts: int = 0
  top: int = 0


@dataclass
class RikanexConfig(ModelConfig):
  """Rikanex: a decoder of parallel layers (one layer norm, attention and feed-forward side by side), windowed
  attention with a sink and an output gate, dense or routed feed-forwards.  ``config.json`` keys: ``architecture``,
  ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``, ``layers[i].{type, mixer, mlp}``; the layers may differ in
  every size.  The design has no position limit of its own; ``max_position_embeddings`` is only the engine's bound."""

  architecture: str = "Rikanex"
  vocab: int = 0
  width: int = 0
  embedding: Dict[str, Any] = field(default_factory=dict)
  norm: Dict[str, Any] = field(default_factory=dict)
  layers: List[Dict[str, Any]] = field(default_factory=list)
  max_position_embeddings: int = 1 << 30
  initializer_range: float = 0.02

  def validate(self) -> None:
    if not self.architectures:
      self.architectures = [self.architecture]
    self.vocab_size = self.vocab
    for key in ("vocab", "width"):
      v = getattr(self, key)
      if not isinstance(v, int) or v <= 0:
        raise ConfigError(f"{key} must be a positive integer, got {v!r}")
    if not isinstance(self.embedding.get("scale"), (int, float)):
      raise ConfigError("embedding.scale must be a number")
    eps = self.norm.get("eps")
    if not isinstance(eps, (int, float)) or not eps > 0:
      raise ConfigError(f"norm.eps must be a positive number, got {eps!r}")
    if not self.layers:
      raise ConfigError("layers must list at least one layer")
    for i in range(len(self.layers)):
      self.mixer_of(i)
      self.mlp_of(i)

  @property
  def embedding_scale(self) -> float:
    return float(self.embedding["scale"])

  @property
  def norm_eps(self) -> float:
    return float(self.norm["eps"])

  def mixer_of(self, i: int) -> RikanexMixerConfig:
    layer = self.layers[i]
    if layer.get("type") != "attention":
      raise ConfigError(f"layers[{i}].type={layer.get('type')!r} is not a mixer of this design (known: 'attention')")
    m = layer.get("mixer")
    if not isinstance(m, dict):
      raise ConfigError(f"layers[{i}].mixer is missing")
    for key in ("heads", "kv_heads", "dim", "vdim"):
      v = m.get(key)
      if not isinstance(v, int) or v <= 0:
        raise ConfigError(f"layers[{i}].mixer.{key} must be a positive integer, got {v!r}")
    if m["heads"] % m["kv_heads"]:
      raise ConfigError(f"layers[{i}].mixer.heads={m['heads']} must be a multiple of kv_heads={m['kv_heads']}")
    if not isinstance(m.get("scale"), (int, float)):
      raise ConfigError(f"layers[{i}].mixer.scale must be a number")
    mask = m.get("mask")
    window = None
    if mask is not None:
      window = mask.get("size") if isinstance(mask, dict) else None
      if not isinstance(window, int) or window <= 0:
        raise ConfigError(f"layers[{i}].mixer.mask.size must be a positive integer, got {mask!r}")
    return RikanexMixerConfig(m["heads"], m["kv_heads"], m["dim"], m["vdim"], float(m["scale"]), window, bool(m.get("v_mix", False)))

  def mlp_of(self, i: int) -> Optional[RikanexMlpConfig]:
    mlp = self.layers[i].get("mlp")
    if mlp is None:
      return None
    kind = mlp.get("kind")
    if kind == "dense":
      ff = mlp.get("ff")
      if not isinstance(ff, int) or ff <= 0:
        raise ConfigError(f"layers[{i}].mlp.ff must be a positive integer, got {ff!r}")
      return RikanexMlpConfig("dense", ff)
    if kind == "moe":
      ff = (mlp.get("expert") or {}).get("ff")
      router = mlp.get("router") or {}
      experts, top = router.get("experts"), router.get("top")
      for key, v in (("expert.ff", ff), ("router.experts", experts), ("router.top", top)):
        if not isinstance(v, int) or v <= 0:
          raise ConfigError(f"layers[{i}].mlp.{key} must be a positive integer, got {v!r}")
      if top > experts:
        raise ConfigError(f"layers[{i}].mlp.router.top={top} is more than experts={experts}")
      return RikanexMlpConfig("moe", ff, experts, top)
    raise ConfigError(f"layers[{i}].mlp.kind={kind!r} is not known (dense, moe)")

  def to_dict(self) -> Dict[str, Any]:
    d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "embedding": dict(self.embedding),
         "norm": dict(self.norm), "layers": [dict(x) for x in self.layers]}
    d.update(self.extra)
    return d


def _positive_int(d: dict, key: str, where: str) -> int:
  v = d.get(key)
  if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
    raise ConfigError(f"{where}.{key} must be a positive integer, got {v!r}")
  return v


def _number(d: dict, key: str, where: str, positive: bool = True) -> float:
  v = d.get(key)
  if not isinstance(v, (int, float)) or isinstance(v, bool) or (positive and not v > 0):
    raise ConfigError(f"{where}.{key} must be a {'positive ' if positive else ''}number, got {v!r}")
  return float(v)


@dataclass
class RotationConfig:
  """``rot``: ``dims`` rotated values of a head, ``base`` of the frequencies, and optionally ``scaling``: the numbers that
  stretch the frequencies for contexts beyond ``original`` - {factor, original, fast, slow} by default, or the keys the
  design names (``scaling_keys``)."""

  dims: int
  base: float
  scaling: Optional[Dict[str, float]] = None

  @classmethod
  def read(cls, m: dict, where: str, scaling_keys=("factor", "original", "fast", "slow")) -> "RotationConfig":
    rot = m.get("rot")
    if not isinstance(rot, dict):
      raise ConfigError(f"{where}.rot is missing")
    dims = _positive_int(rot, "dims", f"{where}.rot")
    if dims % 2:
      raise ConfigError(f"{where}.rot.dims must be even, got {dims}")
    base = _number(rot, "base", f"{where}.rot")
    scaling = rot.get("scaling")
    if scaling is not None:
      if not isinstance(scaling, dict):
        raise ConfigError(f"{where}.rot.scaling must be an object")
      scaling = {k: _number(scaling, k, f"{where}.rot.scaling") for k in scaling_keys}
    return cls(dims, base, scaling)


@dataclass
class LatentAttentionConfig:
  """``layers[i].mixer`` of a ``latent_attention`` layer."""

  heads: int
  dim: int            # unrotated query/key values a head
  rot_dim: int        # rotated ones
  vdim: int
  q_rank: int
  kv_rank: int
  scale: float
  rot: RotationConfig


@dataclass
class WindowedAttentionConfig:
  """The left member of a ``parallel`` layer's mixer: grouped-query attention whose values are its keys."""

  heads: int
  kv_heads: int
  dim: int
  vdim: int
  scale: float
  window: Optional[int]      # ``mask.size``
  keep_first: int            # ``mask.keep_first``
  rot: RotationConfig


@dataclass
class GatedDeltaConfig:
  """The right member of a ``parallel`` layer's mixer.  The two low ranks are read from the tensors' shapes."""

  heads: int
  kv_heads: int
  dim: int
  vdim: int
  conv: int


@dataclass
class SelectiveScanConfig:
  """``layers[i].mixer`` of a ``mamba1`` layer."""

  inner: int
  state: int
  dt_rank: int
  conv: int


@dataclass
class VugudraConfig(ModelConfig):
  """Vugudra: a decoder whose layers are listed one by one (``layers[i].{type, mixer, mlp}``), each a block of a mixer and
  a dense feed-forward side by side with a norm of its own each; mixers of three types - ``latent_attention``, ``parallel``
  (windowed attention beside a gated delta rule) and ``mamba1`` (selective scan); ``loop`` {start, stop, times} runs the layers
  start .. stop - 1 ``times`` times in a row with the same weights.  Other keys: ``architecture``, ``vocab``, ``width``,
  ``norm.eps``.  ``low_ranks`` is not a key of the file: where a size is given by a tensor's shape only (the two low ranks of
  the delta rule's decay and gate), the loader of the configuration reads it from the weights file's header.  The design
  has no position limit of its own; ``max_position_embeddings`` is only the engine's bound."""

  architecture: str = "Vugudra"
  vocab: int = 0
  width: int = 0
  norm: Dict[str, Any] = field(default_factory=dict)
  layers: List[Dict[str, Any]] = field(default_factory=list)
  loop: Optional[Dict[str, Any]] = None
  max_position_embeddings: int = 1 << 30
  initializer_range: float = 0.02
  low_ranks: Optional[Dict[str, int]] = None      # "<layer>.decay" / "<layer>.gate" -> rank, when known

  TYPES = ("latent_attention", "parallel", "mamba1")

  def validate(self) -> None:
    if not self.architectures:
      self.architectures = [self.architecture]
    self.vocab_size = self.vocab
    for key in ("vocab", "width"):
      v = getattr(self, key)
      if not isinstance(v, int) or v <= 0:
        raise ConfigError(f"{key} must be a positive integer, got {v!r}")
    eps = self.norm.get("eps") if isinstance(self.norm, dict) else None
    if not isinstance(eps, (int, float)) or not eps > 0:
      raise ConfigError(f"norm.eps must be a positive number, got {eps!r}")
    if not self.layers:
      raise ConfigError("layers must list at least one layer")
    for i in range(len(self.layers)):
      self.mixer_of(i)
      self.ff_of(i)
    self.layer_order()

  @property
  def norm_eps(self) -> float:
    return float(self.norm["eps"])

  def layer_order(self) -> List[int]:
    """The layers in the order they run: those of the loop ``times`` times in a row, then the rest."""
    n = len(self.layers)
    if self.loop is None:
      return list(range(n))
    if not isinstance(self.loop, dict):
      raise ConfigError("loop must be an object with start, stop and times")
    start, stop, times = (self.loop.get(k) for k in ("start", "stop", "times"))
    for key, v in (("start", start), ("stop", stop), ("times", times)):
      if not isinstance(v, int) or isinstance(v, bool) or v < 0:
        raise ConfigError(f"loop.{key} must be a non-negative integer, got {v!r}")
    if not (start <= stop <= n) or times < 1:
      raise ConfigError(f"loop={self.loop!r} does not fit {n} layers (0 <= start <= stop <= layers, times >= 1)")
    return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

  def type_of(self, i: int) -> str:
    kind = self.layers[i].get("type")
    if kind not in self.TYPES:
      raise ConfigError(f"layers[{i}].type={kind!r} is not a mixer of this design (known: {', '.join(self.TYPES)})")
    return kind

  def mixer_of(self, i: int):
    """The typed mixer configuration of layer ``i``: a ``LatentAttentionConfig``, a ``SelectiveScanConfig`` or, for a
    ``parallel`` layer, the pair (``WindowedAttentionConfig``, ``GatedDeltaConfig``)."""
    kind = self.type_of(i)
    m = self.layers[i].get("mixer")
    where = f"layers[{i}].mixer"
    if not isinstance(m, dict):
      raise ConfigError(f"{where} is missing")
    if kind == "latent_attention":
      c = LatentAttentionConfig(*(_positive_int(m, k, where) for k in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank")),
                                _number(m, "scale", where), RotationConfig.read(m, where))
      if c.rot.dims != c.rot_dim:
        raise ConfigError(f"{where}.rot.dims={c.rot.dims} must equal rot_dim={c.rot_dim}: the rotated part is rotated whole")
      return c
    if kind == "mamba1":
      return SelectiveScanConfig(*(_positive_int(m, k, where) for k in ("inner", "state", "dt_rank", "conv")))
    left, right = m.get("left"), m.get("right")
    if not isinstance(left, dict) or not isinstance(right, dict):
      raise ConfigError(f"{where} of a parallel layer needs 'left' and 'right'")
    lw, rw = where + ".left", where + ".right"
    mask = left.get("mask")
    window, keep = None, 0
    if mask is not None:
      if not isinstance(mask, dict):
        raise ConfigError(f"{lw}.mask must be an object")
      window = _positive_int(mask, "size", lw + ".mask")
      keep = mask.get("keep_first", 0)
      if not isinstance(keep, int) or isinstance(keep, bool) or keep < 0:
        raise ConfigError(f"{lw}.mask.keep_first must be a non-negative integer, got {keep!r}")
    lc = WindowedAttentionConfig(*(_positive_int(left, k, lw) for k in ("heads", "kv_heads", "dim", "vdim")), _number(left, "scale", lw),
                                 window, keep, RotationConfig.read(left, lw))
    if lc.heads % lc.kv_heads:
      raise ConfigError(f"{lw}.heads={lc.heads} must be a multiple of kv_heads={lc.kv_heads}")
    if lc.vdim != lc.dim:
      raise ConfigError(f"{lw}.vdim={lc.vdim} must equal dim={lc.dim}: the values are the keys")
    if lc.rot.dims > lc.dim:
      raise ConfigError(f"{lw}.rot.dims={lc.rot.dims} is more than dim={lc.dim}")
    rc = GatedDeltaConfig(*(_positive_int(right, k, rw) for k in ("heads", "kv_heads", "dim", "vdim", "conv")))
    if rc.heads % rc.kv_heads:
      raise ConfigError(f"{rw}.heads={rc.heads} must be a multiple of kv_heads={rc.kv_heads}")
    return lc, rc

  def ff_of(self, i: int) -> Optional[int]:
    """The width of layer ``i``'s dense feed-forward, or None for a layer without one."""
    mlp = self.layers[i].get("mlp")
    if mlp is None:
      return None
    if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
      raise ConfigError(f"layers[{i}].mlp.kind={mlp.get('kind') if isinstance(mlp, dict) else mlp!r} is not known (dense)")
    return _positive_int(mlp, "ff", f"layers[{i}].mlp")

  def low_rank(self, i: int, which: str, default: int = 16) -> int:
    return int((self.low_ranks or {}).get(f"l{i}.{which}", default))

  def read_tensor_shapes(self, shapes: Dict[str, tuple]) -> None:
    ranks = dict(self.low_ranks or {})
    for i in range(len(self.layers)):
      if self.type_of(i) != "parallel":
        continue
      for which, tensor in (("decay", f"l{i}.mix.right.a1"), ("gate", f"l{i}.mix.right.g1")):
        shape = shapes.get(tensor)
        if shape is not None and len(shape) == 2:
          ranks[f"l{i}.{which}"] = int(shape[0])
    self.low_ranks = ranks or None

  def to_dict(self) -> Dict[str, Any]:
    d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": dict(self.norm),
         "layers": [dict(x) for x in self.layers]}
    if self.loop is not None:
      d["loop"] = dict(self.loop)
    if self.low_ranks:
      d["low_ranks"] = dict(self.low_ranks)
    d.update(self.extra)
    return d


@dataclass
class GatedLinearAttentionConfig:
  """``layers[i].mixer`` of a ``gla`` layer.  The low rank of the decay's projection is read from the tensors' shapes."""

  heads: int
  dim: int
  vdim: int
  tau: float


@dataclass
class BiasedAttentionConfig:
  """The left member of a Famupel ``parallel`` layer's mixer: grouped-query softmax attention over every earlier token."""

  heads: int
  kv_heads: int
  dim: int
  vdim: int
  scale: float
  rot: RotationConfig


@dataclass
class RetentionConfig:
  """The right member of a Famupel ``parallel`` layer's mixer: linear attention with one fixed decay a head."""

  heads: int
  dim: int
  vdim: int
  decay: List[float]
  rot: RotationConfig


@dataclass
class FamupelConfig(ModelConfig):
  """Famupel: a decoder whose layers are listed one by one (``layers[i].{type, mixer, mlp}``), each a pre-norm layer of a
  mixer and a dense squared-ReLU feed-forward (or none); mixers of two types - ``gla`` (gated linear attention) and
  ``parallel`` (biased softmax attention with an output gate beside a retention, summed with ``left_scale`` and
  ``right_scale``).  With ``streams`` the residual stream is that many streams that every sublayer reads as a weighted sum
  and writes through a mixing matrix (hyper-connections); without it the residual sum is the usual one.  Other keys:
  ``architecture``, ``vocab``, ``width``, ``norm.eps``.  ``low_ranks`` is not a key of the file: the rank of a gla layer's
  decay projection is given by a tensor's shape only, and the loader of the configuration reads it from the weights file's
  header.  The design has no position limit of its own; ``max_position_embeddings`` is only the engine's bound."""

  architecture: str = "Famupel"
  vocab: int = 0
  width: int = 0
  norm: Dict[str, Any] = field(default_factory=dict)
  streams: Optional[int] = None
  layers: List[Dict[str, Any]] = field(default_factory=list)
  max_position_embeddings: int = 1 << 30
  initializer_range: float = 0.02
  low_ranks: Optional[Dict[str, int]] = None      # "l<i>.decay" -> rank, when known

  TYPES = ("gla", "parallel")
  SCALING_KEYS = ("factor", "low", "high", "original")

  def validate(self) -> None:
    if not self.architectures:
      self.architectures = [self.architecture]
    self.vocab_size = self.vocab
    for key in ("vocab", "width"):
      v = getattr(self, key)
      if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"{key} must be a positive integer, got {v!r}")
    eps = self.norm.get("eps") if isinstance(self.norm, dict) else None
    if not isinstance(eps, (int, float)) or not eps > 0:
      raise ConfigError(f"norm.eps must be a positive number, got {eps!r}")
    if self.streams is not None and (not isinstance(self.streams, int) or isinstance(self.streams, bool) or self.streams <= 0):
      raise ConfigError(f"streams must be a positive integer or absent, got {self.streams!r}")
    if not self.layers:
      raise ConfigError("layers must list at least one layer")
    for i in range(len(self.layers)):
      self.mixer_of(i)
      self.ff_of(i)

  @property
  def norm_eps(self) -> float:
    return float(self.norm["eps"])

  def type_of(self, i: int) -> str:
    kind = self.layers[i].get("type")
    if kind not in self.TYPES:
      raise ConfigError(f"layers[{i}].type={kind!r} is not a mixer of this design (known: {', '.join(self.TYPES)})")
    return kind

  def mixer_of(self, i: int):
    """The typed mixer configuration of layer ``i``: a ``GatedLinearAttentionConfig`` or, for a ``parallel`` layer, the
    tuple (``BiasedAttentionConfig``, ``RetentionConfig``, left_scale, right_scale)."""
    kind = self.type_of(i)
    m = self.layers[i].get("mixer")
    where = f"layers[{i}].mixer"
    if not isinstance(m, dict):
      raise ConfigError(f"{where} is missing")
    if kind == "gla":
      return GatedLinearAttentionConfig(*(_positive_int(m, k, where) for k in ("heads", "dim", "vdim")), _number(m, "tau", where))
    left, right = m.get("left"), m.get("right")
    if not isinstance(left, dict) or not isinstance(right, dict):
      raise ConfigError(f"{where} of a parallel layer needs 'left' and 'right'")
    lw, rw = where + ".left", where + ".right"
    lc = BiasedAttentionConfig(*(_positive_int(left, k, lw) for k in ("heads", "kv_heads", "dim", "vdim")), _number(left, "scale", lw),
                               RotationConfig.read(left, lw, self.SCALING_KEYS))
    if lc.heads % lc.kv_heads:
      raise ConfigError(f"{lw}.heads={lc.heads} must be a multiple of kv_heads={lc.kv_heads}")
    if lc.rot.dims > lc.dim:
      raise ConfigError(f"{lw}.rot.dims={lc.rot.dims} is more than dim={lc.dim}")
    if lc.rot.scaling is not None and not lc.rot.scaling["high"] > lc.rot.scaling["low"]:
      raise ConfigError(f"{lw}.rot.scaling.high must be more than low, got {lc.rot.scaling!r}")
    decay = right.get("decay")
    heads = _positive_int(right, "heads", rw)
    if not isinstance(decay, list) or len(decay) != heads or not all(isinstance(d, (int, float)) and not isinstance(d, bool) and 0 <= d <= 1 for d in decay):
      raise ConfigError(f"{rw}.decay must list one factor in 0..1 for each of the {heads} heads, got {decay!r}")
    rc = RetentionConfig(heads, _positive_int(right, "dim", rw), _positive_int(right, "vdim", rw), [float(d) for d in decay],
                         RotationConfig.read(right, rw, self.SCALING_KEYS))
    if rc.rot.dims > rc.dim:
      raise ConfigError(f"{rw}.rot.dims={rc.rot.dims} is more than dim={rc.dim}")
    return lc, rc, _number(m, "left_scale", where, positive=False), _number(m, "right_scale", where, positive=False)

  def ff_of(self, i: int) -> Optional[int]:
    """The width of layer ``i``'s dense feed-forward, or None for a layer without one."""
    mlp = self.layers[i].get("mlp")
    if mlp is None:
      return None
    if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
      raise ConfigError(f"layers[{i}].mlp.kind={mlp.get('kind') if isinstance(mlp, dict) else mlp!r} is not known (dense)")
    return _positive_int(mlp, "ff", f"layers[{i}].mlp")

  def low_rank(self, i: int, default: int = 16) -> int:
    return int((self.low_ranks or {}).get(f"l{i}.decay", default))

  def read_tensor_shapes(self, shapes: Dict[str, tuple]) -> None:
    ranks = dict(self.low_ranks or {})
    for i in range(len(self.layers)):
      shape = shapes.get(f"l{i}.mix.a1")
      if self.type_of(i) == "gla" and shape is not None and len(shape) == 2:
        ranks[f"l{i}.decay"] = int(shape[0])
    self.low_ranks = ranks or None

  def to_dict(self) -> Dict[str, Any]:
    d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": dict(self.norm),
         "layers": [dict(x) for x in self.layers]}
    if self.streams is not None:
      d["streams"] = self.streams
    if self.low_ranks:
      d["low_ranks"] = dict(self.low_ranks)
    d.update(self.extra)
    return d


@dataclass
class SigmoidAttentionConfig:
  """``layers[i].mixer`` of a Luporax ``attention`` layer: grouped-query attention over every earlier token whose weights are
  sigmoids of the capped scores (``softcap`` None: no cap)."""

  heads: int
  kv_heads: int
  dim: int
  vdim: int
  scale: float
  softcap: Optional[float]
  rot: RotationConfig


@dataclass
class RglruConfig:
  """``layers[i].mixer`` of a Luporax ``rglru`` layer: ``width`` channels in ``blocks`` equal parts, a convolution of ``conv`` taps."""

  width: int
  blocks: int
  conv: int


@dataclass
class MinGruConfig:
  """``layers[i].mixer`` of a Luporax ``mingru`` layer."""

  width: int


@dataclass
class SharedExpertConfig:
  ff: int
  limit: float


@dataclass
class ClampedMoeConfig:
  """``layers[i].mlp`` of a Luporax layer: ``experts`` experts of width ``ff`` with the clamp ``limit``, ``top`` of them a token,
  and optionally a shared expert."""

  ff: int
  limit: float
  experts: int
  top: int
  shared: Optional[SharedExpertConfig]


@dataclass
class LuporaxConfig(ModelConfig):
  """Luporax: a decoder whose layers are listed one by one (``layers[i].{type, mixer, mlp}``).  A layer reads the residual
  stream itself - its mixer through a token shift - and adds ``residual_mult`` times the RMS norm of each sublayer's output;
  mixers of three types - ``attention`` (sigmoid weights on capped scores), ``rglru`` (a real-gated linear recurrent unit
  behind a short convolution) and ``mingru`` (a minimal gated recurrence); the feed-forward is a mixture of clamped gated
  experts with a gated shared expert, or absent.  A layer with ``weights_of: j`` has no tensors of its own and runs layer
  ``j``'s, with a cache and state of its own.  The head is the embedding table, its logits times ``logit_scale``.  Other keys:
  ``architecture``, ``vocab``, ``width``, ``norm.eps``.  The design has no position limit of its own;
  ``max_position_embeddings`` is only the engine's bound."""

  architecture: str = "Luporax"
  vocab: int = 0
  width: int = 0
  norm: Dict[str, Any] = field(default_factory=dict)
  residual_mult: Any = None
  logit_scale: Any = None
  layers: List[Dict[str, Any]] = field(default_factory=list)
  max_position_embeddings: int = 1 << 30
  initializer_range: float = 0.02

  TYPES = ("attention", "rglru", "mingru")

  def validate(self) -> None:
    if not self.architectures:
      self.architectures = [self.architecture]
    self.vocab_size = self.vocab
    for key in ("vocab", "width"):
      v = getattr(self, key)
      if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"{key} must be a positive integer, got {v!r}")
    eps = self.norm.get("eps") if isinstance(self.norm, dict) else None
    if not isinstance(eps, (int, float)) or isinstance(eps, bool) or not eps > 0:
      raise ConfigError(f"norm.eps must be a positive number, got {eps!r}")
    for key in ("residual_mult", "logit_scale"):
      v = getattr(self, key)
      if not isinstance(v, (int, float)) or isinstance(v, bool):
        raise ConfigError(f"{key} must be a number, got {v!r}")
    if not self.layers:
      raise ConfigError("layers must list at least one layer")
    for i in range(len(self.layers)):
      self.weights_layer(i)
      self.mixer_of(i)
      self.mlp_of(i)

  @property
  def norm_eps(self) -> float:
    return float(self.norm["eps"])

  def weights_layer(self, i: int) -> int:
    """The layer whose tensors layer ``i`` runs: itself, or the one its ``weights_of`` names (which has tensors of its own or
    names a third in turn).  The rest of a sharing layer's entry must equal the other's."""
    seen = [i]
    while self.layers[seen[-1]].get("weights_of") is not None:
      j = self.layers[seen[-1]]["weights_of"]
      if not isinstance(j, int) or isinstance(j, bool) or not (0 <= j < len(self.layers)) or j in seen:
        raise ConfigError(f"layers[{seen[-1]}].weights_of={j!r} must name another layer (0..{len(self.layers) - 1}) and not come back to itself")
      seen.append(j)
    src = seen[-1]
    if src != i:
      mine = {k: v for k, v in self.layers[i].items() if k != "weights_of"}
      theirs = {k: v for k, v in self.layers[src].items() if k != "weights_of"}
      if mine != theirs:
        raise ConfigError(f"layers[{i}] runs the weights of layers[{src}] but its entry differs from that layer's")
    return src

  def type_of(self, i: int) -> str:
    kind = self.layers[i].get("type")
    if kind not in self.TYPES:
      raise ConfigError(f"layers[{i}].type={kind!r} is not a mixer of this design (known: {', '.join(self.TYPES)})")
    return kind

  def mixer_of(self, i: int):
    """The typed mixer configuration of layer ``i``: a ``SigmoidAttentionConfig``, an ``RglruConfig`` or a ``MinGruConfig``."""
    kind = self.type_of(i)
    m = self.layers[i].get("mixer")
    where = f"layers[{i}].mixer"
    if not isinstance(m, dict):
      raise ConfigError(f"{where} is missing")
    if kind == "rglru":
      c = RglruConfig(*(_positive_int(m, k, where) for k in ("width", "blocks", "conv")))
      if c.width % c.blocks:
        raise ConfigError(f"{where}.width={c.width} must be a multiple of blocks={c.blocks}")
      return c
    if kind == "mingru":
      return MinGruConfig(_positive_int(m, "width", where))
    cap = m.get("softcap")
    if cap is not None and (not isinstance(cap, (int, float)) or isinstance(cap, bool) or not cap > 0):
      raise ConfigError(f"{where}.softcap must be a positive number or absent, got {cap!r}")
    c = SigmoidAttentionConfig(*(_positive_int(m, k, where) for k in ("heads", "kv_heads", "dim", "vdim")), _number(m, "scale", where),
                               float(cap) if cap is not None else None, RotationConfig.read(m, where, ()))
    if c.heads % c.kv_heads:
      raise ConfigError(f"{where}.heads={c.heads} must be a multiple of kv_heads={c.kv_heads}")
    if c.rot.dims > c.dim:
      raise ConfigError(f"{where}.rot.dims={c.rot.dims} is more than dim={c.dim}")
    return c

  def mlp_of(self, i: int) -> Optional[ClampedMoeConfig]:
    mlp = self.layers[i].get("mlp")
    if mlp is None:
      return None
    where = f"layers[{i}].mlp"
    if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
      raise ConfigError(f"{where}.kind={mlp.get('kind') if isinstance(mlp, dict) else mlp!r} is not known (moe)")
    expert, router, shared = mlp.get("expert"), mlp.get("router"), mlp.get("shared")
    if not isinstance(expert, dict) or not isinstance(router, dict):
      raise ConfigError(f"{where} needs 'expert' and 'router'")
    sc = None
    if shared is not None:
      if not isinstance(shared, dict):
        raise ConfigError(f"{where}.shared must be an object or absent")
      sc = SharedExpertConfig(_positive_int(shared, "ff", where + ".shared"), _number(shared, "limit", where + ".shared"))
    c = ClampedMoeConfig(_positive_int(expert, "ff", where + ".expert"), _number(expert, "limit", where + ".expert"),
                         _positive_int(router, "experts", where + ".router"), _positive_int(router, "top", where + ".router"), sc)
    if c.top > c.experts:
      raise ConfigError(f"{where}.router.top={c.top} is more than experts={c.experts}")
    return c

  def to_dict(self) -> Dict[str, Any]:
    d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": dict(self.norm),
         "residual_mult": self.residual_mult, "logit_scale": self.logit_scale, "layers": [dict(x) for x in self.layers]}
    d.update(self.extra)
    return d
