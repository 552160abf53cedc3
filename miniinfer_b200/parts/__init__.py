from .base import (Block, Embedding, FeedForward, Head, HostStep, Mixer, Norm, ParamSpec, Part, Piece, PositionEncoding,
                   StepWork, whole)
from .block import OutputNormBlock, ParallelBlock, PreNormBlock
from .embedding import LMHead, TokenEmbedding
from .feedforward import ActivatedFeedForward, RoutedExpertsFeedForward, SwiGLUFeedForward
from .gated_attention import GatedAttentionMixer
from .hyper import HyperConnectionBlock, StreamSumNorm
from .latent_attention import LatentAttentionMixer
from .linear_attention import LinearAttentionMixer
from .mixer import AttentionMixer
from .norm import LayerNorm, RMSNorm
from .position import BandScaledRotaryEncoding, RotaryEncoding, ScaledRotaryEncoding
from .recurrent import GatedDeltaMixer, MinGruMixer, RglruMixer, SelectiveScanMixer
from .side_by_side import SideBySideMixer
from .registry import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, make, register_block,
                       register_feed_forward, register_mixer, register_norm, register_position_encoding)

register_mixer("attention")(AttentionMixer)
register_mixer("gated_attention")(GatedAttentionMixer)
register_mixer("latent_attention")(LatentAttentionMixer)
register_mixer("selective_scan")(SelectiveScanMixer)
register_mixer("gated_delta")(GatedDeltaMixer)
register_mixer("side_by_side")(SideBySideMixer)
register_mixer("linear_attention")(LinearAttentionMixer)
register_mixer("rglru")(RglruMixer)
register_mixer("mingru")(MinGruMixer)
register_feed_forward("swiglu")(SwiGLUFeedForward)
register_feed_forward("routed_experts")(RoutedExpertsFeedForward)
register_feed_forward("activated")(ActivatedFeedForward)
register_norm("rmsnorm")(RMSNorm)
register_norm("layernorm")(LayerNorm)
register_norm("stream_sum_rmsnorm")(StreamSumNorm)
register_position_encoding("rotary")(RotaryEncoding)
register_position_encoding("scaled_rotary")(ScaledRotaryEncoding)
register_position_encoding("band_scaled_rotary")(BandScaledRotaryEncoding)
register_block("pre_norm")(PreNormBlock)
register_block("parallel")(ParallelBlock)
register_block("hyper_connection")(HyperConnectionBlock)
register_block("output_norm")(OutputNormBlock)
