from .base import (CacheSpec, CacheTensor, FeedForward, Mixer, Norm, ParamSpec, Part, PositionEncoding, Source,
                   StateSpec, StreamOp, build_feed_forward, build_mixer, build_norm,
                   build_position_encoding, register_feed_forward, register_mixer, register_norm,
                   register_position_encoding, register_stream_op)
from .norm import GroupRMSNorm, LayerNorm, RMSNorm
from .positions import LearnedPositions
from .rotary import Rotary
from .attention import Attention
from .mlp import GatedMLP
from .linear_attention import HGRN2, MLSTM, GatedLinearAttention, Lightning, Mamba2, Retention
from .latent_attention import LatentAttention
from .moe import MixtureOfExperts
from .side_by_side import SideBySide
from .stream import InputAdd, InputInjection
from .block import ARRANGEMENTS, ParallelBlock, PostNormBlock, PreNormBlock, SandwichBlock, build_block
from .model import BoundCall, DecoderModel, Embedding, LMHead, build_model
