"""Parts a model is composed of: norms, position encodings, mixers, feed-forwards, blocks."""
from .base import (Block, FeedForward, FixedState, Mixer, Norm, PagedKV, Part, PositionEncoding, StateBundle, StateNeed,
                   known, make, register_block, register_feed_forward, register_mixer, register_norm,
                   register_position)
from .norm import GroupRmsNorm, NoNorm, RmsNorm
from .rope import Rope
from .conv import ShortConv
from .attention import ConvGatedAttention, PagedAttention, RowNormAttention, TalkingAttention
from .ssm import Mamba2Mixer
from .latent import LatentAttention
from .delta import GatedDeltaMixer
from .mlstm import MatrixMemory, SideBySide
from .moe import RoutedExperts
from .side import TokenSide
from .ffn import DenseFfn, GatedFfn, PolyNormFfn
from .embedding import Embedding, LmHead
from .block import ParallelBlock, SandwichBlock, ScaledBlock
from .model import DecoderModel, LayerCall, default_schedule
