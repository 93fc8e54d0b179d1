from .base import (Part, TensorSpec, KvCacheNeed, StateNeed, CompositeNeed, Registry, MIXERS, FEED_FORWARDS, NORMS,
                   POSITION_ENCODINGS, BLOCKS, HOOKS, FAMILIES)
from .linear import Linear
from .norm import RMSNorm, DynamicTanh
from .rope import RotaryEncoding, inverse_frequencies
from .attention import PagedAttention
from .mlp import GatedMLP, ClampedGluMLP
from .block import (PreNormResidualBlock, OutputNormResidualBlock, SandwichNormResidualBlock,
                    PreNormStreamResidualBlock)
from .sink_attention import GatedSinkAttention
from .mamba2 import Mamba2Mixer
from .latent_attention import LatentAttention
from .moe import PolyNormMLP, TableMoE, RoutedMoE
from .hooks import LogitSoftcap, StreamOffset, EmbeddingScale
from .sinusoid import SinusoidalEncoding
from .token_input import TokenTableRows, TokenSideInput
from .mamba1 import Mamba1Mixer
from .talking_attention import TalkingHeadsAttention
from .delta_rule import GatedDeltaRule
from .parallel import ParallelMixers
from .unit_attention import UnitQkAttention
from .mlstm import MLstmMixer
