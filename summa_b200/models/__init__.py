from .transformer import Transformer, InferenceState, validate_config
from .layers import (Linear, Norm, MultiHeadAttention, MambaMixer, FeedForward, SparseMoe,
                     ExpertBank, AttentionState, MambaState)
from .memory import MemoryChain, LowRankExpertReserve
