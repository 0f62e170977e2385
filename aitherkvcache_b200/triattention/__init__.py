"""TriAttention: spectral KV compression scored through the RoPE trigonometric series."""
from .config import TriAttentionConfig
from .encoder import SpectralEncoding, SpectralKVEncoder
from .attention import TriAttention, TrigSeriesScorer
from .cache import SpectralKVCache
from .spectral import rope_frequencies, pair_energies, spectral_concentration

__all__ = ["TriAttentionConfig", "SpectralEncoding", "SpectralKVEncoder", "TriAttention", "TrigSeriesScorer", "SpectralKVCache",
           "rope_frequencies", "pair_energies", "spectral_concentration"]
