"""TriAttention: spectral KV compression scored through the RoPE trigonometric series."""
from .config import TriAttentionConfig
from .encoder import SpectralEncoding, SpectralKVEncoder
from .attention import TriAttention, TrigSeriesScorer
from .spectral import rope_frequencies, pair_energies, spectral_concentration

__all__ = ["TriAttentionConfig", "SpectralEncoding", "SpectralKVEncoder", "TriAttention", "TrigSeriesScorer",
           "rope_frequencies", "pair_energies", "spectral_concentration"]
