"""Optimizers: Muon for hidden matrices, AdamW for embeddings / routers / scalars."""
from .muon import Muon, newton_schulz, NS_COEFFICIENTS
from .hybrid import HybridOptimizer, split_parameters

__all__ = ["Muon", "newton_schulz", "NS_COEFFICIENTS", "HybridOptimizer", "split_parameters"]
