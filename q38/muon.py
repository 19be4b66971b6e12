"""Import location kept from the reference layout (`from q38.muon import HybridOptimizer`)."""
from .optim.hybrid import HybridOptimizer, split_parameters
from .optim.muon import MAX_BATCH_ELEMENTS, MUON_MAX_CHUNK_ELEMENTS, NS_COEFFICIENTS, Muon, newton_schulz

NS_COEF = NS_COEFFICIENTS
__all__ = ["HybridOptimizer", "Muon", "newton_schulz", "split_parameters", "NS_COEF", "NS_COEFFICIENTS", "MAX_BATCH_ELEMENTS",
           "MUON_MAX_CHUNK_ELEMENTS"]
