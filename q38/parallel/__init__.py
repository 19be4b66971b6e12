"""Multi-GPU machinery: flat parameter arena with ownership, gradient engine, peer-memory transport,
expert parallelism."""
from .arena import ParamArena, assign_owners, newton_schulz_flops
from .engine import GradEngine

__all__ = ["ParamArena", "GradEngine", "assign_owners", "newton_schulz_flops"]
