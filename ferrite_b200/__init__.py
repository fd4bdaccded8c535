"""ferrite_b200: a Blackwell-datacenter (sm_100a) LLM inference engine with the capabilities of ferrite.

PyTorch holds tensors, streams, graphs and process groups; every hot operator is a hand-written CUDA kernel
in `csrc/` (tcgen05/TMEM GEMMs fed by TMA, fused compute + NVLink collectives), reached through `ops`.
"""
from .config import EngineConfig, ModelConfig, PRESETS, SiteConfig  # noqa: F401

__version__ = "0.1.0"
