"""hippolm_b200: a Blackwell-native (sm_100a) LLM pre-training framework.

Hybrid Kimi-Delta-Attention / full-attention decoder with block attention residuals, tensor +
sequence + data parallelism, NVFP4 FFNs, Muon + AdamW, WSD schedule, packed varlen documents.
"""
__version__ = "0.1.0"
