"""Public causal OAL entry point of the HD path (reference: oal_attention/hd_attention.py:1-5)."""

from .hd_block_gemm_adapters import grouped_causal_attention

__all__ = ("grouped_causal_attention",)
