"""B200-native AlphaFold2 design-step trunk behind the operator surface of BindCraft2's `evoformer_backend=native`.

The compute lives in ``libbc2_b200.so`` (hand-written sm_100a CUDA, C ABI in ``include/bc2_b200.h``); this package is
the thin host side: library loading, weight manifests, and torch-tensor wrappers that mirror the reference's Python
shim (``bindcraft/af/native.py`` in the reference project).  There is no CPU or PyTorch fallback: importing
``bindcraft2_b200.native`` without the built library raises.
"""
__all__ = ['native', 'synthetic', 'build']
