"""B200-native context-parallel DeepSeek-sparse-attention decode path.

Sub-packages mirror the reference project's layout (`events`, `schedule`,
`comm`, `tiles`); every kernel is hand-written CUDA for sm_100a inside
libmdc.so, reached through the C ABI declared in include/mdc.h.
"""

__version__ = "0.1.0"
