"""B200-native (sm_100a) implementation of the reference's ``int4_native_tc`` hot path.

``ops`` mirrors the reference extension's op surface; ``moe`` adds the MoE grouped ops;
``linear`` holds the ``nn.Module`` that plays the vLLM plugin's two-phase protocol.
Importing this package loads ``csrc/libint4tc_b200.so`` and fails if it has not been built.
"""
from . import ops, moe  # noqa: F401
from .ops import *  # noqa: F401,F403

__version__ = "0.1.0"
