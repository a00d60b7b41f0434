"""B200-native (sm_100a) implementation of the reference's ``int4_native_tc`` hot path.

``ops`` mirrors the reference extension's op surface; ``moe`` adds the MoE grouped ops;
``linear`` holds the ``nn.Module`` that plays the vLLM plugin's two-phase protocol.
The CUDA library ``csrc/libint4tc_b200.so`` is loaded by the first access to an op (``ops``, ``moe``, ``linear`` or
any op name) and that access fails if the library has not been built; the pure-PyTorch pieces (``calibration``,
``synthetic``, the bookkeeping of ``moe_ep``) import without it.
"""
import importlib

__version__ = "0.2.0"

_LAZY_MODULES = ("ops", "moe", "linear", "qwen3", "moe_ep", "calibration", "synthetic", "unported", "_cabi")


def __getattr__(name):
    if name in _LAZY_MODULES:
        return importlib.import_module(f"{__name__}.{name}")
    ops = importlib.import_module(f"{__name__}.ops")
    try:
        return getattr(ops, name)
    except AttributeError:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}") from None


def __dir__():
    ops = importlib.import_module(f"{__name__}.ops")
    return sorted(set(globals()) | set(_LAZY_MODULES) | set(dir(ops)))
