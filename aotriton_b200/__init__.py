"""aotriton_b200: a B200-native FlashAttention forward/backward library behind the operator
API of ROCm/aotriton.

  aotriton_b200.cabi      ctypes view of the C-ABI (include/aotriton_b200.h)
  aotriton_b200.flash     attn_fwd / attn_bwd / varlen / debug helpers over the pyaotriton
                          bindings, argument-for-argument like the reference's
                          modules/flash/tests/aotriton_flash.py
  aotriton_b200.autograd  torch.autograd.Function wrappers (attention, varlen_attention)
  aotriton_b200.sharding  batch x head partitioning for multi-GPU runs
  aotriton_b200.build     in-tree nvcc build

There is no CPU implementation: every entry point needs the compiled library and a B200.
"""
from pathlib import Path
import sys

PKG_DIR = Path(__file__).resolve().parent


def load_pyaotriton():
    """Import the in-tree `pyaotriton` extension module (raises if it has not been built)."""
    if str(PKG_DIR) not in sys.path:
        sys.path.insert(0, str(PKG_DIR))
    try:
        import pyaotriton  # noqa: F401
    except ImportError as e:  # fail loudly: there is nothing to fall back to
        raise ImportError(
            "pyaotriton extension not built; run `python -m aotriton_b200.build` (needs nvcc)") from e
    return pyaotriton


__all__ = ["PKG_DIR", "load_pyaotriton"]
