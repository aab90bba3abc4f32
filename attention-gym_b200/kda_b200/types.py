"""Implementation selector shared by the public KDA operations (attn_gym/linear/types.py:12-28)."""

from enum import Enum


class Impl(str, Enum):
    """``fused`` = the sm_100a CUDA kernels, ``reference`` = eager fp32 PyTorch; never a fallback."""

    FUSED = "fused"
    REFERENCE = "reference"


def resolve_impl(impl) -> Impl:
    try:
        return Impl(impl)
    except ValueError:
        valid = ", ".join(repr(m.value) for m in Impl)
        raise ValueError(f"unknown impl {impl!r}; expected one of {valid}") from None


__all__ = ["Impl", "resolve_impl"]
