"""Host-side mirror of the reference's GEMM wrappers on quantised weights
(g_ab / g_abt / g_abt_b / g_atb, cudalm.cu:3133-3202) and the decode GEMV."""
import torch

from ._lib import BF16, F32, KN, NK, check, lib, ptr, stream_ptr  # noqa: F401


def _dt(t):
    return BF16 if t.dtype == torch.bfloat16 else F32
