"""Back-to-back GEMM operator with TileFusion's Python signature.

``fused_two_gemms(input_a, input_b, input_c, output, tm, tn, tk, tp)`` computes
``output = input_a @ input_b.T @ input_c.T`` in place, with the operand
conventions of TileFusion's ``python/ops/fused_two_gemms.py:45-79``: ``input_a``
is ``[M, K]``, ``input_b`` is ``[N, K]``, ``input_c`` is ``[P, N]`` and ``output``
is ``[M, P]``, all with contiguous rows.  The intermediate ``A @ B.T`` is rounded
to the 16-bit dtype; both products accumulate in fp32.  It runs on the attention
kernel with the softmax stage replaced by a conversion, so ``K == P`` must be 64
or 128.  fp16 and bf16.
"""

from __future__ import annotations

import torch

from .._torch_ops import ensure_loaded

__all__ = ["fused_two_gemms"]


def fused_two_gemms(
    input_a: torch.Tensor,
    input_b: torch.Tensor,
    input_c: torch.Tensor,
    output: torch.Tensor,
    tm: int = 64,
    tn: int = 64,
    tk: int = 64,
    tp: int = 64,
) -> None:
    """``output[M, P] = input_a[M, K] @ input_b[N, K].T @ input_c[P, N].T`` (in place)."""
    operands = {"input_a": input_a, "input_b": input_b, "input_c": input_c, "output": output}
    off_device = [n for n, t in operands.items() if t.device.type != "cuda"]
    if off_device:
        raise ValueError(f"{', '.join(off_device)} must be cuda tensor(s)")
    wrong_type = [n for n, t in operands.items() if t.dtype not in (torch.float16, torch.bfloat16)]
    if wrong_type:
        raise TypeError(f"{', '.join(wrong_type)} must be torch.float16 or torch.bfloat16")
    ensure_loaded()
    torch.ops.tilefusion.fused_two_gemms(input_a, input_b, input_c, output, tm, tn, tk, tp)
