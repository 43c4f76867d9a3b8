"""Flash attention operator with TileFusion's Python signature.

Same argument list and conventions as TileFusion's
``python/ops/flash_attention.py:15-129``: ``query`` is ``[Lq, D]``, ``key`` is
``[D, Lk]`` (K transposed, as that module's ``key.t()`` implies and its test
builds it, ``tests/python/test_flash_attn.py:173-175``) and ``value`` is
``[Lk, Dv]``.  Differences, all supersets:

* any number (0, 1 or 2) of leading batch / head dimensions is accepted;
* fp16 and bf16;
* no transposing copies: the reference materialises ``key.t().contiguous()``
  and ``value.t().contiguous()`` on every call, here the transposed *views* go
  to the operator and the kernel reads either storage order directly;
* the tile arguments are hints -- a value that names no compiled variant lets
  the registry choose.
"""

from __future__ import annotations

import torch

from .._torch_ops import ensure_loaded

__all__ = ["FlashAttention", "flash_attention", "flash_attention_bwd", "flash_attention_autograd"]


class FlashAttention:
    """Callable holding the tile hints, scale and mask flag."""

    def __init__(
        self,
        tile_length_q: int,
        tile_length_kv: int,
        tile_hidden_qk: int,
        tile_hidden_v: int,
        softmax_scale: float,
        causal: bool,
    ) -> None:
        self.tile_length_q = tile_length_q
        self.tile_length_kv = tile_length_kv
        self.tile_hidden_qk = tile_hidden_qk
        self.tile_hidden_v = tile_hidden_v
        self.softmax_scale = softmax_scale
        self.causal = causal

    def __call__(
        self,
        query: torch.Tensor,
        key: torch.Tensor,
        value: torch.Tensor,
        return_lse: bool = False,
    ):
        """``query [..., Lq, D]``, ``key [..., D, Lk]``, ``value [..., Lk, Dv]``.

        Returns ``O [..., Lq, Dv]`` (and ``LSE [..., Lq]`` fp32, natural log,
        when ``return_lse``).
        """
        ensure_loaded()
        length_q = query.size(-2)
        hidden_v = value.size(-1)
        lead = tuple(query.shape[:-2])
        output = torch.empty(*lead, length_q, hidden_v, dtype=query.dtype, device=query.device)

        if query.stride(-1) != 1:
            query = query.contiguous()
        k_op = key.transpose(-1, -2)  # [..., Lk, D] view
        if k_op.stride(-1) != 1 and (k_op.stride(-2) != 1 or k_op.stride(-1) % 8 != 0):
            k_op = k_op.contiguous()
        v_op = value.transpose(-1, -2)  # [..., Dv, Lk] view, the operator's V^T
        if v_op.stride(-2) != 1 and (v_op.stride(-1) != 1 or v_op.stride(-2) % 8 != 0):
            v_op = v_op.contiguous()

        if return_lse:
            lse = torch.empty(*lead, length_q, dtype=torch.float32, device=query.device)
            torch.ops.tilefusion.flash_attention_lse(
                query, k_op, v_op, output, lse,
                self.tile_length_q, self.tile_length_kv, self.softmax_scale, self.causal,
            )
            return output, lse
        torch.ops.tilefusion.flash_attention(
            query, k_op, v_op, output,
            self.tile_length_q, self.tile_length_kv, self.tile_hidden_qk, self.tile_hidden_v,
            self.softmax_scale, self.causal,
        )
        return output


def flash_attention(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    tile_length_q: int,
    tile_length_kv: int,
    tile_hidden_qk: int,
    tile_hidden_v: int,
    softmax_scale: float,
    causal: bool,
) -> torch.Tensor:
    """``softmax(query @ key * softmax_scale [+ causal mask]) @ value``.

    Args:
        query: ``[..., Lq, D]``.
        key: ``[..., D, Lk]``.
        value: ``[..., Lk, Dv]``.
        tile_length_q, tile_length_kv, tile_hidden_qk, tile_hidden_v: tile
            hints kept for signature compatibility.
        softmax_scale: multiplies ``query @ key`` before the softmax.
        causal: mask key index > query index.

    Returns:
        ``[..., Lq, Dv]`` in the dtype of ``query``.
    """
    attn = FlashAttention(
        tile_length_q, tile_length_kv, tile_hidden_qk, tile_hidden_v, softmax_scale, causal
    )
    return attn(query, key, value)


def flash_attention_bwd(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    output: torch.Tensor,
    grad_output: torch.Tensor,
    lse: torch.Tensor,
    softmax_scale: float,
    causal: bool,
):
    """Gradients of :func:`flash_attention` (TileFusion has no backward pass; this
    extends its operator with one, in the same argument convention).

    ``query [..., Lq, D]``, ``key [..., D, Lk]``, ``value [..., Lk, Dv]``, ``output`` and
    ``grad_output [..., Lq, Dv]``, ``lse [..., Lq]`` as returned by
    ``FlashAttention(...)(q, k, v, return_lse=True)``.  Returns ``(dq, dk, dv)`` shaped
    like ``query``, ``key`` and ``value``.  ``D == Dv`` in {64, 128}.
    """
    ensure_loaded()
    q = query if query.stride(-1) == 1 else query.contiguous()
    k_op = key.transpose(-1, -2)                       # [..., Lk, D]
    if k_op.stride(-1) != 1:
        k_op = k_op.contiguous()
    v_nat = value if value.stride(-1) == 1 else value.contiguous()
    o = output if output.stride(-1) == 1 else output.contiguous()
    d_o = grad_output
    if d_o.stride() != o.stride():
        d_o = torch.empty_strided(o.shape, o.stride(), dtype=o.dtype, device=o.device).copy_(grad_output)
    dq = torch.empty_strided(q.shape, q.stride(), dtype=q.dtype, device=q.device)
    dk = torch.empty_strided(k_op.shape, k_op.stride(), dtype=q.dtype, device=q.device)
    dv = torch.empty_strided(v_nat.shape, v_nat.stride(), dtype=q.dtype, device=q.device)
    torch.ops.tilefusion.flash_attention_bwd(
        q, k_op, v_nat.transpose(-1, -2), o, d_o, lse.contiguous(),
        dq, dk, dv.transpose(-1, -2), softmax_scale, causal,
    )
    return dq, dk.transpose(-1, -2), dv


class _FlashAttentionFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, query, key, value, softmax_scale, causal):
        out, lse = FlashAttention(0, 0, 0, 0, softmax_scale, causal)(query, key, value, return_lse=True)
        ctx.save_for_backward(query, key, value, out, lse)
        ctx.softmax_scale, ctx.causal = softmax_scale, causal
        return out

    @staticmethod
    def backward(ctx, grad_output):
        query, key, value, out, lse = ctx.saved_tensors
        dq, dk, dv = flash_attention_bwd(query, key, value, out, grad_output, lse, ctx.softmax_scale, ctx.causal)
        return dq, dk, dv, None, None


def flash_attention_autograd(query, key, value, softmax_scale: float, causal: bool = False) -> torch.Tensor:
    """:func:`flash_attention` as a differentiable function (``key`` as ``[..., D, Lk]``):
    the forward keeps the log-sum-exp rows and ``.backward()`` runs the CUDA backward."""
    return _FlashAttentionFunction.apply(query, key, value, softmax_scale, causal)
