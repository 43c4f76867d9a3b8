"""CPU restatement of TileFusion's attention algorithm.  TEST INFRASTRUCTURE ONLY.

The product never imports this file: it is the checker used by ``tests/``,
``__graft_entry__.smoke()`` and the CPU arms of ``bench.py``.

What is restated, and where it comes from in TileFusion's tree:

* ``attention_fp32`` -- the closed form ``softmax(Q K^T * s [+ mask]) V`` that
  TileFusion's own test oracle ``FlashAttentionRef`` computes blockwise
  (``tests/python/test_flash_attn.py:21-134``); evaluated in fp32 on the
  16-bit-rounded inputs.  This is the authoritative oracle and the timed CPU
  baseline.
* ``attention_blocked`` -- the same KV-tiled online-softmax recurrence as
  ``FlashAttentionRef.__call__`` (``tests/python/test_flash_attn.py:86-132``:
  per-tile max, exp, row sums, renormalisation by ``exp(prev_max - new_max)``)
  and as the kernel loop (``include/kernels/flash_attention_device.cuh:231-305``),
  with the three defects of the reference left out: state is fp32 (the kernel
  keeps it in fp16, ``flash_attention_device.cuh:253-297``), the running
  maximum starts at -inf instead of 0, and fully masked tiles are skipped
  instead of producing ``-inf - -inf``.
* ``causal_mask`` -- ``col > row`` is masked, with global row/column indices
  (``include/cell/mask.hpp:19-113``; ``torch.tril`` in the test class,
  ``tests/python/test_flash_attn.py:101-108``).
* ``decode_split`` / ``decode_combine`` -- split-KV partials ``(m, l, O)`` and
  their log-sum-exp merge.  TileFusion has no decode path; these restate the
  same recurrence across splits so that the CUDA split/combine kernels have a
  CPU counterpart with identical intermediate quantities.

Pinning: ``tests/test_oracle.py`` checks these functions against fixtures
under ``tests/golden/`` that were produced by running TileFusion's own
``FlashAttentionRef`` class (see ``tests/golden/make_golden.py``), including
the two parameter sets of its test-suite
(``tests/python/test_flash_attn.py:205-230``).
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

LOG2E = 1.4426950408889634


def causal_mask(len_q: int, len_kv: int, device=None) -> torch.Tensor:
    """Boolean [Lq, Lk], True where the score is kept (key index <= query index)."""
    rows = torch.arange(len_q, device=device).unsqueeze(1)
    cols = torch.arange(len_kv, device=device).unsqueeze(0)
    return cols <= rows


def attention_fp32(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                   causal: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """``softmax((Q K^T) * scale) V`` and its log-sum-exp, in fp32.

    q ``[..., Lq, D]``, k ``[..., Lk, D]``, v ``[..., Lk, Dv]`` (any dtype; they
    are upcast).  Returns O ``[..., Lq, Dv]`` fp32 and LSE ``[..., Lq]`` fp32
    (natural log of the sum of ``exp(scale * q.k)``).
    """
    qf, kf, vf = q.float(), k.float(), v.float()
    s = (qf @ kf.transpose(-1, -2)) * scale
    if causal:
        keep = causal_mask(s.size(-2), s.size(-1), device=s.device)
        s = s.masked_fill(~keep, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.softmax(s, dim=-1)
    return p @ vf, lse


def attention_blocked(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                      causal: bool = False, tile_kv: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """KV-tiled online softmax in fp32 (one ``[Lq, D]`` problem, 2-D inputs)."""
    qf, kf, vf = q.float(), k.float(), v.float()
    len_q, len_kv = qf.size(0), kf.size(0)
    m = torch.full((len_q, 1), float("-inf"))
    l = torch.zeros(len_q, 1)
    acc = torch.zeros(len_q, vf.size(1))
    rows = torch.arange(len_q).unsqueeze(1)
    for k0 in range(0, len_kv, tile_kv):
        k1 = min(len_kv, k0 + tile_kv)
        if causal and k0 > len_q - 1:
            break  # every score of this tile is masked
        s = (qf @ kf[k0:k1].t()) * scale
        if causal:
            cols = torch.arange(k0, k1).unsqueeze(0)
            s = s.masked_fill(cols > rows, float("-inf"))
        m_tile = s.max(dim=-1, keepdim=True).values
        m_new = torch.maximum(m, m_tile)
        # rows with nothing visible yet keep (m, l, acc) = (-inf, 0, 0)
        safe = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)
        p = torch.exp(s - safe)
        alpha = torch.exp(torch.where(torch.isinf(m), torch.full_like(m, float("-inf")), m - safe))
        l = l * alpha + p.sum(dim=-1, keepdim=True)
        acc = acc * alpha + p @ vf[k0:k1]
        m = m_new
    return acc / l, (m + torch.log(l)).squeeze(-1)


def decode_split(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                 keys_per_split: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Split-KV partials for one query row per (batch, head).

    q ``[B, H, D]``, k/v ``[B, H, Lk, D]``.  Returns ``part_o [B, H, S, D]``
    (un-normalised, fp32) and ``part_ml [B, H, S, 2]`` with ``m`` the maximum of
    ``scale * log2(e) * q.k`` over the split and ``l = sum 2^(s - m)`` -- the
    quantities the CUDA split kernel writes.
    """
    qf, kf, vf = q.float(), k.float(), v.float()
    b, h, len_kv, d = kf.shape
    n_splits = max(1, (len_kv + keys_per_split - 1) // keys_per_split)
    part_o = torch.zeros(b, h, n_splits, d)
    part_ml = torch.zeros(b, h, n_splits, 2)
    part_ml[..., 0] = float("-inf")
    for s in range(n_splits):
        k0, k1 = s * keys_per_split, min(len_kv, (s + 1) * keys_per_split)
        if k1 <= k0:
            continue
        sc = torch.einsum("bhd,bhkd->bhk", qf, kf[:, :, k0:k1]) * (scale * LOG2E)
        m = sc.max(dim=-1).values
        p = torch.exp2(sc - m.unsqueeze(-1))
        part_ml[:, :, s, 0] = m
        part_ml[:, :, s, 1] = p.sum(dim=-1)
        part_o[:, :, s] = torch.einsum("bhk,bhkd->bhd", p, vf[:, :, k0:k1])
    return part_o, part_ml


def decode_combine(part_o: torch.Tensor, part_ml: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Log-sum-exp merge over the split axis.

    part_o ``[..., S, D]``, part_ml ``[..., S, 2]`` (``m`` in log2 units, ``l``).
    Returns normalised O ``[..., D]``, LSE ``[...]`` (natural log) and the merged
    partial ``(acc [..., D], m [...], l [...])`` packed as ``[..., D + 2]``.
    """
    m = part_ml[..., 0]
    l = part_ml[..., 1]
    m_star = m.max(dim=-1).values
    w = torch.where(torch.isinf(m), torch.zeros_like(m), torch.exp2(m - m_star.unsqueeze(-1)))
    l_star = (l * w).sum(dim=-1)
    acc = (part_o * w.unsqueeze(-1)).sum(dim=-2)
    out = acc / l_star.unsqueeze(-1)
    lse = (m_star + torch.log2(l_star)) * math.log(2.0)
    merged = torch.cat([acc, m_star.unsqueeze(-1), l_star.unsqueeze(-1)], dim=-1)
    return out, lse, merged


def decode_fp32(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Closed-form decode: q ``[B, H, 1, D]``, k/v ``[B, H, Lk, D]``."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.size(-1))
    return attention_fp32(q, k, v, scale, causal=False)


def attention_bwd_fp32(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, d_o: torch.Tensor, scale: float,
                       causal: bool = False) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Gradients of ``attention_fp32`` with respect to q, k and v for the upstream
    gradient ``d_o``, by reverse-mode differentiation of that same closed form in
    fp32 on the host.  TileFusion has no backward pass and therefore pins nothing
    here; the reference point is the gradient of the expression that its
    ``FlashAttentionRef`` class pins for the forward.  q ``[..., Lq, D]``,
    k/v ``[..., Lk, D]``, d_o ``[..., Lq, Dv]``; returns fp32 (dq, dk, dv)."""
    qf = q.detach().float().requires_grad_(True)
    kf = k.detach().float().requires_grad_(True)
    vf = v.detach().float().requires_grad_(True)
    out, _ = attention_fp32(qf, kf, vf, scale, causal)
    out.backward(d_o.float())
    return qf.grad, kf.grad, vf.grad


def fused_two_gemms_fp32(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
    """``(A @ B^T) @ C^T`` as TileFusion's test states it
    (``tests/python/test_fused_two_gemms.py:100``: ``input_a @ input_b.t() @ input_c.t()``
    on 16-bit tensors): fp32 accumulation, the intermediate product rounded to
    the input dtype as a 16-bit matmul returns it.  a ``[M, K]``, b ``[N, K]``,
    c ``[P, N]``; returns fp32 ``[M, P]`` (not rounded)."""
    inter = (a.float() @ b.float().t()).to(a.dtype)
    return inter.float() @ c.float().t()


# ---------------------------------------------------------------- tolerances --
def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    return (a.float() - b.float()).abs().max().item()


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    """||a - b||_2 / ||b||_2 with b the reference."""
    af, bf = a.double(), b.double()
    return ((af - bf).norm() / bf.norm().clamp_min(1e-30)).item()


# Root-mean-square relative error of rounding to bf16 (8 significant bits),
# for values spread log-uniformly over a binade: 2^-8 / sqrt(3) * sqrt(E[1/x^2]).
BF16_ROUNDING_RMS = 1.7e-3


def rounding_floor(ref: torch.Tensor, dtype: torch.dtype) -> float:
    """Relative-L2 error of the *exact* result once rounded to ``dtype``: no
    kernel that returns ``dtype`` can do better than this on ``ref``."""
    return rel_l2(ref.float().to(dtype), ref)


def rel_l2_bound(ref: torch.Tensor, dtype: torch.dtype, p_rounded: bool = True) -> float:
    """Bound on relative-L2(O) for an output of ``dtype``.

    fp16: the north-star figure, 1e-3.  bf16: that figure cannot be met -- the
    rounding of the exact result already costs about 1.7e-3 -- so the bound is
    computed from the reference itself: the rounding floor of ``ref``, combined
    in quadrature with a second term of the same size when the kernel feeds the
    probabilities P to the tensor cores as bf16 (``p_rounded``; each p carries an
    independent relative error of BF16_ROUNDING_RMS, which reaches O undamped:
    err(O) = sum p_k d_k (v_k - O) / l has the spread of O itself for zero-mean
    V), times a 15 % margin, plus 1e-4 for the fp32 arithmetic.  For i.i.d.
    inputs this comes to about 2.9e-3 with and 2.1e-3 without P rounding; the
    kernels sit at 2.4e-3 and 1.7e-3."""
    if dtype != torch.bfloat16:
        return 1e-3
    floor = rounding_floor(ref, dtype)
    extra = BF16_ROUNDING_RMS if p_rounded else 0.0
    return 1.15 * math.sqrt(floor * floor + extra * extra) + 1e-4


def seeded_inputs(seed: int, shape_q, shape_k, shape_v, sigma: float, dtype=torch.float16):
    """i.i.d. N(0, sigma^2) Q, K, V from a CPU generator, drawn in that order in
    fp32 and rounded to ``dtype`` -- the seeded inputs of the benchmark configs."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = (torch.randn(shape_q, generator=g) * sigma).to(dtype)
    k = (torch.randn(shape_k, generator=g) * sigma).to(dtype)
    v = (torch.randn(shape_v, generator=g) * sigma).to(dtype)
    return q, k, v
