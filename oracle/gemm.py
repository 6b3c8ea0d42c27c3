"""CPU oracle: m-grouped FP8 x FP4 GEMMs as dequantise-then-matmul. TEST INFRASTRUCTURE ONLY (see quant.py).

The dequantised operands are exact in BF16 (at most 3 significant mantissa bits times a power of two), so the
matmul runs in fp32 over exact values and only the final rounding to BF16 remains, as in the reference's
torch checks (tests/test_fp8_fp4.py:64-183 compare against ``a @ b.T``; tests/generators.py:329-410 build the
layouts restated here)."""
from typing import Optional

import torch

from .quant import align, dequantize_fp4, dequantize_fp8


def dequantize_b(b_q: torch.Tensor, b_sf: torch.Tensor, gran_k_b: int) -> torch.Tensor:
    """[G, N, K/2] int8 packed E2M1 (or [G, N, K] e4m3) + fp32 scales [G, N, K/gran] -> fp32 [G, N, K]."""
    out = []
    for g in range(b_q.shape[0]):
        if b_q.dtype == torch.int8:
            out.append(dequantize_fp4(b_q[g], b_sf[g], gran_k_b))
        else:
            out.append(dequantize_fp8(b_q[g], b_sf[g], gran_k_b))
    return torch.stack(out)


def grouped_gemm_contiguous(a_q, a_sf, b_q, b_sf, grouped_layout, gran_k_a=128, gran_k_b=32,
                            use_psum_layout=False, alignment=128, out_dtype=torch.bfloat16,
                            valid_only: bool = True):
    """D[m] = deq(A)[m] @ deq(B[group(m)]).T for the contiguous layouts.

    ``grouped_layout``: int32 [M] group id per row, -1 on padding (tests/generators.py:345-357), or with
    ``use_psum_layout`` int32 [G] cumulative end rows where group g starts at align(end[g-1], alignment)
    (tests/generators.py:391-395; deep_gemm/include/deep_gemm/scheduler/gemm.cuh:217-237).
    Returns (d, row_mask): rows outside ``row_mask`` are zero and must not be compared."""
    a = dequantize_fp8(a_q, a_sf, gran_k_a)
    b = dequantize_b(b_q, b_sf, gran_k_b)
    m, n = a.shape[0], b.shape[1]
    d = torch.zeros((m, n), dtype=torch.float32)
    mask = torch.zeros(m, dtype=torch.bool)
    if use_psum_layout:
        start = 0
        for g in range(b.shape[0]):
            end = int(grouped_layout[g])
            if end > start:
                d[start:end] = a[start:end] @ b[g].T
                mask[start:end] = True
            start = align(end, alignment)
    else:
        for g in range(b.shape[0]):
            rows = grouped_layout == g
            if bool(rows.any()):
                d[rows] = a[rows] @ b[g].T
                mask |= rows
    return d.to(out_dtype), mask


def grouped_gemm_masked(a_q, a_sf, b_q, b_sf, masked_m, gran_k_a=128, gran_k_b=32, out_dtype=torch.bfloat16):
    """a_q [G, max_m, K], a_sf fp32 [G, max_m, K/gran]; only rows < masked_m[g] are defined
    (tests/test_fp8_fp4.py:159-167 checks exactly those). Returns (d [G, max_m, N], row_mask [G, max_m])."""
    g_count, max_m, _ = a_q.shape
    b = dequantize_b(b_q, b_sf, gran_k_b)
    d = torch.zeros((g_count, max_m, b.shape[1]), dtype=torch.float32)
    mask = torch.zeros((g_count, max_m), dtype=torch.bool)
    for g in range(g_count):
        rows = int(masked_m[g])
        if rows > 0:
            a = dequantize_fp8(a_q[g, :rows], a_sf[g, :rows], gran_k_a)
            d[g, :rows] = a @ b[g].T
            mask[g, :rows] = True
    return d.to(out_dtype), mask


def bf16_grouped_gemm_contiguous(a, b, grouped_layout, use_psum_layout=False, alignment=128, out_dtype=torch.bfloat16):
    """D[m] = A[m] @ B[group(m)].T on bfloat16 operands with FP32 accumulation: the reference's own check for the
    BF16 family is the torch product of the same tensors (tests/generators.py:329-410 with use_bf16,
    tests/test_bf16.py:58-89). Layouts as in grouped_gemm_contiguous. Returns (d, row_mask)."""
    a32, b32 = a.float(), b.float()
    m, n = a32.shape[0], b32.shape[1]
    d = torch.zeros((m, n), dtype=torch.float32)
    mask = torch.zeros(m, dtype=torch.bool)
    if use_psum_layout:
        start = 0
        for g in range(b32.shape[0]):
            end = int(grouped_layout[g])
            if end > start:
                d[start:end] = a32[start:end] @ b32[g].T
                mask[start:end] = True
            start = align(end, alignment)
    else:
        for g in range(b32.shape[0]):
            rows = grouped_layout == g
            if bool(rows.any()):
                d[rows] = a32[rows] @ b32[g].T
                mask |= rows
    return d.to(out_dtype), mask


def bf16_grouped_gemm_masked(a, b, masked_m, out_dtype=torch.bfloat16):
    """a [G, max_m, K], b [G, N, K] bfloat16; only rows < masked_m[g] are defined (tests/test_bf16.py:118-144).
    Returns (d [G, max_m, N], row_mask [G, max_m])."""
    g_count, max_m, _ = a.shape
    d = torch.zeros((g_count, max_m, b.shape[1]), dtype=torch.float32)
    mask = torch.zeros((g_count, max_m), dtype=torch.bool)
    for g in range(g_count):
        rows = int(masked_m[g])
        if rows > 0:
            d[g, :rows] = a[g, :rows].float() @ b[g].float().T
            mask[g, :rows] = True
    return d.to(out_dtype), mask


def k_grouped_gemm(a_q, a_sf, b_q, b_sf, c, ks, gran_k=128):
    """d[g] = c[g] + deq(A_g).T @ deq(B_g) for the K-grouped layout: a_q e4m3 [sum_k, m] with a_sf fp32
    [sum_k / gran_k, m] (one scale per gran_k K rows and channel, groups concatenated), likewise b; ks = K rows per group.
    The reference checks its kernel against the unquantised product (tests/generators.py:449-453,
    tests/test_fp8_fp4.py:186-230); here the dequantised operands are multiplied, as in the other GEMM oracles."""
    a = a_q.float() * a_sf.repeat_interleave(gran_k, dim=0)
    b = b_q.float() * b_sf.repeat_interleave(gran_k, dim=0)
    d = c.clone().float()
    start = 0
    for g, k in enumerate(ks):
        if k > 0:
            d[g] += a[start:start + k].T @ b[start:start + k]
        start += k
    return d


def k_grouped_gemm_psum(a_q, a_sf, b_q, b_sf, c, ends, alignment, gran_k=128):
    """K-grouped GEMM with the psum layout (tests/generators.py:482-533): ends[g] = end K row of group g, group g starts
    at align(ends[g - 1], alignment); the scale factors hold ceil(k_g / gran_k) rows per group, groups concatenated.
    Operands may be quantised (a_sf / b_sf given) or plain (a_sf = b_sf = None)."""
    d = c.clone().float()
    prev_end, sf_row = 0, 0
    for g, end in enumerate(ends):
        start = align(prev_end, alignment)
        k = max(int(end) - start, 0)
        prev_end = int(end)
        if k == 0:
            continue
        a, b = a_q[start:start + k].float(), b_q[start:start + k].float()
        if a_sf is not None:
            blocks = (k + gran_k - 1) // gran_k
            a = a * a_sf[sf_row:sf_row + blocks].repeat_interleave(gran_k, dim=0)[:k]
            b = b * b_sf[sf_row:sf_row + blocks].repeat_interleave(gran_k, dim=0)[:k]
            sf_row += blocks
        d[g] += a.T @ b
    return d
