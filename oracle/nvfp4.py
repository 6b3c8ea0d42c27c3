"""CPU oracle for the NVFP4 variant of the path. TEST INFRASTRUCTURE ONLY (see quant.py).

PARITY UNPINNED: the reference has no NVFP4 code at all (no UE4M3 scales, no 1x16 blocks, no kind::mxf4nvf4 anywhere
in its tree), so there are no reference outputs or vectors to pin this file to. It is an authored restatement of the
published NVFP4 format on top of the reference's own E2M1 rounding rule:
    value = e2m1(code) * float(ue4m3 block scale, one per 16 elements along K) * fp32 per-tensor scale
    per-tensor scale   s_t  = amax(tensor) / (6 * 448)
    block scale        sf_b = e4m3_round_to_nearest_even((amax(block) / 6) / s_t)          (0 <= sf_b <= 448)
    codes              e2m1_codes(x / (float(sf_b) * s_t)), all-zero where sf_b == 0
E2M1 thresholds, tie rule and nibble order are the reference's (deep_gemm/utils/math.py:84-122, via quant.e2m1_codes).
"""
from typing import Optional, Tuple

import torch

from .quant import align, e2m1_codes, e2m1_values, unpack_fp4


def tensor_scale(x: torch.Tensor) -> torch.Tensor:
    """fp32 per-tensor scale amax / (6 * 448); 1.0 for an all-zero tensor."""
    amax = x.abs().float().amax()
    return torch.where(amax > 0, amax / (6.0 * 448.0), torch.ones(()))


def quantize_nvfp4(x: torch.Tensor, scale: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """[M, K] (K % 16 == 0) -> (packed codes int8 [M, K/2], block scales float8_e4m3fn [M, K/16], fp32 tensor scale).
    ``scale`` fixes the per-tensor scale (calibrated activations); block scales then saturate at 448."""
    m, k = x.shape
    assert k % 16 == 0
    s_t = tensor_scale(x) if scale is None else scale.float().reshape(())
    blocks = x.float().view(m, k // 16, 16)
    amax = blocks.abs().amax(dim=2)
    sf = (amax / 6.0 / s_t).clamp(max=448.0).to(torch.float8_e4m3fn)
    factor = sf.float() * s_t
    scaled = torch.where(factor.unsqueeze(2) > 0, blocks / factor.unsqueeze(2), torch.zeros(()))
    codes = e2m1_codes(scaled).view(m, k)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).view(torch.int8).contiguous()
    return packed, sf, s_t


def dequantize_nvfp4(packed: torch.Tensor, sf: torch.Tensor, s_t: torch.Tensor) -> torch.Tensor:
    values = e2m1_values(unpack_fp4(packed))
    return values * sf.float().repeat_interleave(16, dim=1) * s_t.float()


def pack_sf_bytes_mn_major(sf: torch.Tensor) -> torch.Tensor:
    """UE4M3 block scales [G, MN, K/16] -> contiguous int32 [G, K/64, align(MN, 4)]: int (kq, row) holds the four
    scale bytes of K blocks 4kq .. 4kq+3 (little endian), rows contiguous - the same MN-major packing as the UE8M0 path."""
    g, mn, nb = sf.shape
    assert nb % 4 == 0
    raw = torch.zeros((g, nb, align(mn, 4)), dtype=torch.uint8)
    raw[:, :, :mn] = sf.view(torch.uint8).transpose(1, 2)
    return raw.view(g, nb // 4, 4, -1).permute(0, 1, 3, 2).contiguous().view(torch.int32).view(g, nb // 4, -1)


def grouped_gemm_contiguous(a_q, a_sf, a_scale, b_q, b_sf, b_scales, psum, alignment, out_dtype=torch.bfloat16):
    """D[m] = deq(A)[m] @ deq(B[group(m)]).T over a psum layout (see gemm.grouped_gemm_contiguous).
    The kernel multiplies the block-scaled accumulator by a_scale * b_scales[g] in FP32; the dequantised form is the
    same product in a different order, so parity is within the FP4 tolerance, not bit-exact."""
    a = dequantize_nvfp4(a_q, a_sf, a_scale)
    m, n = a.shape[0], b_q.shape[1]
    d = torch.zeros((m, n), dtype=torch.float32)
    mask = torch.zeros(m, dtype=torch.bool)
    start = 0
    for g in range(b_q.shape[0]):
        end = int(psum[g])
        if end > start:
            d[start:end] = a[start:end] @ dequantize_nvfp4(b_q[g], b_sf[g], b_scales[g]).T
            mask[start:end] = True
        start = align(end, alignment)
    return d.to(out_dtype), mask


def swiglu_requant_nvfp4(gate_up: torch.Tensor, weight: torch.Tensor, clamp: Optional[float], out_scale: torch.Tensor):
    """L1 epilogue of the NVFP4 layer: same SwiGLU as moe.swiglu_requant, then NVFP4 quantisation with the given
    (calibrated) per-tensor scale. Returns (packed int8 [rows, I/2], block scales e4m3 [rows, I/16])."""
    half = gate_up.shape[1] // 2
    gate = gate_up[:, :half].bfloat16().float()
    up = gate_up[:, half:].bfloat16().float()
    if clamp is not None:
        gate = gate.clamp(max=clamp)
        up = up.clamp(min=-clamp, max=clamp)
    act = gate / (1.0 + torch.exp(-gate)) * up * weight.float().unsqueeze(1)
    q, sf, _ = quantize_nvfp4(act, out_scale)
    return q, sf


def moe_layer_nvfp4(x_q, x_sf, x_scale, topk_idx, topk_weights, l1_q, l1_sf, l1_scales, l2_q, l2_sf, l2_scales,
                    act_scale, clamp: Optional[float] = None):
    """The layer of moe.moe_layer with NVFP4 activations and weights: x and the post-SwiGLU activations are NVFP4
    (per-tensor scales x_scale and the calibrated act_scale), weights NVFP4 with one fp32 scale per expert matrix."""
    tokens, hidden = x_q.shape[0], x_q.shape[1] * 2
    num_experts, topk = l1_q.shape[0], topk_idx.shape[1]
    x = dequantize_nvfp4(x_q, x_sf, x_scale)
    slot_rows = torch.zeros((tokens, topk, hidden), dtype=torch.bfloat16)
    for e in range(num_experts):
        tok, slot = torch.nonzero(topk_idx == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        acc1 = x[tok] @ dequantize_nvfp4(l1_q[e], l1_sf[e], l1_scales[e]).T
        a2_q, a2_sf = swiglu_requant_nvfp4(acc1, topk_weights[tok, slot], clamp, act_scale)
        acc2 = dequantize_nvfp4(a2_q, a2_sf, act_scale) @ dequantize_nvfp4(l2_q[e], l2_sf[e], l2_scales[e]).T
        slot_rows[tok, slot] = acc2.bfloat16()
    valid = (topk_idx >= 0) & (topk_idx < num_experts)
    y = torch.zeros((tokens, hidden), dtype=torch.float32)
    for k in range(topk):
        y += torch.where(valid[:, k, None], slot_rows[:, k].float(), torch.zeros(()))
    return y.bfloat16()


def calibrate_act_scale(x_q, x_sf, x_scale, topk_idx, topk_weights, l1_q, l1_sf, l1_scales, clamp: Optional[float] = None):
    """Per-tensor scale of the post-SwiGLU activations over every routed (token, slot): amax / (6 * 448). Stands in
    for the offline calibration an NVFP4 deployment does; the layer takes the result as an input."""
    x = dequantize_nvfp4(x_q, x_sf, x_scale)
    amax = torch.zeros(())
    for e in range(l1_q.shape[0]):
        tok, slot = torch.nonzero(topk_idx == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        acc1 = x[tok] @ dequantize_nvfp4(l1_q[e], l1_sf[e], l1_scales[e]).T
        half = acc1.shape[1] // 2
        gate, up = acc1[:, :half].bfloat16().float(), acc1[:, half:].bfloat16().float()
        if clamp is not None:
            gate, up = gate.clamp(max=clamp), up.clamp(min=-clamp, max=clamp)
        act = gate / (1.0 + torch.exp(-gate)) * up * topk_weights[tok, slot].float().unsqueeze(1)
        amax = torch.maximum(amax, act.abs().amax())
    return torch.where(amax > 0, amax / (6.0 * 448.0), torch.ones(()))
