"""CPU oracle: scale-factor and weight layouts handed to the kernels. TEST INFRASTRUCTURE ONLY (see quant.py)."""
import torch

from .quant import align, ceil_div, ue8m0_bytes


def pack_sf_dense(sf: torch.Tensor) -> torch.Tensor:
    """fp32 power-of-two scales [G, MN, SFK] -> contiguous int32 [G, ceil(SFK / 4), align(MN, 4)]: the memory image
    of the packed MN-major tensor (byte j of an int = K block 4i + j; K blocks and rows beyond the input pack as 0)."""
    g, mn, sfk = sf.shape
    packed_k, aligned_mn = ceil_div(sfk, 4), align(mn, 4)
    raw = torch.zeros((g, packed_k * 4, aligned_mn), dtype=torch.uint8)
    raw[:, :sfk, :mn] = ue8m0_bytes(sf).transpose(1, 2)
    ints = raw.view(g, packed_k, 4, aligned_mn).permute(0, 1, 3, 2).contiguous().view(torch.int32)
    return ints.view(g, packed_k, aligned_mn)


def pack_sf_mn_major(sf: torch.Tensor) -> torch.Tensor:
    """fp32 power-of-two scales [G?, MN, SFK] -> packed UE8M0 int32 [G?, MN, ceil(SFK / 4)] whose memory is
    MN-major with the MN stride padded to 4 ints: strides (packed_k * align(MN, 4), 1, align(MN, 4)).

    Follows ``get_mn_major_tma_aligned_packed_ue8m0_tensor`` (csrc/jit_kernels/impls/smxx_layout.hpp:180-253)
    and its kernel ``transpose_and_pack_fp32_into_ue8m0`` (deep_gemm/include/deep_gemm/impls/smxx_layout.cuh:56-144),
    whose result the reference's own test restates in torch (tests/test_layout.py:20-42)."""
    squeeze = sf.dim() == 2
    if squeeze:
        sf = sf.unsqueeze(0)
    out = pack_sf_dense(sf).transpose(1, 2)[:, : sf.shape[1], :]  # logical [g, mn, packed_k]
    return out[0] if squeeze else out


def interleave_gate_up(t: torch.Tensor, gran: int) -> torch.Tensor:
    """Rows [gate | up] (first / second half of dim -2 for 3-D, dim 0 for 2-D) -> blocks of ``gran`` gate rows
    followed by the matching ``gran`` up rows. The reference interleaves with gran 8
    (``_interleave_weights``, deep_gemm/mega/__init__.py:97-111); the granularity is a private contract between
    the weight transform and the kernel that consumes it."""
    squeeze = t.dim() == 2
    if squeeze:
        t = t.unsqueeze(0)
    g, n = t.shape[0], t.shape[1]
    rest = t.shape[2:]
    half = n // 2
    gate = t[:, :half].reshape(g, half // gran, gran, *rest)
    up = t[:, half:].reshape(g, half // gran, gran, *rest)
    out = torch.stack([gate, up], dim=2).reshape(g, n, *rest).contiguous()
    return out[0] if squeeze else out
