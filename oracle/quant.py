"""CPU oracle: quantisers, dequantisers and the parity metric of the Mega-MoE hot path.

TEST INFRASTRUCTURE ONLY. Nothing under ``deepgemm_b200/`` imports this package; it is the checker that
``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` compare the CUDA path against.

Each function restates, in torch on the CPU, the arithmetic of one reference function; the reference lines it
follows are cited per function (paths inside the DeepGEMM tree). The restatement is pinned bit-for-bit against
outputs of the reference's own ``deep_gemm/utils/math.py`` and ``deep_gemm/testing/numeric.py`` (imported by
file path when the fixtures were generated): see ``tests/golden/make_golden.py`` and ``tests/test_oracle_golden.py``.
"""
from typing import Tuple

import torch

E2M1_MAGNITUDES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
# Decision thresholds between neighbouring E2M1 magnitudes; a value exactly on a threshold goes DOWN.
E2M1_THRESHOLDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)


def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def align(a: int, b: int) -> int:
    return ceil_div(a, b) * b


def ue8m0_ceil(x: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= |x| as fp32, biased exponent clamped to [1, 254].

    Follows ``ceil_to_ue8m0`` (deep_gemm/utils/math.py:13-16)."""
    bits = x.abs().float().contiguous().view(torch.int32)
    exponent = (bits >> 23) & 0xFF
    has_mantissa = (bits & 0x7FFFFF) != 0
    exponent = (exponent + has_mantissa.to(torch.int32)).clamp_(1, 254)
    return (exponent << 23).view(torch.float32)


def ue8m0_bytes(sf: torch.Tensor) -> torch.Tensor:
    """Biased-exponent byte of a power-of-two fp32 scale (deep_gemm/utils/math.py:19-23, the `>> 23` step)."""
    bits = sf.contiguous().view(torch.int32)
    assert bool((bits >= 0).all()) and bool(((bits & 0x7FFFFF) == 0).all()), 'scales must be positive powers of two'
    return (bits >> 23).to(torch.uint8)


def pack_ue8m0(sf: torch.Tensor) -> torch.Tensor:
    """fp32 power-of-two scales [..., 4n] -> int32 [..., n]; byte j of int i is K block 4i+j (little endian).

    Follows ``pack_ue8m0_to_int`` (deep_gemm/utils/math.py:19-23)."""
    assert sf.dtype == torch.float32 and sf.shape[-1] % 4 == 0
    return ue8m0_bytes(sf).view(torch.int32)


def unpack_ue8m0(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`pack_ue8m0` (deep_gemm/utils/math.py:148-149)."""
    return (packed.contiguous().view(torch.uint8).to(torch.int32) << 23).view(torch.float32)


def _blocked_amax(x: torch.Tensor, gran_k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    m, n = x.shape
    padded = torch.zeros((m, align(n, gran_k)), dtype=x.dtype)
    padded[:, :n] = x
    blocks = padded.view(m, -1, gran_k)
    return blocks, blocks.abs().float().amax(dim=2)


def quantize_fp8_per_token(x: torch.Tensor, gran_k: int = 128, packed: bool = False):
    """Activation quantiser: per row, per ``gran_k`` block, UE8M0 scale + E4M3 round-to-nearest-even.

    Follows ``per_token_cast_to_fp8(use_ue8m0=True)`` (deep_gemm/utils/math.py:26-49):
    ``sf = ue8m0_ceil(max(amax, 1e-4) / 448)``, ``q = e4m3(x * (1 / sf))``. Returns (q [m, n] float8_e4m3fn,
    sf fp32 [m, ceil(n / gran_k)]) or, with ``packed``, sf as int32 [m, ceil(n / gran_k / 4)] (missing scales
    padded with 1.0 = byte 127)."""
    assert x.dim() == 2
    m, n = x.shape
    blocks, amax = _blocked_amax(x, gran_k)
    sf = ue8m0_ceil(amax.clamp(min=1e-4) / 448.0)
    q = (blocks * (1.0 / sf.unsqueeze(2))).to(torch.float8_e4m3fn).view(m, -1)[:, :n].contiguous()
    if packed:
        pad = align(sf.shape[1], 4) - sf.shape[1]
        if pad:
            sf = torch.nn.functional.pad(sf, (0, pad), value=1.0)
        return q, pack_ue8m0(sf)
    return q, sf


def quantize_fp8_per_channel(x: torch.Tensor, gran_k: int = 128):
    """Operand quantiser of the K-grouped GEMM: x [k, mn] with k a multiple of ``gran_k``; one UE8M0 scale per ``gran_k``
    K rows and channel. Follows ``per_channel_cast_to_fp8(use_ue8m0=True)`` (deep_gemm/utils/math.py:52-59):
    ``sf = ue8m0_ceil(max(amax, 1e-4) / 448)``, ``q = e4m3(x * (1 / sf))``. Returns (q e4m3 [k, mn], sf fp32 [k / gran_k, mn])."""
    assert x.dim() == 2 and x.shape[0] % gran_k == 0
    k, mn = x.shape
    view = x.float().view(-1, gran_k, mn)
    sf = ue8m0_ceil(view.abs().amax(dim=1).clamp(min=1e-4) / 448.0)
    q = (view * (1.0 / sf.unsqueeze(1))).to(torch.float8_e4m3fn).view(k, mn)
    return q, sf


def e2m1_codes(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> 4-bit E2M1 codes (uint8): magnitude index 0..7 by strict-greater thresholds, sign in bit 3,
    negative zero canonicalised to +0. Follows ``_quantize_to_fp4_e2m1`` (deep_gemm/utils/math.py:84-93)."""
    thresholds = torch.tensor(E2M1_THRESHOLDS, dtype=torch.float32)
    magnitude = torch.bucketize(x.abs().float().contiguous(), thresholds, right=False).to(torch.uint8)
    negative = (x < 0) & (magnitude != 0)
    return magnitude | (negative.to(torch.uint8) << 3)


def quantize_fp4_per_token(x: torch.Tensor, gran_k: int = 32, packed: bool = False):
    """Weight quantiser (MXFP4): ``sf = ue8m0_ceil(max(amax, 1e-4) / 6)``, E2M1 codes of ``x / sf``, two codes
    per byte with the even K index in the low nibble.

    Follows ``per_token_cast_to_fp4(use_ue8m0=True)`` (deep_gemm/utils/math.py:96-122). Returns
    (int8 [m, n / 2], sf fp32 [m, ceil(n / gran_k)] or packed int32)."""
    m, n = x.shape
    assert n % 2 == 0
    blocks, amax = _blocked_amax(x, gran_k)
    sf = ue8m0_ceil(amax.clamp(min=1e-4) / 6.0)
    codes = e2m1_codes(blocks * (1.0 / sf.unsqueeze(2))).view(m, -1)
    packed_codes = (codes[:, 0::2] | (codes[:, 1::2] << 4)).view(torch.int8)[:, : n // 2].contiguous()
    if packed:
        pad = align(sf.shape[1], 4) - sf.shape[1]
        if pad:
            sf = torch.nn.functional.pad(sf, (0, pad), value=1.0)
        return packed_codes, pack_ue8m0(sf)
    return packed_codes, sf


def e2m1_values(codes: torch.Tensor) -> torch.Tensor:
    """4-bit codes -> fp32 values (deep_gemm/utils/math.py:141-145)."""
    table = torch.tensor(E2M1_MAGNITUDES + tuple(-v for v in E2M1_MAGNITUDES), dtype=torch.float32)
    table[8] = 0.0  # code 0b1000 decodes to +0
    return table[codes.to(torch.int64) & 0xF]


def unpack_fp4(packed: torch.Tensor) -> torch.Tensor:
    """int8 [m, n/2] -> uint8 codes [m, n], low nibble first."""
    raw = packed.contiguous().view(torch.uint8)
    codes = torch.empty((raw.shape[0], raw.shape[1] * 2), dtype=torch.uint8)
    codes[:, 0::2] = raw & 0xF
    codes[:, 1::2] = raw >> 4
    return codes


def dequantize_fp4(packed: torch.Tensor, sf: torch.Tensor, gran_k: int = 32) -> torch.Tensor:
    """Follows ``cast_back_from_fp4`` (deep_gemm/utils/math.py:152-164); ``sf`` fp32 or packed int32."""
    if sf.dtype == torch.int32:
        sf = unpack_ue8m0(sf)
    values = e2m1_values(unpack_fp4(packed))
    block = torch.arange(values.shape[1]) // gran_k
    return values * sf[:, block]


def dequantize_fp8(q: torch.Tensor, sf: torch.Tensor, gran_k: int = 128) -> torch.Tensor:
    """Follows ``cast_back_from_fp8`` (deep_gemm/utils/math.py:167-173); ``sf`` fp32 or packed int32."""
    if sf.dtype == torch.int32:
        sf = unpack_ue8m0(sf)
    block = torch.arange(q.shape[1]) // gran_k
    return q.float() * sf[:, block]


def calc_diff(x: torch.Tensor, y: torch.Tensor) -> float:
    """1 - 2<x,y> / (|x|^2 + |y|^2) in float64; 0 when both are all-zero.

    Follows ``calc_diff`` (deep_gemm/testing/numeric.py:5-11)."""
    x, y = x.double(), y.double()
    denominator = float((x * x + y * y).sum())
    if denominator == 0.0:
        return 0.0
    return 1.0 - 2.0 * float((x * y).sum()) / denominator
