"""CPU tests of the NVFP4 oracle. The reference has no NVFP4 code, so these pin the oracle to the published format
by hand-computed vectors and format properties, not to reference outputs (parity unpinned)."""
import torch

from oracle import nvfp4 as onv
from oracle import quant
from tests.helpers import moe_case_nvfp4


def test_hand_computed_vector():
    # One row of two 16-blocks. Tensor amax = 10.5 -> s_t = 10.5 / 2688 = 2^-8. Block 0 amax 10.5 ->
    # sf = (10.5 / 6) / s_t = 448. Block 1 amax 2.625 -> 112 (exact in e4m3). Elements: x / (sf * s_t).
    x = torch.zeros(1, 32)
    x[0, 0], x[0, 1], x[0, 2] = 10.5, -5.25, 0.875    # / 1.75 -> 6, -3, 0.5
    x[0, 16], x[0, 17] = 2.625, -0.65625               # / 0.4375 -> 6, -1.5
    q, sf, s_t = onv.quantize_nvfp4(x)
    assert float(s_t) == 2.0 ** -8
    assert sf.float().tolist() == [[448.0, 112.0]]
    codes = quant.unpack_fp4(q)[0].tolist()
    assert codes[:3] == [7, 8 | 5, 1] and codes[16:18] == [7, 8 | 3]
    assert all(c == 0 for c in codes[3:16] + codes[18:])
    back = onv.dequantize_nvfp4(q, sf, s_t)
    assert torch.allclose(back, x, rtol=1e-6, atol=0)


def test_zero_tensor_and_zero_block():
    q, sf, s_t = onv.quantize_nvfp4(torch.zeros(3, 64))
    assert float(s_t) == 1.0 and (sf.float() == 0).all() and (q == 0).all()
    x = torch.randn(4, 64)
    x[2, 16:32] = 0
    q, sf, s_t = onv.quantize_nvfp4(x)
    assert float(sf[2, 1].float()) == 0.0 and (quant.unpack_fp4(q)[2, 16:32] == 0).all()


def test_fixed_scale_saturates_block_scales():
    x = torch.randn(8, 128) * 10
    q, sf, s_t = onv.quantize_nvfp4(x, scale=torch.tensor(1e-4))
    assert float(sf.float().max()) == 448.0
    assert torch.isfinite(onv.dequantize_nvfp4(q, sf, s_t)).all()


def test_round_trip_error_bound():
    torch.manual_seed(0)
    x = torch.randn(64, 256).bfloat16()
    q, sf, s_t = onv.quantize_nvfp4(x)
    back = onv.dequantize_nvfp4(q, sf, s_t)
    # E2M1 steps are at most 2 wide at the top of the range (|v| in 4..6): error <= 1 unit of the block scale, plus
    # the e4m3 rounding of the scale itself (<= 1/16 relative on amax)
    bound = (sf.float() * s_t).repeat_interleave(16, dim=1) * 1.0 + x.float().abs() * 0.0625
    assert ((back - x.float()).abs() <= bound + 1e-12).all()
    assert quant.calc_diff(back, x.float()) < 0.01


def test_sf_packing_layout():
    sf = torch.arange(2 * 6 * 8, dtype=torch.uint8).view(2, 6, 8).view(torch.float8_e4m3fn)
    packed = onv.pack_sf_bytes_mn_major(sf)
    assert packed.shape == (2, 2, 8) and packed.dtype == torch.int32
    raw = packed.view(torch.uint8).view(2, 2, 8, 4)
    for g, kq, row, j in [(0, 0, 0, 0), (1, 1, 5, 3), (0, 1, 2, 1)]:
        assert int(raw[g, kq, row, j]) == int(sf.view(torch.uint8)[g, row, kq * 4 + j])
    assert (raw[:, :, 6:] == 0).all()


def test_grouped_gemm_matches_dense_products():
    torch.manual_seed(1)
    a = torch.randn(48, 256).bfloat16()
    b = (torch.randn(2, 64, 256) * 0.05).bfloat16()
    a_q, a_sf, a_s = onv.quantize_nvfp4(a)
    parts = [onv.quantize_nvfp4(b[g]) for g in range(2)]
    b_q, b_sf, b_s = (torch.stack([p[i] for p in parts]) for i in range(3))
    d, mask = onv.grouped_gemm_contiguous(a_q, a_sf, a_s, b_q, b_sf, b_s, torch.tensor([20, 44]), 16, torch.float32)
    assert mask.tolist() == [True] * 20 + [False] * 12 + [True] * 12 + [False] * 4
    assert quant.calc_diff(d[:20], a[:20].float() @ b[0].float().T) < 0.02
    assert quant.calc_diff(d[32:44], a[32:44].float() @ b[1].float().T) < 0.02


def test_layer_equals_per_token_evaluation():
    c = moe_case_nvfp4(10, 256, 256, 4, 2, seed=5)
    act_scale = onv.calibrate_act_scale(c['x_q'], c['x_sf'], c['x_scale'], c['topk_idx'], c['topk_weights'], c['l1_q'],
                                        c['l1_sf'], c['l1_scales'])
    y = onv.moe_layer_nvfp4(c['x_q'], c['x_sf'], c['x_scale'], c['topk_idx'], c['topk_weights'], c['l1_q'], c['l1_sf'],
                            c['l1_scales'], c['l2_q'], c['l2_sf'], c['l2_scales'], act_scale)
    x = onv.dequantize_nvfp4(c['x_q'], c['x_sf'], c['x_scale'])
    for t in range(10):
        acc = torch.zeros(256)
        for k in range(2):
            e = int(c['topk_idx'][t, k])
            a1 = x[t:t + 1] @ onv.dequantize_nvfp4(c['l1_q'][e], c['l1_sf'][e], c['l1_scales'][e]).T
            q, sf = onv.swiglu_requant_nvfp4(a1, c['topk_weights'][t:t + 1, k], None, act_scale)
            a2 = onv.dequantize_nvfp4(q, sf, act_scale) @ onv.dequantize_nvfp4(c['l2_q'][e], c['l2_sf'][e], c['l2_scales'][e]).T
            acc += a2.bfloat16().float()[0]
        assert quant.calc_diff(y[t], acc.bfloat16()) < 1e-6
    # the layer tracks the unquantised computation to FP4 accuracy
    assert torch.isfinite(y.float()).all()
