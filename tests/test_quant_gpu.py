"""Bit-exact parity of the quantisation and scale-factor layout kernels against the CPU oracle."""
import pytest
import torch

from oracle import layout as olay
from oracle import quant

pytestmark = pytest.mark.gpu


@pytest.fixture(scope='module')
def dg():
    import deepgemm_b200
    return deepgemm_b200


def _inputs(rows, k, seed):
    torch.manual_seed(seed)
    x = torch.randn(rows, k)
    x[0] = 0
    if rows > 2:
        x[1] *= 1e-5
        x[2] *= 3e3
    x[-1, :32] = 448.0 * 2.0 ** -4
    return x.bfloat16()


@pytest.mark.parametrize('rows,k', [(1, 128), (33, 7168), (70, 1024), (129, 2048), (5, 1536), (64, 48)])
@pytest.mark.parametrize('gran', [32, 128])
def test_fp8_cast_bit_exact(dg, rows, k, gran):
    x = _inputs(rows, k, seed=rows + k)
    want_q, want_sf = quant.quantize_fp8_per_token(x, gran)
    q, sf = dg.utils.per_token_cast_to_fp8(x.cuda(), use_ue8m0=True, gran_k=gran)
    assert torch.equal(q.cpu().view(torch.uint8), want_q.view(torch.uint8))
    assert torch.equal(sf.cpu(), want_sf)
    _, want_packed = quant.quantize_fp8_per_token(x, gran, packed=True)
    q2, packed = dg.utils.per_token_cast_to_fp8(x.cuda(), use_ue8m0=True, gran_k=gran, use_packed_ue8m0=True)
    assert torch.equal(packed.cpu(), want_packed) and torch.equal(q2.cpu().view(torch.uint8), want_q.view(torch.uint8))
    q3, mn = dg.utils.per_token_cast_to_fp8_mn_major(x.cuda(), gran_k=gran)
    assert mn.stride() == (1, -(-rows // 4) * 4)
    assert torch.equal(mn.cpu(), want_packed)


@pytest.mark.parametrize('rows,k', [(40, 256), (33, 7168), (128, 2048)])
@pytest.mark.parametrize('gran', [32, 128])
def test_fp4_cast_bit_exact(dg, rows, k, gran):
    torch.manual_seed(rows)
    w = (torch.randn(rows, k) * 0.02).bfloat16()
    w[0] = 0
    w[1, :8] = torch.tensor([0.25, -0.75, 1.25, -1.75, 2.5, -3.5, 5.0, -6.0]).bfloat16() * 2.0 ** -6
    want_q, want_sf = quant.quantize_fp4_per_token(w, gran)
    q, sf = dg.utils.per_token_cast_to_fp4(w.cuda(), use_ue8m0=True, gran_k=gran)
    assert torch.equal(q.cpu(), want_q) and torch.equal(sf.cpu(), want_sf)
    back = dg.utils.cast_back_from_fp4(q, sf, gran_k=gran).cpu()
    assert torch.equal(back, quant.dequantize_fp4(want_q, want_sf, gran))


@pytest.mark.parametrize('groups,mn,sf_k', [(1, 70, 8), (3, 132, 16), (2, 64, 18), (4, 5, 1)])
def test_sf_pack_bit_exact(dg, groups, mn, sf_k):
    torch.manual_seed(mn)
    sf = quant.ue8m0_ceil(torch.rand(groups, mn, sf_k) * 8 + 1e-4)
    got = dg.get_mn_major_tma_aligned_packed_ue8m0_tensor(sf.cuda())
    want = olay.pack_sf_mn_major(sf)
    assert got.shape == want.shape and got.stride() == want.stride()
    assert torch.equal(got.cpu(), want)
    # MN-major (transposed) input goes through the same kernel
    sf_t = sf.transpose(1, 2).contiguous().transpose(1, 2)
    assert torch.equal(dg.get_mn_major_tma_aligned_packed_ue8m0_tensor(sf_t.cuda()).cpu(), want)
    if groups == 1:
        got2 = dg.transform_sf_into_required_layout(sf[0].cuda(), mn, sf_k * 32, (1, 32))
        assert torch.equal(got2.cpu(), want[0])


def test_sf_pack_psum_gaps_pack_as_zero(dg):
    """Rows between a group's end and the next aligned start may hold garbage; they must pack as 0."""
    sf = quant.ue8m0_ceil(torch.rand(300, 4) + 0.1)
    sf[100:128] = float('nan')
    sf[200:256] = -3.0
    psum = torch.tensor([100, 200, 300], dtype=torch.int32)
    got = dg.transform_sf_into_required_layout(sf.cuda(), 300, 512, (1, 128), psum_layout=psum.cuda()).cpu()
    clean = sf.clone()
    clean[100:128] = 0
    clean[200:256] = 0
    want = olay.pack_sf_mn_major(torch.where(clean == 0, torch.ones(()), clean))
    valid = torch.ones(300, dtype=torch.bool)
    valid[100:128] = False
    valid[200:256] = False
    assert torch.equal(got[valid], want[valid])
    assert (got[~valid] == 0).all()
    from deepgemm_b200 import _lib
    assert _lib.device_status()[0] == 0


def test_non_power_of_two_scale_is_reported_not_trapped(dg):
    from deepgemm_b200 import _lib
    sf = torch.full((8, 4), 3.0)
    dg.get_mn_major_tma_aligned_packed_ue8m0_tensor(sf.cuda())
    with pytest.raises(RuntimeError, match='device status'):
        _lib.device_status()
    assert _lib.device_status()[0] == 0  # cleared by the read


def test_router_matches_oracle(dg):
    from oracle import moe as omoe
    torch.manual_seed(0)
    logits = torch.randn(1000, 256)
    logits[3, 7] = logits[3, 9]  # a tie: the lower index must win
    idx, w = dg.route_sigmoid_topk(logits.cuda(), 8)
    want_idx, want_w = omoe.route_sigmoid_topk(logits, 8)
    assert torch.equal(idx.cpu(), want_idx)
    assert torch.allclose(w.cpu(), want_w, rtol=2e-6, atol=1e-7)


@pytest.mark.parametrize('k,mn', [(128, 2), (384, 48), (1024, 7168), (256, 4098)])
@pytest.mark.parametrize('gran', [32, 128])
def test_per_channel_fp8_cast_bit_exact(dg, k, mn, gran):
    """Operand quantiser of the K-grouped GEMM: one scale per `gran` K rows and channel."""
    x = _inputs(k, mn, seed=k + mn)
    x[:gran, 0] = 0  # an all-zero (K block, channel)
    want_q, want_sf = quant.quantize_fp8_per_channel(x, gran)
    q, sf = dg.utils.per_channel_cast_to_fp8(x.cuda(), use_ue8m0=True, gran_k=gran)
    assert torch.equal(q.cpu().view(torch.uint8), want_q.view(torch.uint8))
    assert torch.equal(sf.cpu(), want_sf)
    with pytest.raises(RuntimeError):
        dg.utils.per_channel_cast_to_fp8(x[:gran - 1].cuda(), use_ue8m0=True, gran_k=gran)
