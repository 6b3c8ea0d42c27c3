"""Parity of the K-grouped FP8 GEMM (CUDA, through the C ABI) against the CPU oracle: d[g] = c[g] + A_g^T B_g with
per-channel UE8M0 scales over 128 K rows. FP8 x FP8 tolerance as stated for the task: calc_diff <= 1e-3."""
import pytest
import torch

from oracle import gemm as ogemm
from oracle import quant

pytestmark = pytest.mark.gpu
FP8_TOL = 1e-3


@pytest.fixture(scope='module')
def dg():
    import deepgemm_b200
    return deepgemm_b200


def _per_channel_fp8(x):
    """[k, mn] bf16 -> (e4m3 [k, mn], fp32 [k / 128, mn]): one UE8M0 scale per 128 K rows and channel, the
    reference's per_channel_cast_to_fp8(use_ue8m0=True) (deep_gemm/utils/math.py:52-59)."""
    q, sf = quant.quantize_fp8_per_token(x.T.contiguous(), 128)
    return q.T.contiguous(), sf.T.contiguous()


def _case(ks, m, n, seed):
    torch.manual_seed(seed)
    k = sum(ks)
    a = torch.randn(k, m).bfloat16()
    b = torch.randn(k, n).bfloat16()
    c = torch.randn(len(ks), m, n) * 32
    a_q, a_sf = _per_channel_fp8(a)
    b_q, b_sf = _per_channel_fp8(b)
    return a_q, a_sf, b_q, b_sf, c


@pytest.mark.parametrize('ks,m,n', [
    ([128], 128, 128),
    ([256, 128, 640], 128, 256),
    ([512, 0, 1024, 384], 256, 128),
    ([128 * 5, 128 * 9, 128 * 2], 192, 384),
    ([4096, 2048], 512, 512),
])
@pytest.mark.parametrize('alias', [True, False])
def test_k_grouped_matches_oracle(dg, ks, m, n, alias):
    from deepgemm_b200 import _lib
    a_q, a_sf, b_q, b_sf, c = _case(ks, m, n, seed=sum(ks) + m)
    want = ogemm.k_grouped_gemm(a_q, a_sf, b_q, b_sf, c, ks)
    c_dev = c.cuda()
    d = c_dev if alias else torch.full_like(c_dev, float('nan'))
    layout = torch.tensor(ks, dtype=torch.int32, device='cuda')
    dg.k_grouped_fp8_gemm_tn_contiguous((a_q.cuda(), a_sf.cuda()), (b_q.cuda(), b_sf.cuda()), d, ks, layout, c=c_dev)
    assert _lib.device_status()[0] == 0
    got = d.cpu()
    assert not torch.isnan(got).any()
    for g, k in enumerate(ks):
        if k == 0:
            assert torch.equal(got[g], c[g]), 'an empty group must pass c through'
        else:
            # compare the product alone: c is 32x larger than it needs to be to hide an error in the sum
            assert quant.calc_diff(got[g] - c[g], want[g] - c[g]) <= FP8_TOL


def test_rejected_inputs(dg):
    a_q, a_sf, b_q, b_sf, c = _case([128], 128, 128, seed=1)
    d = c.cuda()
    layout = torch.tensor([128], dtype=torch.int32, device='cuda')
    args = ((a_q.cuda(), a_sf.cuda()), (b_q.cuda(), b_sf.cuda()), d)
    with pytest.raises(RuntimeError):
        dg.k_grouped_fp8_gemm_tn_contiguous(*args, [128], layout, c=None)
    with pytest.raises(RuntimeError):
        dg.k_grouped_fp8_gemm_tn_contiguous(*args, [128], layout, c=d, recipe=(1, 1, 32))
    with pytest.raises(RuntimeError):
        dg.k_grouped_fp8_gemm_tn_contiguous(*args, [64], layout, c=d)
    with pytest.raises(RuntimeError):
        dg.k_grouped_fp8_gemm_tn_contiguous(*args, [128], layout, c=d, use_psum_layout=True)


@pytest.mark.parametrize('ks,m,n', [
    ([64], 128, 128),
    ([192, 64, 640], 128, 256),
    ([512, 0, 1088, 320], 256, 128),
    ([64 * 5, 64 * 9], 200, 384),
    ([4096, 2048], 512, 512),
])
def test_k_grouped_bf16_matches_oracle(dg, ks, m, n):
    """BF16 form: the reference checks it against the torch product of the same tensors with calc_diff < 1e-5 ... here
    the FP32 product of the BF16 operands."""
    from deepgemm_b200 import _lib
    torch.manual_seed(sum(ks) + n)
    k = sum(ks)
    a, b = torch.randn(k, m).bfloat16(), torch.randn(k, n).bfloat16()
    c = torch.randn(len(ks), m, n) * 32
    d = c.cuda()
    layout = torch.tensor(ks, dtype=torch.int32, device='cuda')
    dg.k_grouped_bf16_gemm_tn_contiguous(a.cuda(), b.cuda(), d, ks, layout, c=d)
    assert _lib.device_status()[0] == 0
    got, start = d.cpu(), 0
    for g, kg in enumerate(ks):
        if kg == 0:
            assert torch.equal(got[g], c[g])
        else:
            want = a[start:start + kg].float().T @ b[start:start + kg].float()
            assert quant.calc_diff(got[g] - c[g], want) < 1e-5
        start += kg
