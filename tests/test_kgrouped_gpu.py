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
    return quant.quantize_fp8_per_channel(x, 128)


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
        dg.k_grouped_fp8_gemm_tn_contiguous(*args, [128], layout, c=d, recipe=(1, 1, 64))
    with pytest.raises(RuntimeError):
        dg.k_grouped_fp8_gemm_tn_contiguous(*args, [64], layout, c=d)


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


def _psum_case(real_ks, m, n, alignment, seed):
    """Inputs as the reference's generate_k_grouped_contiguous_psum builds them (tests/generators.py:492-533): every group
    starts at a multiple of the alignment, the gap rows are zero."""
    torch.manual_seed(seed)
    ends, prev = [], 0
    for k in real_ks:
        prev = -(-prev // alignment) * alignment + k
        ends.append(prev)
    total = -(-ends[-1] // alignment) * alignment
    a, b = torch.zeros(total, m).bfloat16(), torch.zeros(total, n).bfloat16()
    for k, end in zip(real_ks, ends):
        a[end - k:end] = torch.randn(k, m).bfloat16()
        b[end - k:end] = torch.randn(k, n).bfloat16()
    return a, b, ends, total


@pytest.mark.parametrize('real_ks,m,n', [([300, 0, 129, 1000], 128, 256), ([128, 5, 2049], 256, 128), ([4000, 1111], 384, 512)])
@pytest.mark.parametrize('fp8', [True, False])
def test_k_grouped_psum_layout(dg, real_ks, m, n, fp8):
    from deepgemm_b200 import _lib
    alignment = dg.get_mk_alignment_for_contiguous_layout()
    assert alignment == 128
    a, b, ends, total = _psum_case(real_ks, m, n, alignment, seed=sum(real_ks))
    c = torch.randn(len(real_ks), m, n) * 32
    d = c.cuda()
    layout = torch.tensor(ends, dtype=torch.int32, device='cuda')
    if fp8:
        a_q, b_q = torch.zeros(total, m, dtype=torch.float8_e4m3fn), torch.zeros(total, n, dtype=torch.float8_e4m3fn)
        a_sfs, b_sfs = [], []
        for k, end in zip(real_ks, ends):  # per group, padded to a multiple of 128 rows (tests/generators.py:425-433)
            if k == 0:
                continue
            pad = -(-k // 128) * 128
            for src, q_out, sfs, mn in ((a, a_q, a_sfs, m), (b, b_q, b_sfs, n)):
                block = torch.zeros(pad, mn).bfloat16()
                block[:k] = src[end - k:end]
                q, sf = _per_channel_fp8(block)
                q_out[end - k:end] = q[:k]
                sfs.append(sf)
        a_sf, b_sf = torch.cat(a_sfs), torch.cat(b_sfs)
        want = ogemm.k_grouped_gemm_psum(a_q, a_sf, b_q, b_sf, c, ends, alignment)
        dg.k_grouped_fp8_gemm_tn_contiguous((a_q.cuda(), a_sf.cuda()), (b_q.cuda(), b_sf.cuda()), d, None, layout, c=d,
                                            use_psum_layout=True)
        tol = FP8_TOL
    else:
        want = ogemm.k_grouped_gemm_psum(a, None, b, None, c, ends, alignment)
        dg.k_grouped_bf16_gemm_tn_contiguous(a.cuda(), b.cuda(), d, None, layout, c=d, use_psum_layout=True)
        tol = 1e-5
    assert _lib.device_status()[0] == 0
    got = d.cpu()
    for g, k in enumerate(real_ks):
        if k == 0:
            assert torch.equal(got[g], c[g])
        else:
            assert quant.calc_diff(got[g] - c[g], want[g] - c[g]) <= tol


@pytest.mark.parametrize('ks,m,n', [([256, 128, 640], 128, 256), ([4096, 0, 2048], 256, 512)])
def test_k_grouped_recipe_32(dg, ks, m, n):
    """One scale per 32 K rows and channel (recipe (1, 1, 32))."""
    from deepgemm_b200 import _lib
    torch.manual_seed(sum(ks))
    k = sum(ks)
    a_q, a_sf = quant.quantize_fp8_per_channel(torch.randn(k, m).bfloat16() * torch.logspace(-2, 2, k).unsqueeze(1), 32)
    b_q, b_sf = quant.quantize_fp8_per_channel(torch.randn(k, n).bfloat16(), 32)
    c = torch.randn(len(ks), m, n)
    want = ogemm.k_grouped_gemm(a_q, a_sf, b_q, b_sf, c, ks, gran_k=32)
    d = c.cuda()
    layout = torch.tensor(ks, dtype=torch.int32, device='cuda')
    dg.k_grouped_fp8_gemm_tn_contiguous((a_q.cuda(), a_sf.cuda()), (b_q.cuda(), b_sf.cuda()), d, ks, layout, c=d,
                                        recipe=(1, 1, 32))
    assert _lib.device_status()[0] == 0
    got = d.cpu()
    for g, kg in enumerate(ks):
        if kg == 0:
            assert torch.equal(got[g], c[g])
        else:
            assert quant.calc_diff(got[g] - c[g], want[g] - c[g]) <= FP8_TOL


def test_k_grouped_rejects_extents_that_disagree_with_the_host_list(dg):
    """Plain layout: the kernel only sees the device-side extents. Extents that are not whole K blocks (or that overrun
    the operands) are reported through the status block and their groups left untouched (d keeps c); nothing reads the
    neighbouring group's rows."""
    from deepgemm_b200 import _lib
    torch.manual_seed(5)
    ks_host = [128, 128]
    m, n = 128, 128
    a, b = torch.randn(sum(ks_host), m).bfloat16().cuda(), torch.randn(sum(ks_host), n).bfloat16().cuda()
    c = torch.randn(2, m, n)
    d = c.cuda()
    lying = torch.tensor([96, 160], dtype=torch.int32, device='cuda')  # same sum, neither a multiple of 64
    dg.k_grouped_bf16_gemm_tn_contiguous(a, b, d, ks_host, lying, c=d)
    status = _lib.device_status(raise_on_error=False)
    assert status[0] == 6, status  # bad argument
    assert _lib.device_status()[0] == 0  # reading the status block clears it
    assert torch.equal(d.cpu(), c)
    overrun = torch.tensor([128, 256], dtype=torch.int32, device='cuda')  # the second group runs past the operands
    dg.k_grouped_bf16_gemm_tn_contiguous(a, b, d, ks_host, overrun, c=d)
    status = _lib.device_status(raise_on_error=False)
    assert status[0] == 6 and status[2] == 1, status
    got = d.cpu()
    assert torch.equal(got[1], c[1])
    assert quant.calc_diff(got[0] - c[0], a[:128].float().T.cpu() @ b[:128].float().cpu()) < 1e-5
