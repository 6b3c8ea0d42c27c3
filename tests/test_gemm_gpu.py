"""Parity of the m-grouped FP8 x FP4 GEMMs (CUDA, through the C ABI) against the CPU oracle.
Tolerances are the ones the task states: calc_diff <= 2e-3 with an FP4 operand, <= 1e-3 for FP8 x FP8."""
import pytest
import torch

from oracle import gemm as ogemm
from oracle import layout as olay
from oracle import quant
from tests.helpers import contiguous_case, quantize_groups

pytestmark = pytest.mark.gpu

FP4_TOL, FP8_TOL = 2e-3, 1e-3


@pytest.fixture(scope='module')
def dg():
    import deepgemm_b200
    return deepgemm_b200


def _cuda_packed(sf):
    """oracle-packed MN-major scale factors on the GPU with their strides intact"""
    three = sf.dim() == 3
    dense = olay.pack_sf_dense(sf if three else sf.unsqueeze(0)).cuda()
    view = dense.transpose(1, 2)[:, :sf.shape[-2], :]
    return view if three else view[0]


def _finish(dg):
    from deepgemm_b200 import _lib
    assert _lib.device_status()[0] == 0


@pytest.mark.parametrize('use_psum', [False, True])
@pytest.mark.parametrize('sf_as_fp32', [False, True])
def test_config1_contiguous(dg, use_psum, sf_as_fp32):
    """4 experts, N=512, K=1024, rows per expert uniform in [64, 256], segments padded to 128 (seed 0)."""
    c = contiguous_case(4, 512, 1024, 64, 256, seed=0)
    layout = c['psum'] if use_psum else c['row_ids']
    want, mask = ogemm.grouped_gemm_contiguous(c['a_q'], c['a_sf'], c['b_q'], c['b_sf'], layout, 128, 32,
                                               use_psum_layout=use_psum)
    d = torch.full((c['m'], 512), float('nan'), dtype=torch.bfloat16, device='cuda')
    a_sf = c['a_sf'].cuda() if sf_as_fp32 else _cuda_packed(c['a_sf'])
    b_sf = c['b_sf'].cuda() if sf_as_fp32 else _cuda_packed(c['b_sf'])
    dg.m_grouped_fp8_fp4_gemm_nt_contiguous((c['a_q'].cuda(), a_sf), (c['b_q'].cuda(), b_sf), d, layout.cuda(),
                                            recipe_a=(1, 128), recipe_b=(1, 32), use_psum_layout=use_psum,
                                            ensure_zero_padding=False)
    _finish(dg)
    got = d.cpu()
    assert not torch.isnan(got[mask].float()).any()
    assert quant.calc_diff(got[mask], want[mask]) <= FP4_TOL
    assert (got[mask].float() - want[mask].float()).abs().max() <= 0.02 * want.float().abs().max()
    if use_psum:
        assert torch.isnan(got[~mask].float()).all(), 'rows outside the groups must not be written'


def test_psum_zero_padding_rows_are_written(dg):
    """ensure_zero_padding=True: rows up to each group's aligned end are written and are zero when A's padding is."""
    c = contiguous_case(3, 256, 512, 40, 200, seed=3)
    d = torch.full((c['m'], 256), float('nan'), dtype=torch.bfloat16, device='cuda')
    dg.m_grouped_fp8_fp4_gemm_nt_contiguous((c['a_q'].cuda(), c['a_sf'].cuda()), (c['b_q'].cuda(), c['b_sf'].cuda()),
                                            d, c['psum'].cuda(), recipe_a=(1, 128), recipe_b=(1, 32),
                                            use_psum_layout=True, ensure_zero_padding=True)
    _finish(dg)
    got = d.cpu().float()
    assert not torch.isnan(got).any()
    assert (got[c['row_ids'] < 0] == 0).all()


@pytest.mark.parametrize('gran_a', [32, 128])
def test_fp8_activation_granularities_and_odd_alignment(dg, gran_a):
    """psum layout with a 16-row alignment: tiles start off the 128-row grid and span group boundaries."""
    dg.set_mk_alignment_for_contiguous_layout(16)
    try:
        c = contiguous_case(5, 256, 768, 1, 300, seed=11, alignment=16, gran_a=gran_a)
        want, mask = ogemm.grouped_gemm_contiguous(c['a_q'], c['a_sf'], c['b_q'], c['b_sf'], c['psum'], gran_a, 32,
                                                   use_psum_layout=True, alignment=16)
        d = torch.full((c['m'], 256), float('nan'), dtype=torch.bfloat16, device='cuda')
        dg.m_grouped_fp8_fp4_gemm_nt_contiguous((c['a_q'].cuda(), _cuda_packed(c['a_sf'])),
                                                (c['b_q'].cuda(), _cuda_packed(c['b_sf'])), d, c['psum'].cuda(),
                                                recipe_a=(1, gran_a), recipe_b=(1, 32), use_psum_layout=True,
                                                ensure_zero_padding=False)
        _finish(dg)
    finally:
        dg.set_mk_alignment_for_contiguous_layout(128)
    got = d.cpu()
    assert quant.calc_diff(got[mask], want[mask]) <= FP4_TOL
    assert torch.isnan(got[~mask].float()).all()


def test_fp8_x_fp8_weights(dg):
    """The FP8-only alias: B is e4m3 with per-128 scales (1x128 on both sides)."""
    c = contiguous_case(2, 256, 512, 100, 128, seed=5, gran_b=128, b_fp4=False)
    want, mask = ogemm.grouped_gemm_contiguous(c['a_q'], c['a_sf'], c['b_q'], c['b_sf'], c['row_ids'], 128, 128)
    d = torch.zeros((c['m'], 256), dtype=torch.bfloat16, device='cuda')
    dg.m_grouped_fp8_gemm_nt_contiguous((c['a_q'].cuda(), _cuda_packed(c['a_sf'])),
                                        (c['b_q'].cuda(), _cuda_packed(c['b_sf'])), d, c['row_ids'].cuda(),
                                        recipe=(1, 1, 128))
    _finish(dg)
    assert quant.calc_diff(d.cpu()[mask], want[mask]) <= FP8_TOL


def _masked_case(num_groups, max_m, n, k, masked, seed):
    torch.manual_seed(seed)
    a = torch.randn(num_groups, max_m, k).bfloat16()
    b = (torch.randn(num_groups, n, k) * 0.02).bfloat16()
    a_q, a_sf = quantize_groups(a, 128, False)
    b_q, b_sf = quantize_groups(b, 32, True)
    return a_q, a_sf, b_q, b_sf, torch.tensor(masked, dtype=torch.int32)


def test_masked_edge_counts(dg):
    """masked_m of 0, 1, a tile boundary, boundary + 1 and the full buffer; rows past masked_m stay untouched."""
    a_q, a_sf, b_q, b_sf, masked = _masked_case(6, 256, 512, 1024, [0, 1, 128, 129, 255, 256], seed=1)
    want, mask = ogemm.grouped_gemm_masked(a_q, a_sf, b_q, b_sf, masked, 128, 32)
    d = torch.full((6, 256, 512), float('nan'), dtype=torch.bfloat16, device='cuda')
    dg.m_grouped_fp8_fp4_gemm_nt_masked((a_q.cuda(), a_sf.cuda()), (b_q.cuda(), b_sf.cuda()), d, masked.cuda(), 64,
                                        recipe_a=(1, 128), recipe_b=(1, 32))
    _finish(dg)
    got = d.cpu()
    assert quant.calc_diff(got[mask], want[mask]) <= FP4_TOL
    assert torch.isnan(got[~mask].float()).all()


def test_masked_max_m_not_a_tile_multiple(dg):
    """max_m = 200: the last tile of a full group must not spill into the next group's rows."""
    a_q, a_sf, b_q, b_sf, masked = _masked_case(3, 200, 256, 512, [200, 130, 200], seed=2)
    want, mask = ogemm.grouped_gemm_masked(a_q, a_sf, b_q, b_sf, masked, 128, 32)
    d = torch.full((3, 200, 256), float('nan'), dtype=torch.bfloat16, device='cuda')
    dg.m_grouped_fp8_fp4_gemm_nt_masked((a_q.cuda(), a_sf.cuda()), (b_q.cuda(), b_sf.cuda()), d, masked.cuda(), 200,
                                        recipe_a=(1, 128), recipe_b=(1, 32))
    _finish(dg)
    got = d.cpu()
    assert quant.calc_diff(got[mask], want[mask]) <= FP4_TOL
    assert torch.isnan(got[~mask].float()).all()


def test_config2_masked_decode_full_size(dg):
    """32 experts x 256-row buffers, valid rows ~ Poisson(64), N=4096, K=7168. Inputs are quantised on the GPU (the
    cast kernels are bit-exact against the oracle, see test_quant_gpu); four groups are checked against the oracle,
    all groups through linearity: doubling every A scale doubles D exactly."""
    torch.manual_seed(0)
    g, max_m, n, k = 32, 256, 4096, 7168
    masked = torch.poisson(torch.full((g,), 64.0)).clamp(0, max_m).to(torch.int32)
    a = torch.randn(g * max_m, k, device='cuda', dtype=torch.bfloat16)
    a_q, a_sf = dg.utils.per_token_cast_to_fp8(a, use_ue8m0=True, gran_k=128)
    del a
    b_q = torch.empty((g, n, k // 2), dtype=torch.int8, device='cuda')
    b_sf = torch.empty((g, n, k // 32), dtype=torch.float32, device='cuda')
    for i in range(g):
        w = torch.randn(n, k, device='cuda', dtype=torch.bfloat16) * 0.02
        b_q[i], b_sf[i] = dg.utils.per_token_cast_to_fp4(w, use_ue8m0=True, gran_k=32)
    a_q, a_sf = a_q.view(g, max_m, k), a_sf.view(g, max_m, -1)
    d = torch.full((g, max_m, n), float('nan'), dtype=torch.bfloat16, device='cuda')
    dg.m_grouped_fp8_fp4_gemm_nt_masked((a_q, a_sf), (b_q, b_sf), d, masked.cuda(), 64, recipe_a=(1, 128), recipe_b=(1, 32))
    d2 = torch.full_like(d, float('nan'))
    dg.m_grouped_fp8_fp4_gemm_nt_masked((a_q, a_sf * 2), (b_q, b_sf), d2, masked.cuda(), 64, recipe_a=(1, 128),
                                        recipe_b=(1, 32))
    _finish(dg)
    rows = torch.arange(max_m)[None, :] < masked[:, None]
    got, got2 = d.cpu(), d2.cpu()
    assert not torch.isnan(got[rows].float()).any()
    assert torch.isnan(got[~rows].float()).all()
    assert torch.equal(got2[rows].float(), got[rows].float() * 2)
    for i in (0, 7, 19, 31):
        m_i = int(masked[i])
        if m_i == 0:
            continue
        want, _ = ogemm.grouped_gemm_masked(a_q[i:i + 1].cpu(), a_sf[i:i + 1].cpu(), b_q[i:i + 1].cpu(),
                                            b_sf[i:i + 1].cpu(), masked[i:i + 1], 128, 32)
        assert quant.calc_diff(got[i, :m_i], want[0, :m_i]) <= FP4_TOL


def test_empty_and_rejected_inputs(dg):
    c = contiguous_case(2, 128, 256, 10, 20, seed=7)
    b = (c['b_q'].cuda(), c['b_sf'].cuda())
    # m == 0 is a no-op
    dg.m_grouped_fp8_fp4_gemm_nt_contiguous(
        (torch.empty((0, 256), dtype=torch.float8_e4m3fn, device='cuda'), torch.empty((0, 2), device='cuda')), b,
        torch.empty((0, 128), dtype=torch.bfloat16, device='cuda'), torch.empty(0, dtype=torch.int32, device='cuda'),
        recipe_a=(1, 128), recipe_b=(1, 32))
    a = (c['a_q'].cuda(), c['a_sf'].cuda())
    d = torch.empty((c['m'], 128), dtype=torch.bfloat16, device='cuda')
    with pytest.raises(RuntimeError):  # both recipe forms at once
        dg.m_grouped_fp8_fp4_gemm_nt_contiguous(a, b, d, c['row_ids'].cuda(), recipe=(1, 1, 128), recipe_a=(1, 128),
                                                recipe_b=(1, 32))
    with pytest.raises(RuntimeError):  # wrong output dtype
        dg.m_grouped_fp8_fp4_gemm_nt_contiguous(a, b, d.float(), c['row_ids'].cuda(), recipe_a=(1, 128), recipe_b=(1, 32))
    with pytest.raises(RuntimeError):  # layout length
        dg.m_grouped_fp8_fp4_gemm_nt_contiguous(a, b, d, c['row_ids'].cuda()[:-1].contiguous(), recipe_a=(1, 128),
                                                recipe_b=(1, 32))
    with pytest.raises(RuntimeError):  # scale-factor extent does not match the recipe
        dg.m_grouped_fp8_fp4_gemm_nt_contiguous(a, b, d, c['row_ids'].cuda(), recipe_a=(1, 32), recipe_b=(1, 32))
    _finish(dg)


@pytest.mark.parametrize('m,n,k,b_fp4,out', [
    (200, 512, 1024, True, torch.bfloat16),     # ragged M: the last tile is clipped at m
    (384, 256, 512, False, torch.float32),      # FP8 x FP8, FP32 output, 256-wide tiles with whole-tile TMA... stores
    (1, 128, 128, True, torch.bfloat16),
])
def test_dense_gemm(dg, m, n, k, b_fp4, out):
    """fp8_fp4_gemm_nt = the grouped kernel with one group and no layout array."""
    torch.manual_seed(m + n)
    a = torch.randn(m, k).bfloat16()
    b = (torch.randn(1, n, k) * 0.02).bfloat16()
    a_q, a_sf = quant.quantize_fp8_per_token(a, 128)
    b_q, b_sf = quantize_groups(b, 32 if b_fp4 else 128, b_fp4)
    want, _ = ogemm.grouped_gemm_contiguous(a_q, a_sf, b_q, b_sf, torch.zeros(m, dtype=torch.int32), 128, 32 if b_fp4 else 128,
                                            out_dtype=out)
    d = torch.full((m, n), float('nan'), dtype=out, device='cuda')
    dg.fp8_fp4_gemm_nt((a_q.cuda(), a_sf.cuda()), (b_q[0].cuda(), b_sf[0].cuda()), d, recipe_a=(1, 128),
                       recipe_b=(1, 32 if b_fp4 else 128))
    _finish(dg)
    assert not torch.isnan(d.float()).any()
    assert quant.calc_diff(d.cpu().float(), want.float()) <= (FP4_TOL if b_fp4 else FP8_TOL)
    args = ((a_q.cuda(), a_sf.cuda()), (b_q[0].cuda(), b_sf[0].cuda()))
    recipes = dict(recipe_a=(1, 128), recipe_b=(1, 32 if b_fp4 else 128))
    if out == torch.float32:
        # the accumulator input: d = c + a @ b.T, c given separately or as d itself
        c = torch.randn(m, n, device='cuda') * 3
        d2 = torch.full_like(d, float('nan'))
        dg.fp8_fp4_gemm_nt(*args, d2, c=c, **recipes)
        d3 = c.clone()
        dg.fp8_fp4_gemm_nt(*args, d3, c=d3, **recipes)
        _finish(dg)
        assert torch.equal(d2, c + d) and torch.equal(d3, d2)
    else:
        with pytest.raises(RuntimeError):
            dg.fp8_fp4_gemm_nt(*args, d, c=d, **recipes)  # accumulation needs float32


def _transpose_packed_fp4(q):
    """[N, K / 2] packed along K -> [K, N / 2] packed along N (even N index in the low nibble), the storage of an
    MN-major FP4 operand (the reference's test helper of the same purpose: deep_gemm/utils/math.py:125-138)."""
    n = q.shape[0]
    codes = torch.stack([q & 0x0F, (q >> 4) & 0x0F], dim=2).reshape(n, -1)  # [N, K] one code per element
    t = codes.t().contiguous().view(-1, n // 2, 2)
    return ((t[:, :, 0] & 0x0F) | ((t[:, :, 1] & 0x0F) << 4)).to(torch.int8).contiguous()


@pytest.mark.parametrize('b_fp4', [False, True])
@pytest.mark.parametrize('via_nn', [False, True])
def test_mn_major_b(dg, b_fp4, via_nn):
    """b stored [G, K, N] (N contiguous; packed FP4: [G, K, N / 2]): the operand of m_grouped_fp8_fp4_gemm_nn_contiguous,
    which the NT form also accepts as a transposed view (reference: csrc/apis/gemm.hpp:181-183, :234-248). Same numbers
    as the K-major storage of the same weights."""
    gran_b = 32 if b_fp4 else 128
    c = contiguous_case(3, 384, 512, 50, 260, seed=17, gran_b=gran_b, b_fp4=b_fp4)
    want, mask = ogemm.grouped_gemm_contiguous(c['a_q'], c['a_sf'], c['b_q'], c['b_sf'], c['row_ids'], 128, gran_b)
    if b_fp4:
        storage = torch.stack([_transpose_packed_fp4(c['b_q'][g]) for g in range(3)]).cuda()  # [G, K, N / 2]
    else:
        storage = c['b_q'].transpose(1, 2).contiguous().cuda()                                 # [G, K, N]
    sf = _cuda_packed(c['b_sf'])
    d = torch.full((c['m'], 384), float('nan'), dtype=torch.bfloat16, device='cuda')
    a = (c['a_q'].cuda(), _cuda_packed(c['a_sf']))
    if via_nn:
        dg.m_grouped_fp8_fp4_gemm_nn_contiguous(a, (storage, sf.transpose(1, 2)), d, c['row_ids'].cuda(),
                                                recipe_a=(1, 128), recipe_b=(1, gran_b))
    else:
        dg.m_grouped_fp8_fp4_gemm_nt_contiguous(a, (storage.transpose(1, 2), sf), d, c['row_ids'].cuda(),
                                                recipe_a=(1, 128), recipe_b=(1, gran_b))
    _finish(dg)
    got = d.cpu()
    assert not torch.isnan(got[mask].float()).any()
    assert quant.calc_diff(got[mask], want[mask]) <= (FP4_TOL if b_fp4 else FP8_TOL)
