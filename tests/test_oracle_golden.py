"""Pins the CPU oracle bit-for-bit to outputs of the reference's own torch helpers (fixtures made by
tests/golden/make_golden.py from deep_gemm/utils/math.py and deep_gemm/testing/numeric.py)."""
import os

import numpy as np
import pytest
import torch

from oracle import layout as olay
from oracle import quant


@pytest.fixture(scope='module')
def gq(golden_dir):
    return np.load(os.path.join(golden_dir, 'quant.npz'))


@pytest.fixture(scope='module')
def gl(golden_dir):
    return np.load(os.path.join(golden_dir, 'layout.npz'))


def _bf16(arr):
    return torch.from_numpy(arr.copy()).view(torch.bfloat16)


@pytest.mark.parametrize('gran', [32, 128])
def test_fp8_quantiser_matches_reference(gq, gran):
    x = _bf16(gq['x_bf16'])
    q, sf = quant.quantize_fp8_per_token(x, gran)
    assert np.array_equal(q.view(torch.uint8).numpy(), gq[f'fp8_g{gran}_q'])
    assert np.array_equal(sf.numpy(), gq[f'fp8_g{gran}_sf'])
    _, sfp = quant.quantize_fp8_per_token(x, gran, packed=True)
    assert np.array_equal(sfp.numpy(), gq[f'fp8_g{gran}_sf_packed'])
    back = quant.dequantize_fp8(q, sf, gran)
    assert np.array_equal(back.numpy(), gq[f'fp8_g{gran}_back'])
    assert np.array_equal(quant.dequantize_fp8(q, sfp, gran).numpy(), gq[f'fp8_g{gran}_back'])


@pytest.mark.parametrize('gran', [32, 128])
@pytest.mark.parametrize('name', ['x', 'w'])
def test_fp4_quantiser_matches_reference(gq, gran, name):
    t = _bf16(gq[f'{name}_bf16'])
    q, sf = quant.quantize_fp4_per_token(t, gran)
    assert np.array_equal(q.numpy(), gq[f'fp4_{name}_g{gran}_q'])
    assert np.array_equal(sf.numpy(), gq[f'fp4_{name}_g{gran}_sf'])
    _, sfp = quant.quantize_fp4_per_token(t, gran, packed=True)
    assert np.array_equal(sfp.numpy(), gq[f'fp4_{name}_g{gran}_sf_packed'])
    assert np.array_equal(quant.dequantize_fp4(q, sf, gran).numpy(), gq[f'fp4_{name}_g{gran}_back'])


def test_ue8m0_ceil_and_pack_roundtrip(gq):
    probe = torch.from_numpy(gq['ue8m0_probe'].copy())
    assert np.array_equal(quant.ue8m0_ceil(probe).numpy(), gq['ue8m0_ceil'])
    sf = quant.ue8m0_ceil(torch.rand(7, 8) * 100 + 1e-5)
    assert torch.equal(quant.unpack_ue8m0(quant.pack_ue8m0(sf)), sf)


def test_calc_diff_matches_reference(gq):
    a, b = torch.from_numpy(gq['diff_a'].copy()), torch.from_numpy(gq['diff_b'].copy())
    assert quant.calc_diff(a, b) == pytest.approx(float(gq['diff_ab']), abs=1e-15)
    assert quant.calc_diff(a, a) == pytest.approx(float(gq['diff_aa']), abs=1e-15)
    assert quant.calc_diff(a, a * 1.01 + 0.001 * b) == pytest.approx(float(gq['diff_a_scaled']), abs=1e-15)
    assert quant.calc_diff(torch.zeros(4), torch.zeros(4)) == 0.0


@pytest.mark.parametrize('tag', ['a', 'b', 'c'])
def test_packed_sf_layout_matches_reference(gl, tag):
    sf = torch.from_numpy(gl[f'{tag}_sf'].copy())
    packed = olay.pack_sf_mn_major(sf)
    assert np.array_equal(packed.numpy(), gl[f'{tag}_packed'])
    assert list(packed.stride()) == list(gl[f'{tag}_strides'])
    assert np.array_equal(olay.pack_sf_mn_major(sf[0]).numpy(), gl[f'{tag}_packed'][0])


def test_gate_up_interleave_matches_reference(gl):
    """The fixtures are outputs of the reference's own _interleave_weights / _transpose_sf_for_utccp
    (deep_gemm/mega/__init__.py:97-128): the oracle's and the package's row maps must reproduce them bit for bit."""
    from deepgemm_b200 import mega
    t = torch.from_numpy(gl['interleave_in'].copy())
    for gran in (8, 16, 128):
        want = gl[f'interleave_g{gran}']
        assert np.array_equal(olay.interleave_gate_up(t, gran).numpy(), want)
        assert np.array_equal(mega._interleave_rows(t, gran).numpy(), want)
    assert np.array_equal(olay.interleave_gate_up(t[0], 8).numpy(), gl['interleave_2d_g8'])
    sf = torch.from_numpy(gl['utccp_in'].copy())
    assert np.array_equal(mega._sf_rows_to_cp_order(sf).numpy(), gl['utccp_out'])


def test_k_grouped_quantiser_and_product_match_reference(golden_dir):
    """per_channel_cast_to_fp8 bit for bit; the K-grouped product over the dequantised operands to FP32 rounding."""
    from oracle import gemm as ogemm
    g = np.load(os.path.join(golden_dir, 'kgrouped.npz'))
    ks = [int(k) for k in g['ks']]
    qs = {}
    for name in ('a', 'b'):
        x = _bf16(g[f'{name}_bf16'])
        q, sf = quant.quantize_fp8_per_channel(x, 128)
        assert np.array_equal(q.view(torch.uint8).numpy(), g[f'{name}_q'])
        assert np.array_equal(sf.numpy(), g[f'{name}_sf'])
        qs[name] = (q, sf)
    d = ogemm.k_grouped_gemm(qs['a'][0], qs['a'][1], qs['b'][0], qs['b'][1], torch.from_numpy(g['c'].copy()), ks)
    assert np.allclose(d.numpy(), g['d'], rtol=0, atol=1e-4)
    ends = np.cumsum(ks).tolist()  # K extents that are multiples of the alignment: the psum layout is the same split
    d2 = ogemm.k_grouped_gemm_psum(qs['a'][0], qs['a'][1], qs['b'][0], qs['b'][1], torch.from_numpy(g['c'].copy()), ends, 128)
    assert torch.equal(d2, d)
