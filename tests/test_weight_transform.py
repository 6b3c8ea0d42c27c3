"""CPU tests of the weight transform of the layer (plain tensor code, no GPU): gate/up interleave by 128 and the
tcgen05.cp row order of packed scale factors. The reference pre-permutes its scale factors the same way for its own
kernel (deep_gemm/include/deep_gemm/impls/sm100_fp8_fp4_mega_moe.cuh:136-140: dst = (r & ~127) + (r & 31) * 4 +
((r >> 5) & 3)); the interleave granularity differs (8 there, 128 here) because the epilogues differ."""
import torch

from deepgemm_b200 import mega


def test_sf_rows_follow_the_tcgen05_cp_order():
    g, n, kp = 2, 384, 5
    sf = torch.arange(g * n * kp, dtype=torch.int32).view(g, kp, n).transpose(1, 2)  # MN-major like the packed layout
    out = mega._sf_rows_to_cp_order(sf)
    assert out.stride() == sf.stride()
    for r in (0, 1, 31, 32, 33, 127, 128, 200, 383):
        dst = (r & ~127) + (r & 31) * 4 + ((r >> 5) & 3)
        assert torch.equal(out[:, dst, :], sf[:, r, :])
    # a permutation inside every group of 128 rows
    assert torch.equal(torch.sort(out[0, :128, 0]).values, torch.sort(sf[0, :128, 0]).values)


def test_gate_up_interleave_by_128():
    inter = 256
    w = torch.arange(2 * inter, dtype=torch.int32).view(1, 2 * inter, 1).repeat(1, 1, 3)  # row index as content
    out = mega._interleave_rows(w, 128)
    rows = out[0, :, 0].tolist()
    assert rows[:128] == list(range(0, 128))                    # gate 0..127
    assert rows[128:256] == list(range(inter, inter + 128))     # up 0..127
    assert rows[256:384] == list(range(128, 256))               # gate 128..255
    assert rows[384:512] == list(range(inter + 128, inter + 256))


def test_transform_keeps_shapes_and_handles_shared_2d_weights():
    e, inter, hidden = 2, 128, 256
    l1 = (torch.zeros((e, 2 * inter, hidden // 2), dtype=torch.int8),
          torch.zeros((e, hidden // 128, 2 * inter), dtype=torch.int32).transpose(1, 2))
    l2 = (torch.zeros((e, hidden, inter // 2), dtype=torch.int8),
          torch.zeros((e, inter // 128, hidden), dtype=torch.int32).transpose(1, 2))
    t1, t2 = mega.transform_weights_for_mega_moe(l1, l2)
    assert t1[0].shape == l1[0].shape and t1[1].stride() == l1[1].stride() and t2[1].stride() == l2[1].stride()
    s1 = (torch.zeros((2 * inter, hidden), dtype=torch.float8_e4m3fn), torch.zeros((hidden // 128, 2 * inter), dtype=torch.int32).t())
    s2 = (torch.zeros((hidden, inter), dtype=torch.float8_e4m3fn), torch.zeros((inter // 128, hidden), dtype=torch.int32).t())
    u1, u2 = mega.transform_weights_for_mega_moe(s1, s2)
    assert u1[0].shape == s1[0].shape and u1[1].shape == s1[1].shape and u2[0].dtype == torch.float8_e4m3fn


def test_bf16_weights_only_get_the_gate_up_interleave():
    """bfloat16 layer weights (bare tensors, 3-D per expert or 2-D for shared experts): L1 rows interleaved by 128,
    L2 untouched (reference: transform_weights_for_mega_moe on bare tensors, deep_gemm/mega/__init__.py:131-149)."""
    import pytest
    e, inter, hidden = 3, 256, 64
    w1 = torch.arange(e * 2 * inter, dtype=torch.float32).view(e, 2 * inter, 1).repeat(1, 1, hidden).bfloat16()
    w2 = torch.randn(e, hidden, inter).bfloat16()
    t1, t2 = mega.transform_weights_for_mega_moe(w1, w2)
    assert t1.is_contiguous() and t1.shape == w1.shape and t2 is w2
    assert torch.equal(t1, mega._interleave_rows(w1, 128))
    assert torch.equal(t1[:, 128:256], w1[:, inter:inter + 128]) and torch.equal(t1[:, 256:384], w1[:, 128:256])
    s1, s2 = mega.transform_weights_for_mega_moe(w1[0], w2[0])
    assert torch.equal(s1, t1[0]) and s2.shape == w2[0].shape
    with pytest.raises(RuntimeError):
        mega.transform_weights_for_mega_moe(w1.float(), w2)
