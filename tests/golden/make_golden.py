"""Generates tests/golden/*.npz from the reference's own torch helpers.

Run once where the reference tree is available: ``python tests/golden/make_golden.py <path-to-the-DeepGEMM-tree>``
(or set ``DEEPGEMM_REFERENCE_ROOT``). The reference's ``deep_gemm/utils/math.py`` and ``deep_gemm/testing/numeric.py`` are
pure torch and are imported BY FILE PATH (``import deep_gemm`` itself needs the compiled ``_C`` module); the
functions run on seeded CPU inputs and their inputs/outputs are stored as small fixtures. The fixtures, not the
reference tree, travel with this repository: tests only read the ``.npz`` files.

What is pinned:
  quant.npz    per_token_cast_to_fp8 / per_token_cast_to_fp4 (gran 32 and 128, fp32 and packed scales),
               cast_back_from_fp8 / cast_back_from_fp4, ceil_to_ue8m0, pack/unpack, calc_diff
  layout.npz   the packed MN-major scale-factor layout as restated by the reference's own layout test
               (tests/test_layout.py:20-42) and the mega-MoE weight interleave (deep_gemm/mega/__init__.py:97-111)
  kgrouped.npz per_channel_cast_to_fp8 (the K-grouped GEMM's operand quantiser, one scale per 128 K rows and channel) and
               the K-grouped product d[g] = c[g] + a_g^T b_g over the dequantised operands, as the reference's generator
               forms it (tests/generators.py:413-453); written by ``make_golden.py <tree> --only kgrouped`` without
               touching the other two files
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_by_path(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def u8(t):
    return t.contiguous().view(torch.uint8).numpy()


def load_functions(path, names):
    """Executes only the named top-level functions of a Python source file (with torch in scope) and returns them."""
    import ast
    with open(path) as f:
        tree = ast.parse(f.read())
    picked = [node for node in tree.body if isinstance(node, ast.FunctionDef) and node.name in names]
    assert len(picked) == len(names), f'{path} no longer defines {names}'
    scope = {'torch': torch}
    exec(compile(ast.Module(body=picked, type_ignores=[]), path, 'exec'), scope)
    return {name: scope[name] for name in names}


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get('DEEPGEMM_REFERENCE_ROOT')
    if not ref_root:
        raise SystemExit('usage: make_golden.py <path-to-the-DeepGEMM-tree>')
    rmath = load_by_path('ref_math', os.path.join(ref_root, 'deep_gemm/utils/math.py'))
    rnum = load_by_path('ref_numeric', os.path.join(ref_root, 'deep_gemm/testing/numeric.py'))
    if '--only' in sys.argv and sys.argv[sys.argv.index('--only') + 1] == 'kgrouped':
        make_kgrouped(rmath)
        return

    out = {}
    torch.manual_seed(1234)
    # inputs: normal activations, small-magnitude weights, plus rows engineered to hit edge cases
    x = torch.randn(24, 384, dtype=torch.float32)
    x[0] = 0.0                                   # all-zero row: amax clamp at 1e-4
    x[1, :32] = 448.0 * 2.0 ** -3                # amax/448 exactly a power of two
    x[2, :32] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0] * 4) * 2.0 ** -5   # E2M1 thresholds
    x[3] = x[3] * 1e-6
    x[4] = x[4] * 1e4
    x[5, ::2] = -x[5, ::2].abs()
    x = x.bfloat16()
    w = (torch.randn(40, 256) * 0.02).bfloat16()
    w[0] = 0.0
    w[1, :32] = torch.tensor([0.25, -0.75, 1.25, -1.75, 2.5, -3.5, 5.0, -6.0] * 4).bfloat16() * 2.0 ** -6
    out['x_bf16'] = u8(x)
    out['w_bf16'] = u8(w)
    for gran in (32, 128):
        q, sf = rmath.per_token_cast_to_fp8(x, use_ue8m0=True, gran_k=gran)
        out[f'fp8_g{gran}_q'] = u8(q)
        out[f'fp8_g{gran}_sf'] = sf.numpy()
        q2, sfp = rmath.per_token_cast_to_fp8(x, use_ue8m0=True, gran_k=gran, use_packed_ue8m0=True)
        out[f'fp8_g{gran}_sf_packed'] = sfp.numpy()
        out[f'fp8_g{gran}_back'] = rmath.cast_back_from_fp8(q, sf, gran_k=gran).numpy()
        for name, t in (('x', x), ('w', w)):
            q, sf = rmath.per_token_cast_to_fp4(t, use_ue8m0=True, gran_k=gran)
            out[f'fp4_{name}_g{gran}_q'] = q.numpy()
            out[f'fp4_{name}_g{gran}_sf'] = sf.numpy()
            q2, sfp = rmath.per_token_cast_to_fp4(t, use_ue8m0=True, gran_k=gran, use_packed_ue8m0=True)
            out[f'fp4_{name}_g{gran}_sf_packed'] = sfp.numpy()
            out[f'fp4_{name}_g{gran}_back'] = rmath.cast_back_from_fp4(q, sf, gran_k=gran).numpy()
    probe = torch.tensor([0.0, 1e-10, 0.5, 0.50001, 1.0, 3.0, 4.0, 1e30, 3e38, -2.5], dtype=torch.float32)
    out['ue8m0_probe'] = probe.numpy()
    out['ue8m0_ceil'] = rmath.ceil_to_ue8m0(probe).numpy()
    a, b = torch.randn(64, 64), torch.randn(64, 64)
    out['diff_a'], out['diff_b'] = a.numpy(), b.numpy()
    out['diff_ab'] = np.float64(rnum.calc_diff(a, b))
    out['diff_aa'] = np.float64(rnum.calc_diff(a, a))
    out['diff_a_scaled'] = np.float64(rnum.calc_diff(a, a * 1.01 + 0.001 * b))
    np.savez_compressed(os.path.join(HERE, 'quant.npz'), **out)

    # layout fixtures: scales packed by the reference's pack_ue8m0_to_int (deep_gemm/utils/math.py:19-23), then laid
    # out as its packing kernel does (MN-major, MN stride = align(mn, 4), csrc/jit_kernels/impls/smxx_layout.hpp:183-186;
    # the reference's own layout test asserts exactly this image and these strides, tests/test_layout.py:20-60)
    lay = {}
    for tag, (g, mn, k, gran) in {'a': (1, 70, 1024, 128), 'b': (3, 132, 512, 32), 'c': (2, 64, 2304, 128)}.items():
        t = torch.randn(g * mn, k).bfloat16()
        _, sf = rmath.per_token_cast_to_fp8(t, use_ue8m0=True, gran_k=gran)
        sf_k = sf.shape[-1]
        padded_sf = torch.nn.functional.pad(sf, (0, (-sf_k) % 4), value=0.0)
        # a zero fp32 has exponent byte 0, which is what the kernel writes for K blocks beyond SF_K
        ints = rmath.pack_ue8m0_to_int(padded_sf).view(g, mn, -1)
        lay[f'{tag}_sf'] = sf.view(g, mn, sf_k).numpy()
        lay[f'{tag}_packed'] = ints.numpy()                      # logical [g, mn, packed_k]
        lay[f'{tag}_strides'] = np.array([ints.shape[2] * rmath.align(mn, 4), 1, rmath.align(mn, 4)], dtype=np.int64)
    # gate/up interleave and tcgen05.cp ("UTCCP") row order of the reference's weight transform: the two function
    # bodies are lifted out of deep_gemm/mega/__init__.py (:97-128) with ast and executed here, because importing that
    # module needs the compiled _C extension; what is stored is therefore the reference's own output
    mega_fns = load_functions(os.path.join(ref_root, 'deep_gemm', 'mega', '__init__.py'),
                              ('_interleave_weights', '_transpose_sf_for_utccp'))
    t = torch.arange(2 * 512 * 3, dtype=torch.int32).view(2, 512, 3)
    lay['interleave_in'] = t.numpy()
    for gran in (8, 16, 128):
        lay[f'interleave_g{gran}'] = mega_fns['_interleave_weights'](t, gran).numpy()
    lay['interleave_2d_g8'] = mega_fns['_interleave_weights'](t[0], 8).numpy()
    sf_in = torch.arange(2 * 384 * 5, dtype=torch.int32).view(2, 384, 5)
    lay['utccp_in'] = sf_in.numpy()
    lay['utccp_out'] = mega_fns['_transpose_sf_for_utccp'](sf_in).numpy()
    np.savez_compressed(os.path.join(HERE, 'layout.npz'), **lay)
    print('wrote quant.npz, layout.npz')
    make_kgrouped(rmath)


def make_kgrouped(rmath):
    torch.manual_seed(4321)
    ks = [256, 128, 384]
    m, n = 48, 40
    a = torch.randn(sum(ks), m).bfloat16()
    b = torch.randn(sum(ks), n).bfloat16()
    a[0:128, 0] = 0.0                       # an all-zero (K block, channel): amax clamp at 1e-4
    a[128:256, 1] = 448.0 * 2.0 ** -2       # amax / 448 exactly a power of two
    b[256:384] = b[256:384] * 1e-5
    out = {'ks': np.array(ks, dtype=np.int64), 'a_bf16': u8(a), 'b_bf16': u8(b)}
    (a_q, a_sf), (b_q, b_sf) = (rmath.per_channel_cast_to_fp8(t, use_ue8m0=True, gran_k=128) for t in (a, b))
    out.update({'a_q': u8(a_q), 'a_sf': a_sf.numpy(), 'b_q': u8(b_q), 'b_sf': b_sf.numpy()})
    c = torch.randn(len(ks), m, n) * 32
    d = c.clone()
    a_deq = a_q.float() * a_sf.repeat_interleave(128, dim=0)
    b_deq = b_q.float() * b_sf.repeat_interleave(128, dim=0)
    start = 0
    for g, k in enumerate(ks):
        d[g] = c[g] + a_deq[start:start + k].T @ b_deq[start:start + k]
        start += k
    out.update({'c': c.numpy(), 'd': d.numpy()})
    np.savez_compressed(os.path.join(HERE, 'kgrouped.npz'), **out)
    print('wrote kgrouped.npz')


if __name__ == '__main__':
    main()
