"""The fused expert-MLP kernel (both GEMMs of the FP8 x MXFP4 layer in one persistent launch: CTA pairs with
tcgen05 cta_group::2, or single CTAs) against the same oracle cases as the default kernels.

Which kernels serve the layer is fixed per process (the weights' gate/up interleave and tile order depend on it:
dgb200_get_gate_up_interleave_for_mega_moe), so each variant runs the layer's parity tests in a process of its own with
DGB200_MLP_KERNEL set: 2 = CTA pairs, 1 = single CTAs. The cases include hidden sizes that only the single-CTA form can
take (not a multiple of 256), experts of more than one token tile, empty experts, masked slots, the clamp, buffer
reuse, the full-size configuration and the peer-timeout path."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize('variant', ['2', '1'])
def test_layer_parity_with_the_fused_kernel(variant):
    if not torch.cuda.is_available():
        pytest.skip('needs a GPU')
    env = dict(os.environ, DGB200_MLP_KERNEL=variant)
    proc = subprocess.run([sys.executable, '-m', 'pytest', os.path.join(ROOT, 'tests', 'test_moe_gpu.py'), '-x', '-q', '-p', 'no:cacheprovider'],
                          cwd=ROOT, env=env, capture_output=True, text=True, timeout=1200)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-2000:]
    probe = subprocess.run([sys.executable, '-c', 'from deepgemm_b200 import _lib; print(_lib.lib().dgb200_get_gate_up_interleave_for_mega_moe())'],
                           cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert probe.stdout.strip() == '16', 'the fused kernel was not selected: ' + probe.stdout + probe.stderr
