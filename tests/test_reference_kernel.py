"""The reference's own emitted kernel (its committed tf32x3 PTX for the 128^3 example, assembled for sm_100a by
oracle/build_ref.py) run on the same B200 as this build's kernels, on the same inputs: outputs must be identical
bit for bit, for every native GEMM variant, and hash to the output the reference published from its own GPU run."""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

from deuteron_b200 import ops
from oracle import ref_kernel, reference_math as R


def test_recipe_refuses_unexpected_ptx(tmp_path):
    from oracle import build_ref
    fake = tmp_path / 'docs' / 'video' / 'demo' / 'capture'
    fake.mkdir(parents=True)
    (fake / 'kernel.ptx').write_text('.version 8.7\n.target sm_120\n.visible .entry other_kernel()\n{\n ret;\n}\n')
    with pytest.raises(RuntimeError, match='not the PTX'):
        build_ref.build(tmp_path, tmp_path / 'out.cubin')
    (fake / 'kernel.ptx').write_text('.version 8.7\n.target sm_120\n.visible .entry matmul_tiled_128(\n)\n{\n$L: bra $L;\n}\n')
    with pytest.raises(RuntimeError, match='branches'):
        build_ref.build(tmp_path, tmp_path / 'out.cubin')
    assert build_ref.build(tmp_path / 'absent', tmp_path / 'out.cubin') is None and not (tmp_path / 'out.cubin').exists()


@pytest.mark.gpu
def test_reference_emitted_kernel_and_native_kernels_agree_bit_for_bit(cuda, published):
    if not ref_kernel.available():
        pytest.skip('oracle/_ref cubin was not built (the reference tree was absent at build time)')
    reference = ref_kernel.ReferenceMatmul()
    stream = cuda.cuda.current_stream().cuda_stream
    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
    try:
        for name, make in (('normal', R.seeded_normal), ('uniform', R.seeded_uniform)):
            left, right = make(7, (128, 128)), make(11, (128, 128))
            d_left, d_right = cuda.from_numpy(left).to('cuda:0'), cuda.from_numpy(right).to('cuda:0')
            result = cuda.full((128, 128), float('nan'), device='cuda:0')
            reference.launch(d_right.data_ptr(), d_left.data_ptr(), result.data_ptr(), stream)   # arg_order: right, left, result
            cuda.cuda.synchronize()
            expected = result.cpu().numpy()
            np.testing.assert_allclose(expected, R.gemm_f64(left, right), rtol=1e-3, atol=1e-3)
            if name == 'normal':   # the reference's example inputs: its published GPU output hash
                assert sha(expected) == published['results']['tensor_tf32x3']['output_sha256']['result']
            for variant in (0, 1, 2, 3, 4, 5):
                ops.set_gemm_variant(variant)
                mine = ops.gemm(d_left, d_right, 'tf32x3').cpu().numpy()
                assert np.array_equal(mine.view(np.uint32), expected.view(np.uint32)), (name, variant)
    finally:
        ops.set_gemm_variant(0)
        reference.close()
