"""The reference's own kernels run on the same B200 as this build's kernels, on the same inputs.

Two sets, both built by oracle/build_ref.py where the reference checkout is present:
  * the PTX file the reference committed itself (tf32x3, 128^3): outputs identical bit for bit for every native GEMM
    variant, and hashing to the output the reference published from its own GPU run;
  * the kernels the unmodified reference compiler emits for sm_100 (GEMM in three modes up to 8192^3, its attention
    and f16 examples, vector add, the memory-bound kernels at benchmark size, the fifteen open workloads): each is
    launched through the driver API exactly as the reference's runner launches it, and the same IR and meta are handed
    to this build's compile_kernel + LocalRunner. Bars: bit-exact for vector add and the f16 kernels; elsewhere this
    build's maximum error against float64 is at most twice the reference kernel's own on this GPU."""
import hashlib
import json
import math
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
        build_ref.build_committed_ptx(tmp_path, tmp_path / 'out.cubin')
    (fake / 'kernel.ptx').write_text('.version 8.7\n.target sm_120\n.visible .entry matmul_tiled_128(\n)\n{\n$L: bra $L;\n}\n')
    with pytest.raises(RuntimeError, match='branches'):
        build_ref.build_committed_ptx(tmp_path, tmp_path / 'out.cubin')
    assert build_ref.build_committed_ptx(tmp_path / 'absent', tmp_path / 'out.cubin') is None and not (tmp_path / 'out.cubin').exists()
    assert build_ref.reference_root(tmp_path / 'absent') in (None, build_ref.reference_root())   # no checkout there


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


# ------------------------------------------------------------------------------------------------
# kernels emitted by the unmodified reference compiler for sm_100
# ------------------------------------------------------------------------------------------------

COMPILED = sorted(ref_kernel.manifest())
BIT_EXACT = ('vector_add', 'f16_', 'open_p00', 'open_p01')


def _exact_outputs(cuda, name, launch, device):
    """float64 expectation of every output of a case, computed on the GPU in float64 from the same inputs (a subset of
    rows for the largest products). Returns {output: (expected tensor, row selector or None)}."""
    t = {key: value.double() for key, value in device.items()}
    if name.startswith(('gemm_', 'open_m01')):
        left, right, out = ('left', 'right', 'result')
        rows = cuda.arange(0, t[left].shape[0], max(1, t[left].shape[0] // 64), device='cuda:0') if t[left].shape[0] > 2048 else None
        product = (t[left][rows] if rows is not None else t[left]) @ t[right]
        return {out: (product, rows)}
    if name == 'open_m02_matmul_rect':
        return {'matmul': (t['x0'] @ t['x1'], None)}
    if name.startswith(('attention_', 'open_a0')):
        scale = float(np.float32(1 / math.sqrt(t['q'].shape[1])))
        return {'out': (cuda.softmax(t['q'] @ t['kt'] * scale, dim=1) @ t['v'], None)}
    if name.startswith(('row_sum', 'open_r01', 'open_r02', 'open_r04')):
        x = t['x'] if t['x'].dim() == 2 else t['x'][None, :]
        return {launch['arg_order'][-1]: (x.sum(dim=1), None)}
    if name.startswith('row_max'):
        return {launch['arg_order'][-1]: (t['x'].max(dim=1).values, None)}
    if name == 'open_r03_mean':
        return {'mean': (t['x'].mean()[None], None)}
    if name == 'open_p02_scale_shift':
        return {'add': (t['x'] * 2 + 1, None)}
    if name == 'open_p03_relu_mul':
        return {'mul': (t['x'].clamp(min=0) * t['y'], None)}
    if name == 'open_f01_rmsnorm':
        x = t['x']
        return {'mul_1': (x * cuda.rsqrt((x * x).mean(dim=1, keepdim=True) + 1e-5) * t['w'], None)}
    if name == 'open_f02_row_softmax':
        return {'softmax': (cuda.softmax(t['x'], dim=1), None)}
    if name == 'open_f03_l2norm':
        x = t['x']
        return {'div': (x * cuda.rsqrt((x * x).sum(dim=1, keepdim=True)), None)}
    raise AssertionError(f'no expectation for {name}')


@pytest.mark.gpu
@pytest.mark.parametrize('name', COMPILED)
def test_every_reference_emitted_kernel_beside_the_native_one(cuda, name):
    from deuteron_b200 import LocalRunner, Options, argument_array, compile_kernel
    case = json.loads((ref_kernel.ROOT / f'{name}.case.json').read_text())
    launch = case['meta']['kernels'][0]
    host = {arg['name']: argument_array(arg) for arg in launch['args']}
    device = {key: cuda.from_numpy(value).to('cuda:0') for key, value in host.items()}
    outputs = [arg['name'] for arg in launch['args'] if arg.get('output')]
    for key in outputs:
        device[key].fill_(float('nan')) if key not in launch.get('zero_outputs', []) else device[key].zero_()
    with ref_kernel.ReferenceKernel(name) as reference:
        reference.launch({key: value.data_ptr() for key, value in device.items()}, cuda.cuda.current_stream().cuda_stream)
        cuda.cuda.synchronize()
    theirs = {key: device[key].clone() for key in outputs}
    compiled = compile_kernel(case['graph'], case['meta'], arch='sm_100a', opt_level=3, options=Options(**case['options']))
    with LocalRunner(0) as runner:
        mine = runner.run_kernel(launch, compiled, warmup=0, iters=1, samples=1)['outputs']
    ops.check_device_status()
    if name.startswith(BIT_EXACT):
        for key in outputs:
            ours, ref = mine[key], theirs[key].cpu().numpy()
            if ours.dtype == np.float16:
                finite = ~np.isnan(ref)
                assert np.array_equal(ours.view(np.uint16)[finite], ref.view(np.uint16)[finite]) and np.array_equal(np.isnan(ours), np.isnan(ref))
            else:
                assert np.array_equal(ours.view(np.uint32), ref.view(np.uint32))
        return
    inputs = {key: value for key, value in device.items() if key not in outputs}
    for key, (expected, rows) in _exact_outputs(cuda, name, launch, inputs).items():
        ours = cuda.from_numpy(mine[key]).to('cuda:0').double().reshape(-1, *expected.shape[1:]) if expected.dim() > 1 else cuda.from_numpy(mine[key]).to('cuda:0').double().reshape(-1)
        ref = theirs[key].double().reshape(ours.shape)
        if rows is not None:
            ours, ref = ours[rows], ref[rows]
        scale = float(expected.abs().max().item())
        if name.startswith(('row_sum', 'open_r0')):
            # A sum's rounding error is proportional to the sum of the magnitudes, not to the sum: 65 536 values of
            # either sign cancel to a few hundred, and two correct summation orders then differ by more than an ulp
            # of the result.
            x = inputs['x'].double()
            magnitudes = (x if x.dim() == 2 else x[None, :]).abs().sum(dim=1).max()
            scale = max(scale, float((magnitudes / x.numel() if name == 'open_r03_mean' else magnitudes).item()))
        error_mine = float((ours - expected.reshape(ours.shape)).abs().max().item()) / scale
        error_ref = float((ref - expected.reshape(ref.shape)).abs().max().item()) / scale
        assert error_ref < 1e-3, (name, key, error_ref)     # the reference kernel itself ran correctly here
        # twice the reference kernel's own error; below four units in the last place of the largest output the two
        # are rounding noise of different summation orders and the comparison means nothing
        assert error_mine <= max(2 * error_ref, 2.0 ** -22), (name, key, error_mine, error_ref)
