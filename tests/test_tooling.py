"""The compile cache on disk, the command line and the problem-directory driver (the reference's
tests/test_cache.py, tests/test_cli.py and the conventions of benchmark.py:290-308, 497-557)."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from deuteron_b200 import benchmark, build, cache, cli, compile_kernel, schedules

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture()
def problem(tmp_path):
    graph, meta = schedules.rms_norm_example(8, 512)
    schedules.write_problem(tmp_path / 'f01_rmsnorm', graph, meta)
    return tmp_path / 'f01_rmsnorm'


def test_disk_cache_round_trip_and_rejection_of_damaged_records(tmp_path, monkeypatch):
    root = tmp_path / 'cache'
    monkeypatch.setenv('DEUTERON_CACHE', str(root))
    graph, meta = schedules.row_softmax_example()
    build.clear_cache()
    first = compile_kernel(graph, meta)
    records = list(root.glob('*.json'))
    assert len(records) == 1 and len(records[0].stem) == 64
    build.clear_cache()
    again = compile_kernel(graph, meta)             # served from disk: same plan, same text, same launch
    assert again.plan == first.plan and again.ptx == first.ptx and again.launch == first.launch
    assert isinstance(again.plan.buffers['x'], tuple)
    key = records[0].stem
    stored = json.loads(records[0].read_text())
    # a record whose content was altered, whose key disagrees, or which is not JSON is ignored, never trusted
    for damage in (lambda d: d['params'].update(cols=999), lambda d: d.update(key='0' * 64), lambda d: d.update(version=2),
                   lambda d: d.pop('launch')):
        altered = json.loads(json.dumps(stored))
        damage(altered)
        records[0].write_text(json.dumps(altered))
        assert cache.read(str(root), key) is None
    records[0].write_text('{not json')
    assert cache.read(str(root), key) is None
    build.clear_cache()
    assert compile_kernel(graph, meta).plan == first.plan     # recompiled and rewritten
    assert cache.read(str(root), key) is not None
    assert cache.read(str(root), '../' + key) is None and cache.read(None, key) is None
    assert not list(root.glob('*.tmp'))
    # an unwritable cache directory is not an error
    monkeypatch.setenv('DEUTERON_CACHE', str(records[0] / 'below-a-file'))
    build.clear_cache()
    assert compile_kernel(graph, meta).plan == first.plan


def test_command_line_prints_the_selection_and_protects_inputs(problem, capsys, tmp_path):
    kernel = problem / 'k_rms_norm.ir.json'
    assert cli.main([str(kernel)]) == 0
    text = capsys.readouterr().out
    assert 'row_fused(' in text and 'target sm_100a' in text
    dump = tmp_path / 'selection.ll'
    assert cli.main([str(kernel), '--dump-llvm', str(dump), '--contraction-precision', 'tf32x3', '--no-approximate-math']) == 0
    assert dump.read_text() == capsys.readouterr().out
    before = (problem / 'meta.json').read_bytes()
    assert cli.main([str(kernel), '--dump-llvm', str(problem / 'meta.json')]) == 1
    assert 'would overwrite an input file' in capsys.readouterr().err and (problem / 'meta.json').read_bytes() == before
    assert cli.main([str(kernel), '--dump-llvm', str(dump), '--dump-unoptimized', str(dump)]) == 1
    assert cli.main([str(kernel), '--dump-llvm', str(tmp_path / 'missing' / 'x.ll')]) == 1
    assert cli.main([str(kernel), '--arch', 'sm_89']) == 1
    assert 'sm_100a' in capsys.readouterr().err
    assert cli.main([str(problem / 'absent.ir.json')]) == 1
    with pytest.raises(SystemExit):
        cli.main([str(kernel), '--opt-level', '7'])
    done = subprocess.run([sys.executable, '-m', 'deuteron_b200', str(kernel)], capture_output=True, text=True, cwd=ROOT)
    assert done.returncode == 0 and 'row_fused(' in done.stdout


def test_driver_refuses_bad_arguments_and_reused_artifact_directories(problem, tmp_path, capsys):
    artifacts = tmp_path / 'out'
    artifacts.mkdir()
    benchmark.reserve_artifacts(artifacts)
    with pytest.raises(ValueError, match='already reserved'):
        benchmark.reserve_artifacts(artifacts)
    benchmark.write_json(artifacts / 'manifest.json', {'a': 1})
    assert json.loads((artifacts / 'manifest.json').read_text()) == {'a': 1} and not list(artifacts.glob('*.tmp'))
    with pytest.raises(ValueError, match='new artifacts directory'):
        benchmark.reserve_artifacts(artifacts)
    for argv in (['--problems-dir', str(tmp_path / 'nowhere')], ['--problems-dir', str(problem.parent), 'zzz'],
                 ['--problems-dir', str(problem.parent), '--devices', '0,0'], ['--problems-dir', str(problem.parent), '--iters', '0'],
                 ['--problems-dir', str(problem.parent), '--artifacts', str(artifacts)]):
        with pytest.raises(SystemExit):
            benchmark.main(argv)
    capsys.readouterr()


def test_generated_problem_set_has_the_published_launches():
    workloads = schedules.open_workloads()
    assert len(workloads) == 15
    launch = workloads['f01_rmsnorm'][1]['kernels'][0]
    assert launch['arg_order'] == ['mean_count', 'add_c1', 'x', 'w', 'mul_1'] and launch['grid'] == [64, 1, 1] and launch['block'] == [128, 1, 1]
    launch = workloads['m02_matmul_rect'][1]['kernels'][0]
    assert launch['arg_order'] == ['x1', 'x0', 'matmul'] and launch['grid'] == [512, 1, 1] and launch['zero_outputs'] == ['matmul']
    launch = workloads['r03_mean'][1]['kernels'][0]
    assert launch['arg_order'] == ['x', 'mean_keepdim_count', 'mean'] and launch['grid'] == [1, 1, 1]
    assert workloads['p02_scale_shift'][1]['kernels'][0]['grid'] == [4, 1, 1]
    assert workloads['m01_matmul_512'][1]['kernels'][0]['grid'] == [128, 1, 1]


@pytest.mark.gpu
def test_driver_runs_the_generated_problem_set(tmp_path, cuda):
    from deuteron_b200 import argument_array
    from oracle import reference_math as R
    inputs = lambda meta: {a['name']: argument_array(a) for a in meta['kernels'][0]['args'] if not a.get('output')}
    expected = {
        'p00_scalar_add': lambda v: {'sum': v['lhs'] + v['rhs']}, 'p01_vector_add': lambda v: {'sum': v['lhs'] + v['rhs']},
        'p02_scale_shift': lambda v: {'add': v['x'] * np.float32(2) + np.float32(1)},
        'p03_relu_mul': lambda v: {'mul': np.maximum(v['x'], np.float32(0)) * v['y']},
        'r01_array_sum': lambda v: {'out': R.row_sum_f64(v['x'])}, 'r02_big_sum': lambda v: {'out': R.row_sum_f64(v['x'])},
        'r03_mean': lambda v: {'mean': R.row_mean_f64(v['x'][None, :])}, 'r04_row_sum': lambda v: {'out': R.row_sum_f64(v['x'])},
        'm01_matmul_512': lambda v: {'result': R.gemm_f64(v['left'], v['right'])},
        'm02_matmul_rect': lambda v: {'matmul': R.gemm_f64(v['x0'], v['x1'])},
        'f01_rmsnorm': lambda v: {'mul_1': R.rms_norm_f64(v['x'], v['w'], 1024.0, 1e-5)},
        'f02_row_softmax': lambda v: {'softmax': R.row_softmax_f64(v['x'])}, 'f03_l2norm': lambda v: {'div': R.l2_norm_f64(v['x'])},
        'a01_attention': lambda v: {'out': R.attention_f64(v['q'], v['kt'], v['v'], np.float32(1 / np.sqrt(64)))},
        'a02_attention_128': lambda v: {'out': R.attention_f64(v['q'], v['kt'], v['v'], np.float32(1 / np.sqrt(32)))},
    }
    problems = tmp_path / 'problems'
    for name, (graph, meta) in schedules.open_workloads().items():
        schedules.write_problem(problems / name, graph, meta)
        np.savez(problems / name / 'expected.npz', **expected[name](inputs(meta)))
    artifacts = tmp_path / 'artifacts'
    assert benchmark.main(['--problems-dir', str(problems), '--artifacts', str(artifacts), '--warmup', '2', '--iters', '20', '--samples', '3']) == 0
    results = json.loads((artifacts / 'results.json').read_text())
    assert len(results) == 15 and all(r['passed'] for r in results)
    one = json.loads((artifacts / 'f02_row_softmax' / 'result.json').read_text())
    assert one['kernels'][0]['entry'] == 'k_softmax' and one['kernels'][0]['median_us'] > 0 and one['max_abs_error']['softmax'] < 1e-6
    assert (artifacts / 'f02_row_softmax' / 'actual.npz').exists() and (artifacts / 'manifest.json').exists()
    # a second run into the same directory is refused
    with pytest.raises(SystemExit):
        benchmark.main(['--problems-dir', str(problems), '--artifacts', str(artifacts)])


@pytest.mark.gpu
def test_driver_chains_kernels_through_intermediate_buffers(tmp_path, cuda):
    """Two kernels in one problem: y = 2x + 1, then mean(y); the second reads the first's output as an `intermediate`
    buffer (benchmark.py:57-62, 466-470)."""
    first_graph, first_meta = schedules.pointwise_example('affine', 4096)
    second_graph, second_meta = schedules.mean_example(4096)
    second_text = json.dumps(second_graph).replace("input='x'", "input='add'").replace('"x"', '"add"')
    second_launch = json.loads(json.dumps(second_meta['kernels'][0]).replace('"x"', '"add"'))
    for arg in second_launch['args']:
        if arg['name'] == 'add':
            arg.pop('seed')
            arg['intermediate'] = True
    first_launch = dict(first_meta['kernels'][0], final=False)
    meta = {'id': 'chained', 'rtol': 1e-5, 'atol': 1e-6, 'graph_inputs': ['x'], 'graph_outputs': ['mean'],
            'kernels': [first_launch, second_launch]}
    problem = tmp_path / 'problems' / 'c00_chained'
    problem.mkdir(parents=True)
    (problem / 'meta.json').write_text(json.dumps(meta))
    (problem / (first_launch['entry'] + '.ir.json')).write_text(json.dumps(first_graph))
    (problem / (second_launch['entry'] + '.ir.json')).write_text(second_text)
    x = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    y = x * np.float32(2) + np.float32(1)
    np.savez(problem / 'expected.npz', mean=np.array([y.astype(np.float64).mean()]))
    artifacts = tmp_path / 'artifacts'
    assert benchmark.main(['--problems-dir', str(problem.parent), '--artifacts', str(artifacts), '--warmup', '1', '--iters', '5', '--samples', '2']) == 0
    report = json.loads((artifacts / 'c00_chained' / 'result.json').read_text())
    assert report['passed'] and [k['entry'] for k in report['kernels']] == ['k_add_pointwise', 'k_mean']
    with np.load(artifacts / 'c00_chained' / 'actual.npz') as actual:
        np.testing.assert_array_equal(actual['add'], y)


def test_command_line_dump_protection_by_every_name_and_all_or_nothing_writes(problem, tmp_path, capsys, monkeypatch):
    """The negative cases of the reference's tests/test_cli.py, restated: aliases of the inputs, dumps aliasing each
    other, bad destinations, a failure while staging, a failed rename, a failed compilation, an interrupt."""
    kernel, meta = problem / 'k_rms_norm.ir.json', problem / 'meta.json'
    original = {path: path.read_bytes() for path in (kernel, meta)}
    symlink, hardlink = tmp_path / 'symbolic.ll', tmp_path / 'hard.ll'
    symlink.symlink_to(kernel)
    os.link(meta, hardlink)
    for alias in (kernel, meta, symlink, hardlink):
        for flag in ('--dump-llvm', '--dump-unoptimized'):
            assert cli.main([str(kernel), flag, str(alias)]) == 1
            captured = capsys.readouterr()
            assert captured.out == '' and 'overwrite an input' in captured.err
    assert all(path.read_bytes() == content for path, content in original.items())
    first = tmp_path / 'first.ll'
    first.write_text('old contents')
    other_name = tmp_path / 'alias.ll'
    os.link(first, other_name)
    for second in (first, first.parent / '.' / first.name, other_name):
        assert cli.main([str(kernel), '--dump-llvm', str(first), '--dump-unoptimized', str(second)]) == 1
        captured = capsys.readouterr()
        assert captured.out == '' and 'different files' in captured.err and first.read_text() == 'old contents'
    fresh = tmp_path / 'fresh.ll'
    assert cli.main([str(kernel), '--dump-llvm', str(fresh), '--dump-unoptimized', str(tmp_path / 'sub' / '..' / 'fresh.ll')]) == 1
    assert not fresh.exists()
    for invalid in (tmp_path, tmp_path / 'absent' / 'dump.ll'):
        assert cli.main([str(kernel), '--dump-llvm', str(first), '--dump-unoptimized', str(invalid)]) == 1
        assert capsys.readouterr().err and first.read_text() == 'old contents'
    # a failure while the second dump is staged leaves both old files and no staging file
    second = tmp_path / 'second.ll'
    second.write_text('old second')
    before = set(tmp_path.iterdir())
    factory, calls = cli.tempfile.NamedTemporaryFile, []

    def fail_second_stage(*args, **kwargs):
        calls.append(1)
        if len(calls) == 2:
            raise PermissionError(13, 'write denied', str(second))
        return factory(*args, **kwargs)

    monkeypatch.setattr(cli.tempfile, 'NamedTemporaryFile', fail_second_stage)
    assert cli.main([str(kernel), '--dump-llvm', str(first), '--dump-unoptimized', str(second)]) == 1
    monkeypatch.setattr(cli.tempfile, 'NamedTemporaryFile', factory)
    captured = capsys.readouterr()
    assert captured.out == '' and 'write denied' in captured.err
    assert first.read_text() == 'old contents' and second.read_text() == 'old second' and set(tmp_path.iterdir()) == before
    # a rename that fails keeps the old file and removes the staging file
    with monkeypatch.context() as patched:
        def no_space(self, target):
            raise OSError(28, 'No space left')
        patched.setattr(Path, 'replace', no_space)
        assert cli.main([str(kernel), '--dump-llvm', str(first)]) == 1
    assert 'No space left' in capsys.readouterr().err and first.read_text() == 'old contents' and set(tmp_path.iterdir()) == before
    # a failed compilation touches no dump; an interrupt is status 130
    with monkeypatch.context() as patched:
        def invalid(*args, **kwargs):
            raise ValueError('invalid scheduled IR')
        patched.setattr(cli, 'compile_kernel', invalid)
        assert cli.main([str(kernel), '--dump-llvm', str(first)]) == 1
        assert 'invalid scheduled IR' in capsys.readouterr().err and first.read_text() == 'old contents'

        def interrupt(*args, **kwargs):
            raise KeyboardInterrupt
        patched.setattr(cli, 'compile_kernel', interrupt)
        assert cli.main([str(kernel)]) == 130
        captured = capsys.readouterr()
        assert captured.out == '' and 'interrupted' in captured.err
    # diagnostics printed during compilation go to stderr; every option of Options has its flag
    with monkeypatch.context() as patched:
        real = cli.compile_kernel

        def noisy(*args, **kwargs):
            print('compiler diagnostic')
            return real(*args, **kwargs)
        patched.setattr(cli, 'compile_kernel', noisy)
        assert cli.main([str(kernel)]) == 0
        captured = capsys.readouterr()
        assert captured.err == 'compiler diagnostic\n' and 'row_fused(' in captured.out
    import dataclasses
    from deuteron_b200 import Options
    helped = cli.build_parser().format_help()
    assert all('--' + field.name.replace('_', '-') in helped for field in dataclasses.fields(Options))
    seen = {}

    def record(path, **kwargs):
        seen.update(kwargs, path=path)
        return compile_kernel(path)
    monkeypatch.setattr(cli, 'compile_kernel', record)
    argv = [str(kernel), '--opt-level', '1', '--unroll', '8', '--vector-width', '16', '--contraction-precision', 'f32']
    argv += ['--no-' + f.name.replace('_', '-') for f in dataclasses.fields(Options) if isinstance(f.default, bool)]
    assert cli.main(argv) == 0
    expected = Options(unroll=8, vector_width=16, contraction_precision='f32',
                       **{f.name: False for f in dataclasses.fields(Options) if isinstance(f.default, bool)})
    assert seen['options'] == expected and seen['opt_level'] == 1 and seen['arch'] == 'sm_100a'


def test_command_line_survives_a_closed_or_full_stdout(problem):
    kernel = problem / 'k_rms_norm.ir.json'
    with subprocess.Popen([sys.executable, '-m', 'deuteron_b200', str(kernel)], cwd=ROOT, stdout=subprocess.PIPE,
                          stderr=subprocess.PIPE, text=True) as process:
        process.stdout.close()
        stderr = process.stderr.read()
        code = process.wait(timeout=120)
    assert code == 1 and 'Broken pipe' in stderr and 'Traceback' not in stderr and 'Exception ignored' not in stderr
    if Path('/dev/full').exists():
        with open('/dev/full', 'wb') as stream:
            done = subprocess.run([sys.executable, '-m', 'deuteron_b200', str(kernel)], cwd=ROOT, stdout=stream,
                                  stderr=subprocess.PIPE, text=True, timeout=120)
        assert done.returncode == 1 and 'No space left' in done.stderr and 'Traceback' not in done.stderr
        assert 'Exception ignored' not in done.stderr
