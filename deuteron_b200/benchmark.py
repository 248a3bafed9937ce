"""Driver over problem directories, with the conventions and result schema of the reference's
benchmark.py (benchmark.py:434-557): every problem directory holds `meta.json`, one `<entry>.ir.json`
per kernel of the meta, and `expected.npz`; kernels of one problem run in order and hand their outputs
on as `intermediate` buffers; each problem gets `<artifacts>/<problem>/result.json`, `actual.npz` and
the compile output per entry, and the run leaves `manifest.json` and `results.json`.

    python -m deuteron_b200.benchmark --problems-dir DIR [problem ...] [--devices 0,1] [--artifacts OUT]

Differences from the reference: kernels run on the native sm_100a library (no remote runner, no PTX
assembly), and `--arch` defaults to sm_100a.
"""
from __future__ import annotations

import argparse
import dataclasses
import hashlib
import json
import multiprocessing
import os
import sys
import tempfile
import time
from concurrent.futures import ProcessPoolExecutor
from pathlib import Path
from typing import Any

import numpy as np

from .build import compile_kernel, compile_many
from .native import CudaError
from .options import Options
from .runner import LocalRunner, compare_outputs


def write_json(path: Any, value: Any) -> None:
    """Atomic JSON write (temporary file beside the destination, then replace)."""
    path = Path(path)
    temporary = None
    try:
        with tempfile.NamedTemporaryFile(mode='w', encoding='utf-8', dir=path.parent, prefix=path.name + '.', suffix='.tmp',
                                         delete=False) as stream:
            temporary = Path(stream.name)
            stream.write(json.dumps(value, indent=2) + '\n')
        temporary.replace(path)
    finally:
        if temporary is not None:
            temporary.unlink(missing_ok=True)


def reserve_artifacts(path: Path) -> None:
    """One run per artifacts directory: earlier measurements are never overwritten (benchmark.py:301-308)."""
    if (path / 'manifest.json').exists():
        raise ValueError(f'use a new artifacts directory to preserve previous measurements: {path}')
    try:
        with (path / '.deuteron-run').open('x') as stream:
            stream.write(json.dumps({'pid': os.getpid(), 'started': time.time()}) + '\n')
    except FileExistsError as exc:
        raise ValueError(f'artifacts directory is already reserved by another run: {path}') from exc


def run_partition(device: int, problems: list[str], settings: dict) -> list[dict]:
    """All `problems` on one device, in this process (benchmark.py:434-495)."""
    overrides = {k: settings[k] for k in ('contraction_precision', 'approximate_math') if settings.get(k) is not None}
    options = dataclasses.replace(Options(), **overrides)
    arch = settings.get('arch') or 'sm_100a'
    reports = []
    runner = LocalRunner(device)
    try:
        batched: dict = {}
        batch_seconds = 0.0
        if settings.get('jobs', 1) > 1:
            order = [(Path(problem), launch['entry']) for problem in problems
                     for launch in json.loads((Path(problem) / 'meta.json').read_text())['kernels']]
            started = time.perf_counter()
            results = compile_many([(problem / (entry + '.ir.json'), arch, settings['opt_level'], options) for problem, entry in order],
                                   settings['jobs'])
            batch_seconds = (time.perf_counter() - started) / max(len(results), 1)
            batched = dict(zip(order, results))
        for problem in map(Path, problems):
            destination = Path(settings['artifacts']) / problem.name
            destination.mkdir(parents=True, exist_ok=True)
            produced: dict = {}
            records: list = []
            report = {'problem': problem.name, 'device': runner.device_info, 'options': dataclasses.asdict(options),
                      'opt_level': settings['opt_level'], 'compiler_sha256': settings.get('compiler_sha256')}
            try:
                metadata = json.loads((problem / 'meta.json').read_text())
                report.update(rtol=metadata['rtol'], atol=metadata['atol'])
                for launch in metadata['kernels']:
                    entry = launch['entry']
                    path = problem / (entry + '.ir.json')
                    if (problem, entry) in batched:
                        compilation, seconds = batched[(problem, entry)], batch_seconds
                    else:
                        started = time.perf_counter()
                        compilation = compile_kernel(path, arch=arch, opt_level=settings['opt_level'], options=options)
                        seconds = time.perf_counter() - started
                    (destination / f'{entry}.ptx').write_text(compilation.ptx)
                    record = runner.run_kernel(launch, compilation, produced, warmup=settings['warmup'], iters=settings['iters'],
                                               samples=settings['samples'])
                    produced.update(record.pop('outputs'))
                    np.savez(destination / 'actual.npz', **produced)
                    record.update(compile_seconds=seconds, ptx_sha256=hashlib.sha256(compilation.ptx.encode()).hexdigest(),
                                  ir_sha256=hashlib.sha256(path.read_bytes()).hexdigest(), plan=compilation.plan.describe())
                    records.append(record)
                report.update(passed=True, max_abs_error=compare_outputs(problem, metadata, produced), kernels=records)
                print(f"PASS {problem.name}: {sum(r['median_us'] for r in records):.3f} us", flush=True)
            except Exception as error:   # one failing problem must not stop the others (benchmark.py:486-491)
                report.update(passed=False, error=str(error), kernels=records)
                print(f'FAIL {problem.name}: {error}', file=sys.stderr, flush=True)
                if isinstance(error, CudaError):
                    runner.close()
                    runner = LocalRunner(device)
            write_json(destination / 'result.json', report)
            reports.append(report)
    finally:
        runner.close()
    return reports


def main(argv: Any = None) -> int:
    parser = argparse.ArgumentParser(prog='deuteron_b200.benchmark')
    parser.add_argument('problems', nargs='*')
    parser.add_argument('--problems-dir', required=True, type=Path)
    parser.add_argument('--devices', default='0')
    parser.add_argument('--jobs', type=int, default=1)
    parser.add_argument('--artifacts', type=Path, default=Path('benchmark-results'))
    parser.add_argument('--arch')
    parser.add_argument('--opt-level', type=int, choices=range(4), default=3)
    parser.add_argument('--contraction-precision', choices=('f32', 'tf32x3', 'bf16x3'))
    parser.add_argument('--approximate-math', action=argparse.BooleanOptionalAction)
    parser.add_argument('--warmup', type=int, default=20)
    parser.add_argument('--iters', type=int, default=200)
    parser.add_argument('--samples', type=int, default=7)
    args = parser.parse_args(argv)
    if args.warmup < 0 or args.iters < 1 or args.samples < 1:
        parser.error('warmup must be nonnegative and iters/samples positive')
    if args.jobs < 1:
        parser.error('jobs must be positive')
    if not args.problems_dir.is_dir():
        parser.error(f'problems directory does not exist: {args.problems_dir}')
    available = sorted(p for p in args.problems_dir.resolve().iterdir() if (p / 'meta.json').is_file())
    problems = []
    for name in args.problems:
        matches = [p for p in available if p.name == name] or [p for p in available if p.name.startswith(name)]
        if len(matches) != 1:
            parser.error(f'problem {name!r} must match one directory')
        problems.append(matches[0])
    problems = problems or available
    if not problems or len(set(problems)) != len(problems):
        parser.error('select one or more distinct problems')
    try:
        devices = [int(d) for d in args.devices.split(',')]
    except ValueError:
        parser.error('devices must be comma-separated integers')
    if min(devices) < 0 or len(set(devices)) != len(devices):
        parser.error('devices must be distinct nonnegative ordinals')
    args.artifacts = args.artifacts.resolve()
    args.artifacts.mkdir(parents=True, exist_ok=True)
    try:
        reserve_artifacts(args.artifacts)
    except ValueError as exc:
        parser.error(str(exc))
    settings = {k: str(v) if isinstance(v, Path) else v for k, v in vars(args).items()}
    root = Path(__file__).parent
    sources = sorted(root.rglob('*.py')) + sorted((root / 'csrc').glob('*.cu*')) + sorted((root.parent / 'include').glob('*.h'))
    settings['compiler_sha256'] = {str(path.relative_to(root.parent)): hashlib.sha256(path.read_bytes()).hexdigest() for path in sources}
    write_json(args.artifacts / 'manifest.json', settings)
    partitions = [(d, [str(p) for p in problems[i::len(devices)]], settings) for i, d in enumerate(devices) if problems[i::len(devices)]]
    if len(partitions) == 1:
        reports = run_partition(*partitions[0])
    else:
        with ProcessPoolExecutor(max_workers=len(partitions), mp_context=multiprocessing.get_context('spawn')) as pool:
            reports = [report for future in [pool.submit(run_partition, *part) for part in partitions] for report in future.result()]
    reports.sort(key=lambda report: report['problem'])
    write_json(args.artifacts / 'results.json', reports)
    print(f"{sum(r['passed'] for r in reports)}/{len(reports)} passed")
    return int(not all(r['passed'] for r in reports))


if __name__ == '__main__':
    raise SystemExit(main())
