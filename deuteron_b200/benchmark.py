"""Runs directories of problems through compile_kernel + LocalRunner and records what happened.

    python -m deuteron_b200.benchmark --problems-dir DIR [problem ...] [--devices 0,1] [--artifacts OUT]

Conventions of the reference's benchmark driver (benchmark.py:289-308, 434-557), so that its problem
directories and its result files keep working: a problem is a directory with `meta.json`, one
`<entry>.ir.json` per kernel named there and `expected.npz`; the kernels of a problem run in the order of
the meta and hand their outputs on (`intermediate` buffers); a run owns its artifacts directory (a second
run into it is refused) and leaves `manifest.json`, `results.json` and, per problem, `result.json`,
`actual.npz` and `<entry>.ptx`. A failing problem is recorded and the run goes on. Kernels run on the
native sm_100a library on this machine's GPUs: there is no remote runner and `--arch` defaults to sm_100a.
"""
from __future__ import annotations

import argparse
import dataclasses
import hashlib
import json
import multiprocessing
import os
import sys
import time
import uuid
from concurrent.futures import ProcessPoolExecutor
from pathlib import Path
from typing import Any, Iterable

import numpy as np

from .build import compile_kernel, compile_many
from .native import CudaError
from .options import Options
from .runner import LocalRunner, compare_outputs

RESERVATION = '.deuteron-run'


def _sha256(data: bytes) -> str:
    return hashlib.sha256(data).hexdigest()


def write_json(path: Any, value: Any) -> None:
    """Replaces `path` by the JSON text of `value` in one step: readers see the old file or the new one."""
    path = Path(path)
    scratch = path.with_name(f'{path.name}.{uuid.uuid4().hex}.tmp')
    try:
        scratch.write_text(json.dumps(value, indent=2) + '\n', encoding='utf-8')
        os.replace(scratch, path)
    finally:
        scratch.unlink(missing_ok=True)


def reserve_artifacts(path: Path) -> None:
    """Claims an artifacts directory for this run. A directory that holds a finished run's manifest, or that another
    run has claimed, is refused: measurements are never overwritten."""
    path = Path(path)
    if (path / 'manifest.json').exists():
        raise ValueError(f'use a new artifacts directory to preserve previous measurements: {path}')
    claim = json.dumps({'pid': os.getpid(), 'started': time.time()}) + '\n'
    try:
        descriptor = os.open(path / RESERVATION, os.O_WRONLY | os.O_CREAT | os.O_EXCL, 0o644)
    except FileExistsError:
        raise ValueError(f'artifacts directory is already reserved by another run: {path}') from None
    with os.fdopen(descriptor, 'w') as stream:
        stream.write(claim)


@dataclasses.dataclass(frozen=True)
class RunSettings:
    """What every device worker needs; plain data, so that it crosses a process boundary."""
    artifacts: str
    arch: str
    opt_level: int
    warmup: int
    iters: int
    samples: int
    jobs: int
    option_overrides: tuple          # ((field, value), ...) applied on top of Options()
    sources_sha256: tuple            # ((relative path, sha256), ...) of this build's sources

    def options(self) -> Options:
        return dataclasses.replace(Options(), **dict(self.option_overrides))


class Problem:
    """One problem directory."""

    def __init__(self, folder: Path) -> None:
        self.folder = Path(folder)
        self.name = self.folder.name
        self.metadata = json.loads((self.folder / 'meta.json').read_text())

    def kernels(self) -> Iterable[tuple[dict, Path]]:
        for launch in self.metadata['kernels']:
            yield launch, self.folder / f"{launch['entry']}.ir.json"


class DeviceWorker:
    """Runs problems one after another on one GPU, in the calling process."""

    def __init__(self, device: int, settings: RunSettings) -> None:
        self.device, self.settings, self.options = device, settings, settings.options()
        self.runner = LocalRunner(device)
        self.precompiled: dict[Path, tuple[Any, float]] = {}

    def close(self) -> None:
        self.runner.close()

    def precompile(self, problems: list[Problem]) -> None:
        """With --jobs > 1 every kernel of every problem is compiled up front by a pool of processes."""
        paths = [path for problem in problems for _, path in problem.kernels()]
        if self.settings.jobs <= 1 or not paths:
            return
        began = time.perf_counter()
        compiled = compile_many([(path, self.settings.arch, self.settings.opt_level, self.options) for path in paths], self.settings.jobs)
        each = (time.perf_counter() - began) / len(paths)
        self.precompiled = {path: (result, each) for path, result in zip(paths, compiled)}

    def _compile(self, path: Path) -> tuple[Any, float]:
        if path in self.precompiled:
            return self.precompiled[path]
        began = time.perf_counter()
        result = compile_kernel(path, arch=self.settings.arch, opt_level=self.settings.opt_level, options=self.options)
        return result, time.perf_counter() - began

    def run(self, problem: Problem) -> dict:
        settings = self.settings
        out = Path(settings.artifacts) / problem.name
        out.mkdir(parents=True, exist_ok=True)
        report: dict[str, Any] = {'problem': problem.name, 'device': self.runner.device_info, 'options': dataclasses.asdict(self.options),
                                  'opt_level': settings.opt_level, 'compiler_sha256': dict(settings.sources_sha256)}
        buffers: dict[str, np.ndarray] = {}
        measured: list[dict] = []
        try:
            report['rtol'], report['atol'] = problem.metadata['rtol'], problem.metadata['atol']
            for launch, source in problem.kernels():
                compilation, seconds = self._compile(source)
                (out / f"{launch['entry']}.ptx").write_text(compilation.ptx)
                record = self.runner.run_kernel(launch, compilation, buffers, warmup=settings.warmup, iters=settings.iters,
                                                samples=settings.samples)
                buffers.update(record.pop('outputs'))
                np.savez(out / 'actual.npz', **buffers)
                record['compile_seconds'] = seconds
                record['ptx_sha256'] = _sha256(compilation.ptx.encode())
                record['ir_sha256'] = _sha256(source.read_bytes())
                record['plan'] = compilation.plan.describe()
                measured.append(record)
            report['max_abs_error'] = compare_outputs(problem.folder, problem.metadata, buffers)
            report['passed'] = True
            print(f"PASS {problem.name}: {sum(r['median_us'] for r in measured):.3f} us", flush=True)
        except Exception as failure:   # noqa: BLE001 - recorded; the other problems still run
            report['passed'], report['error'] = False, str(failure)
            print(f'FAIL {problem.name}: {failure}', file=sys.stderr, flush=True)
            if isinstance(failure, CudaError):      # the context may be unusable: start over on this device
                self.runner.close()
                self.runner = LocalRunner(self.device)
        report['kernels'] = measured
        write_json(out / 'result.json', report)
        return report


def run_on_device(device: int, folders: list[str], settings: RunSettings) -> list[dict]:
    """Entry point of one device's share of the run (also the target of the spawned per-device processes)."""
    worker = DeviceWorker(device, settings)
    try:
        problems = [Problem(Path(folder)) for folder in folders]
        worker.precompile(problems)
        return [worker.run(problem) for problem in problems]
    finally:
        worker.close()


def _select(parser: argparse.ArgumentParser, root: Path, wanted: list[str]) -> list[Path]:
    if not root.is_dir():
        parser.error(f'problems directory does not exist: {root}')
    present = sorted(folder for folder in root.resolve().iterdir() if (folder / 'meta.json').is_file())
    if not wanted:
        chosen = present
    else:
        chosen = []
        for text in wanted:
            exact = [folder for folder in present if folder.name == text]
            hits = exact or [folder for folder in present if folder.name.startswith(text)]
            if len(hits) != 1:
                parser.error(f'problem {text!r} must match one directory')
            chosen.append(hits[0])
    if not chosen or len(set(chosen)) != len(chosen):
        parser.error('select one or more distinct problems')
    return chosen


def _devices(parser: argparse.ArgumentParser, text: str) -> list[int]:
    try:
        ordinals = [int(part) for part in text.split(',')]
    except ValueError:
        parser.error('devices must be comma-separated integers')
    if any(ordinal < 0 for ordinal in ordinals) or len(set(ordinals)) != len(ordinals):
        parser.error('devices must be distinct nonnegative ordinals')
    return ordinals


def _source_hashes() -> tuple:
    package = Path(__file__).resolve().parent
    files = [*sorted(package.rglob('*.py')), *sorted((package / 'csrc').glob('*.cu*')), *sorted((package.parent / 'include').glob('*.h'))]
    return tuple((str(path.relative_to(package.parent)), _sha256(path.read_bytes())) for path in files)


def main(argv: Any = None) -> int:
    parser = argparse.ArgumentParser(prog='deuteron_b200.benchmark', description=__doc__.splitlines()[0])
    parser.add_argument('problems', nargs='*', help='names (or unique prefixes) of problem directories; default: all')
    parser.add_argument('--problems-dir', required=True, type=Path)
    parser.add_argument('--devices', default='0', help='comma-separated GPU ordinals; problems are dealt out over them')
    parser.add_argument('--jobs', type=int, default=1, help='processes compiling ahead of the runs')
    parser.add_argument('--artifacts', type=Path, default=Path('benchmark-results'))
    parser.add_argument('--arch', default='sm_100a')
    parser.add_argument('--opt-level', type=int, choices=(0, 1, 2, 3), default=3)
    parser.add_argument('--contraction-precision', choices=('f32', 'tf32x3', 'bf16x3'))
    parser.add_argument('--approximate-math', action=argparse.BooleanOptionalAction)
    parser.add_argument('--warmup', type=int, default=20)
    parser.add_argument('--iters', type=int, default=200)
    parser.add_argument('--samples', type=int, default=7)
    args = parser.parse_args(argv)
    if args.warmup < 0 or min(args.iters, args.samples) < 1:
        parser.error('warmup must be nonnegative and iters/samples positive')
    if args.jobs < 1:
        parser.error('jobs must be positive')
    folders = _select(parser, args.problems_dir, args.problems)
    devices = _devices(parser, args.devices)
    artifacts = args.artifacts.resolve()
    artifacts.mkdir(parents=True, exist_ok=True)
    try:
        reserve_artifacts(artifacts)
    except ValueError as refusal:
        parser.error(str(refusal))
    overrides = tuple((name, getattr(args, name)) for name in ('contraction_precision', 'approximate_math') if getattr(args, name) is not None)
    settings = RunSettings(artifacts=str(artifacts), arch=args.arch, opt_level=args.opt_level, warmup=args.warmup, iters=args.iters,
                           samples=args.samples, jobs=args.jobs, option_overrides=overrides, sources_sha256=_source_hashes())
    manifest = {name: (str(value) if isinstance(value, Path) else value) for name, value in vars(args).items()}
    manifest.update(artifacts=str(artifacts), problems=[folder.name for folder in folders], devices=devices,
                    compiler_sha256=dict(settings.sources_sha256))
    write_json(artifacts / 'manifest.json', manifest)
    shares = [(device, [str(folder) for folder in folders[position::len(devices)]]) for position, device in enumerate(devices)]
    shares = [(device, share) for device, share in shares if share]
    if len(shares) == 1:
        reports = run_on_device(shares[0][0], shares[0][1], settings)
    else:
        with ProcessPoolExecutor(max_workers=len(shares), mp_context=multiprocessing.get_context('spawn')) as pool:
            pending = [pool.submit(run_on_device, device, share, settings) for device, share in shares]
            reports = [report for future in pending for report in future.result()]
    reports.sort(key=lambda report: report['problem'])
    write_json(artifacts / 'results.json', reports)
    passed = sum(bool(report['passed']) for report in reports)
    print(f'{passed}/{len(reports)} passed')
    return 0 if passed == len(reports) else 1


if __name__ == '__main__':
    raise SystemExit(main())
