"""Command line of the compile surface, with the flags of the reference's `deuteron` command
(compiler/cli.py:69-99): `python -m deuteron_b200 KERNEL.ir.json [--arch sm_100a] [--opt-level N]
[--contraction-precision ...] [--dump-llvm PATH] [--dump-unoptimized PATH]`.

The reference prints the PTX it emitted; this build prints the text of the native kernel selection
(`Compilation.ptx`). Diagnostics go to stderr and the exit status is 0, 1 (error) or 130 (interrupt),
as there. Dump paths may not overwrite the kernel or its meta.json and are written atomically.
"""
from __future__ import annotations

import argparse
import os
import sys
import tempfile
from collections.abc import Sequence
from contextlib import redirect_stdout
from pathlib import Path

from .build import compile_kernel
from .options import Options

_SWITCHES = ('approximate-math', 'reduction-sharing', 'recurrence-staging', 'tree-specialization', 'coalesced-reductions',
             'warp-willreturn', 'elementwise-vectorize', 'register-forwarding', 'tail-linearize')


def _same_file(left: Path, right: Path) -> bool:
    return left == right or (left.exists() and right.exists() and left.samefile(right))


def _dump_paths(kernel: Path, requested: tuple[Path | None, ...]) -> list[Path | None]:
    protected = [kernel.resolve(), kernel.with_name('meta.json').resolve()]
    chosen: list[Path | None] = []
    for wanted in requested:
        if wanted is None:
            chosen.append(None)
            continue
        path = wanted.resolve()
        if any(_same_file(path, other) for other in protected):
            raise ValueError(f'dump path would overwrite an input file: {wanted}')
        if any(other is not None and _same_file(path, other) for other in chosen):
            raise ValueError('dump paths must refer to different files')
        if path.exists() and not path.is_file():
            raise ValueError(f'dump path is not a regular file: {wanted}')
        if not path.parent.is_dir():
            raise ValueError(f'dump parent is not an existing directory: {wanted.parent}')
        chosen.append(path)
    return chosen


def _write_atomically(files: list[tuple[Path, str]]) -> None:
    staged: list[tuple[Path, Path]] = []
    try:
        for destination, content in files:
            with tempfile.NamedTemporaryFile(mode='w', encoding='utf-8', newline='\n', dir=destination.parent,
                                             prefix='.' + destination.name + '.', suffix='.tmp', delete=False) as stream:
                staged.append((Path(stream.name), destination))
                stream.write(content)
                stream.flush()
                os.fsync(stream.fileno())
        for temporary, destination in staged:
            temporary.replace(destination)
    finally:
        for temporary, _ in staged:
            temporary.unlink(missing_ok=True)


def main(argv: Sequence[str] | None = None) -> int:
    from . import __version__
    parser = argparse.ArgumentParser(prog='deuteron_b200', description='Select the native sm_100a kernel for scheduled Kernel IR')
    parser.add_argument('--version', action='version', version=f'deuteron_b200 {__version__}')
    parser.add_argument('kernel', type=Path)
    parser.add_argument('--arch', default='sm_100a')
    parser.add_argument('--opt-level', type=int, choices=range(4), default=3)
    parser.add_argument('--unroll', type=int, choices=(0, 1, 2, 4, 8, 16, 32), default=0)
    parser.add_argument('--vector-width', type=int, choices=(1, 2, 4, 8, 16), default=4)
    parser.add_argument('--contraction-precision', choices=('f32', 'tf32x3', 'bf16x3'), default='bf16x3')
    for flag in _SWITCHES:
        parser.add_argument('--' + flag, action=argparse.BooleanOptionalAction, default=True)
    parser.add_argument('--dump-llvm', type=Path)
    parser.add_argument('--dump-unoptimized', type=Path)
    args = parser.parse_args(argv)
    try:
        paths = _dump_paths(args.kernel, (args.dump_llvm, args.dump_unoptimized))
        options = Options(**{name: getattr(args, name) for name in Options.__dataclass_fields__})
        with redirect_stdout(sys.stderr):
            result = compile_kernel(args.kernel, arch=args.arch, opt_level=args.opt_level, options=options)
        _write_atomically([(path, text) for path, text in zip(paths, (result.optimized, result.unoptimized)) if path is not None])
        sys.stdout.write(result.ptx)
        sys.stdout.flush()
    except (OSError, ValueError, NotImplementedError, RuntimeError) as exc:
        print(f'{parser.prog}: error: {exc}', file=sys.stderr)
        return 1
    except KeyboardInterrupt:
        print(f'{parser.prog}: interrupted', file=sys.stderr)
        return 130
    return 0
