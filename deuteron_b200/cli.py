"""`python -m deuteron_b200 KERNEL.ir.json [flags]`: the compile surface from a shell.

Behaviour contract of the reference's `deuteron` command (compiler/cli.py:69-99, tests/test_cli.py): one
positional kernel path with its meta.json beside it; `--arch`, `--opt-level`, one flag per field of Options
(booleans as `--name` / `--no-name`), `--dump-llvm PATH`, `--dump-unoptimized PATH`, `--version`. The text of the
compilation goes to stdout (there: PTX; here: the description of the native kernel selection, `Compilation.ptx`),
everything else to stderr; exit status 0, 1 on any error, 130 on an interrupt. A dump may not land on the kernel
file or its meta.json (by any name: symlink, hard link, `dir/./file`), two dumps may not land on one file, and
existing files change only after the compilation succeeded and every dump has been staged.
"""
from __future__ import annotations

import argparse
import contextlib
import dataclasses
import os
import sys
import tempfile
from collections.abc import Sequence
from pathlib import Path

from .build import compile_kernel
from .options import Options

PROGRAM = 'deuteron_b200'
_CHOICES = {'contraction_precision': ('f32', 'tf32x3', 'bf16x3'), 'vector_width': (1, 2, 4, 8, 16), 'unroll': (0, 1, 2, 4, 8, 16, 32)}


def _file_identity(path: Path) -> tuple:
    """What makes two names the same file: device and inode when it exists, else its resolved spelling."""
    try:
        status = os.stat(path)
        return ('inode', status.st_dev, status.st_ino)
    except OSError:
        return ('name', os.path.realpath(path))


class DumpPlan:
    """The dump destinations of one invocation, checked before anything is compiled and written all-or-nothing."""

    def __init__(self, kernel: Path) -> None:
        self._taken = {_file_identity(kernel): 'input', _file_identity(kernel.with_name('meta.json')): 'input'}
        self._targets: list[tuple[Path, str]] = []     # (destination, which text of the Compilation)

    def claim(self, destination: Path | None, text_of: str) -> None:
        if destination is None:
            return
        owner = self._taken.get(_file_identity(destination))
        if owner == 'input':
            raise ValueError(f'dump path would overwrite an input file: {destination}')
        if owner == 'dump':
            raise ValueError('dump paths must refer to different files')
        if os.path.lexists(destination) and not os.path.isfile(destination):
            raise ValueError(f'dump path is not a regular file: {destination}')
        folder = destination.parent
        if not folder.is_dir():
            raise ValueError(f'dump parent is not an existing directory: {folder}')
        self._taken[_file_identity(destination)] = 'dump'
        self._targets.append((Path(os.path.realpath(destination)), text_of))

    def publish(self, compilation) -> None:
        """Stage every dump beside its destination, then rename them into place; on any failure nothing that existed
        before has changed and no staging file is left."""
        with contextlib.ExitStack() as cleanup:
            renames = []
            for destination, text_of in self._targets:
                handle = tempfile.NamedTemporaryFile(mode='w', encoding='utf-8', newline='\n', delete=False, dir=destination.parent,
                                                     prefix=f'.{destination.name}.', suffix='.tmp')
                staged = Path(handle.name)
                cleanup.callback(staged.unlink, missing_ok=True)
                with handle:
                    handle.write(getattr(compilation, text_of))
                    handle.flush()
                    os.fsync(handle.fileno())
                renames.append((staged, destination))
            for staged, destination in renames:
                staged.replace(destination)


def build_parser() -> argparse.ArgumentParser:
    from . import __version__
    parser = argparse.ArgumentParser(prog=PROGRAM, description='Select the native sm_100a kernel for scheduled Kernel IR')
    parser.add_argument('--version', action='version', version=f'{PROGRAM} {__version__}')
    parser.add_argument('kernel', type=Path, help='scheduled Kernel IR (JSON); meta.json is read from the same directory')
    parser.add_argument('--arch', default='sm_100a')
    parser.add_argument('--opt-level', type=int, choices=(0, 1, 2, 3), default=3)
    for field in dataclasses.fields(Options):
        flag = '--' + field.name.replace('_', '-')
        if isinstance(field.default, bool):
            parser.add_argument(flag, action=argparse.BooleanOptionalAction, default=field.default)
        else:
            parser.add_argument(flag, type=type(field.default), choices=_CHOICES[field.name], default=field.default)
    parser.add_argument('--dump-llvm', type=Path, metavar='PATH', help='also write the optimized text here')
    parser.add_argument('--dump-unoptimized', type=Path, metavar='PATH', help='also write the unoptimized text here')
    return parser


def _run(args: argparse.Namespace) -> None:
    dumps = DumpPlan(args.kernel)
    dumps.claim(args.dump_llvm, 'optimized')
    dumps.claim(args.dump_unoptimized, 'unoptimized')
    options = Options(**{field.name: getattr(args, field.name) for field in dataclasses.fields(Options)})
    with contextlib.redirect_stdout(sys.stderr):        # whatever the compile step prints is a diagnostic
        compilation = compile_kernel(args.kernel, arch=args.arch, opt_level=args.opt_level, options=options)
    dumps.publish(compilation)
    sys.stdout.write(compilation.ptx)
    sys.stdout.flush()


def main(argv: Sequence[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    try:
        _run(args)
        return 0
    except KeyboardInterrupt:
        print(f'{PROGRAM}: interrupted', file=sys.stderr)
        return 130
    except (OSError, ValueError, NotImplementedError, RuntimeError) as problem:
        if isinstance(problem, BrokenPipeError):
            # the reader went away: keep the interpreter from complaining again when it flushes stdout at exit
            with contextlib.suppress(OSError):
                os.dup2(os.open(os.devnull, os.O_WRONLY), sys.stdout.fileno())
        print(f'{PROGRAM}: error: {problem}', file=sys.stderr)
        return 1
