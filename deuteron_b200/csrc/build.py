"""Builds libdeuteron_b200.so in-tree with nvcc for sm_100a.

Usage: python -m deuteron_b200.csrc.build [--force] [--verbose]

Each .cu file is compiled to an object (in parallel) and the objects are linked into
deuteron_b200/libdeuteron_b200.so. Objects are rebuilt only when a source or header is newer.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PACKAGE = CSRC.parent
LIBRARY = PACKAGE / 'libdeuteron_b200.so'
OBJECTS = CSRC / 'build'
ARCH_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a']
COMMON_FLAGS = ['-O3', '-std=c++17', '-lineinfo', '-Xcompiler', '-fPIC', '--expt-relaxed-constexpr']


def nvcc() -> str:
    found = shutil.which('nvcc') or '/usr/local/cuda/bin/nvcc'
    if not Path(found).exists():
        raise RuntimeError('nvcc not found; the CUDA toolkit is required to build deuteron_b200')
    return found


def sources() -> list[Path]:
    return sorted(CSRC.glob('*.cu'))


def _newest_header() -> float:
    headers = list(CSRC.glob('*.cuh')) + list((PACKAGE.parent / 'include').glob('*.h'))
    return max((h.stat().st_mtime for h in headers), default=0.0)


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJECTS.mkdir(exist_ok=True)
    compiler = nvcc()
    header_time = _newest_header()
    jobs = []
    for source in sources():
        obj = OBJECTS / (source.stem + '.o')
        stale = force or not obj.exists() or obj.stat().st_mtime < max(source.stat().st_mtime, header_time)
        if stale:
            command = [compiler, *ARCH_FLAGS, *COMMON_FLAGS, '-c', str(source), '-o', str(obj)]
            if verbose:
                command.insert(1, '-Xptxas=-v')
            jobs.append(command)

    def run(command: list[str]) -> None:
        result = subprocess.run(command, capture_output=True, text=True)
        if verbose or result.returncode:
            sys.stderr.write(' '.join(command) + '\n' + result.stdout + result.stderr)
        if result.returncode:
            raise RuntimeError(f'nvcc failed for {command[-3]}')

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        list(pool.map(run, jobs))
    objects = [OBJECTS / (s.stem + '.o') for s in sources()]
    if jobs or not LIBRARY.exists() or force:
        link = [compiler, *ARCH_FLAGS, '-shared', '-o', str(LIBRARY), *map(str, objects), '-lcudart']
        result = subprocess.run(link, capture_output=True, text=True)
        if result.returncode:
            sys.stderr.write(result.stdout + result.stderr)
            raise RuntimeError('linking libdeuteron_b200.so failed')
    return LIBRARY


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument('--force', action='store_true')
    parser.add_argument('--verbose', action='store_true')
    args = parser.parse_args()
    print(build(args.force, args.verbose))


if __name__ == '__main__':
    main()
