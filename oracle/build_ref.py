"""Builds the one piece of the reference that can be built here: its own emitted kernel.

Test infrastructure, not product code. The reference is a Python compiler that needs the absent
`emmy-ml` package, so it cannot emit PTX in this container; but it commits one PTX file it emitted
itself, `docs/video/demo/capture/kernel.ptx` -- `matmul_tiled_128` of examples/tensor_matmul compiled
with `--contraction-precision tf32x3 --opt-level 3` (docs/video/demo/capture/command.txt). That file
is straight-line code (no branches, ends in `ret`), written for `.target sm_120`. This recipe reads it
where it lies, retargets it to sm_100a and assembles it with ptxas into
`oracle/_ref/matmul_tiled_128_tf32x3.cubin`; nothing of the reference is copied into the tracked
tree. The cubin is loaded by oracle/ref_kernel.py so that the reference's own kernel and this
build's kernels can be run on the same B200 with the same inputs.

    python -m oracle.build_ref [/path/to/reference]
"""
from __future__ import annotations

import re
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUTPUT = HERE / '_ref' / 'matmul_tiled_128_tf32x3.cubin'
SOURCE = Path('docs') / 'video' / 'demo' / 'capture' / 'kernel.ptx'


def build(reference_root: str | Path = '/root/reference', output: Path = OUTPUT) -> Path | None:
    """Assembles the reference's committed PTX for sm_100a. Returns the cubin path, or None when the reference
    tree (or ptxas) is not present -- then an earlier build of the cubin, if any, is left in place."""
    source = Path(reference_root) / SOURCE
    ptxas = shutil.which('ptxas') or '/usr/local/cuda/bin/ptxas'
    if not source.is_file() or not Path(ptxas).exists():
        return output if output.exists() else None
    text = source.read_text()
    retargeted, count = re.subn(r'^\.target\s+sm_120\b', '.target sm_100a', text, count=1, flags=re.MULTILINE)
    if count != 1 or '.entry matmul_tiled_128(' not in retargeted:
        raise RuntimeError(f'{source}: not the PTX this recipe expects')
    if re.search(r'\bbra\b', retargeted):
        raise RuntimeError(f'{source}: contains branches; it was straight-line code when this recipe was written')
    output.parent.mkdir(parents=True, exist_ok=True)
    with tempfile.TemporaryDirectory() as scratch:
        ptx = Path(scratch) / 'kernel_sm100a.ptx'
        ptx.write_text(retargeted)
        subprocess.run([ptxas, '-arch=sm_100a', '-O3', '-o', str(output), str(ptx)], check=True)
    return output


if __name__ == '__main__':
    built = build(sys.argv[1] if len(sys.argv) > 1 else '/root/reference')
    print(built if built else 'reference PTX or ptxas not found; nothing built')
