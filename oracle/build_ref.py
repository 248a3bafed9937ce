"""Builds the reference's own kernels for sm_100a. Test infrastructure, not product code.

Two sources, both read where the reference checkout lies; nothing of the reference is copied into the tracked
tree and every output goes to oracle/_ref/ (git-ignored):

  1. The one PTX file the reference committed after emitting it itself, docs/video/demo/capture/kernel.ptx
     (`matmul_tiled_128` of examples/tensor_matmul, tf32x3, written for sm_120): retargeted and assembled as
     `matmul_tiled_128_tf32x3.cubin`.
  2. The UNMODIFIED reference compiler, run here on scheduled IR with `arch='sm_100'`. It imports its IR classes
     from the third-party package emmy-ml, which is not available offline; oracle/emmy_standin supplies
     stand-ins for exactly those classes (see its README). With them the compiler emits, for its committed
     tensor_matmul IR, PTX with the same instruction mix as the PTX it committed (48 mma.sync.m16n8k8, 192
     cvt.rna.tf32, 12 cp.async.cg, 4 bar.sync, 96 shared loads; the LLVM behind llvmlite differs, so register
     names and a few moves differ). The kernels built this way:
       gemm_<mode>_<n>      n^3 compensated GEMM, mode in bf16x3 / tf32x3 / f32: the committed IR at 128, the
                            same schedule scaled by deuteron_b200.schedules.matmul_example above that
       attention_*          examples/attention.py `example(rows, keys, depth[, inplace_denominator])`
       f16_<kind>           examples/f16_storage.py `example(kind)`
       vector_add           examples/vector_add (committed IR)
       vector_add_2p28, f16_<kind>_2p28, row_<op>_65536x4096
                            the memory-bound kernels at their benchmark sizes (the reference's f16 generator; vector add
                            and row reductions from deuteron_b200.schedules in the reference's launch shapes)
       open_<name>          the fifteen open workloads in the reference's launch shapes, from
                            deuteron_b200.schedules.open_workloads() (the reference's own files for them are
                            not in the checkout); the reference's validator and passes accept every one
     Each becomes `<name>.cubin`; `manifest.json` records entry, launch geometry, argument order and buffers
     (the launch of its meta.json), so that oracle/ref_kernel.py can run it on the GPU box, where neither the
     reference nor llvmlite need to be present.

    python -m oracle.build_ref /path/to/deuteron        (or DEUTERON_REFERENCE=/path/to/deuteron)
"""
from __future__ import annotations

import hashlib
import importlib.util
import json
import os
import re
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / '_ref'
OUTPUT = OUT / 'matmul_tiled_128_tf32x3.cubin'
MANIFEST = OUT / 'manifest.json'
COMMITTED_PTX = Path('docs') / 'video' / 'demo' / 'capture' / 'kernel.ptx'
GEMM_SIZES = (128, 512, 2048, 8192)
ATTENTION_CASES = {
    'attention_3x64x32': dict(rows=3, keys=64, depth=32),
    'attention_64x64x64': dict(rows=64, keys=64, depth=64),
    'attention_128x128x32': dict(rows=128, keys=128, depth=32),
    'attention_128x128x32_inplace': dict(rows=128, keys=128, depth=32, inplace_denominator=True),
    'attention_256x256x128': dict(rows=256, keys=256, depth=128),
}
F16_KINDS = ('copy', 'widen', 'narrow', 'affine', 'cancellation')


def reference_root(explicit: str | Path | None = None) -> Path | None:
    """The reference checkout: the argument, else $DEUTERON_REFERENCE, else a `reference` directory beside this
    repository. None when there is none."""
    candidates = [explicit, os.environ.get('DEUTERON_REFERENCE'), HERE.parent.parent / 'reference']
    for candidate in candidates:
        if candidate and (Path(candidate) / 'compiler' / 'build.py').is_file():
            return Path(candidate)
    return None


def _ptxas() -> str | None:
    found = shutil.which('ptxas') or '/usr/local/cuda/bin/ptxas'
    return found if Path(found).exists() else None


def _assemble(ptx_text: str, output: Path) -> dict:
    """PTX text (any .target) -> cubin for sm_100a. Returns ptxas's resource line."""
    retargeted, count = re.subn(r'^\.target\s+sm_\d+a?\b', '.target sm_100a', ptx_text, count=1, flags=re.MULTILINE)
    if count != 1:
        raise RuntimeError('PTX without a .target line')
    output.parent.mkdir(parents=True, exist_ok=True)
    with tempfile.TemporaryDirectory() as scratch:
        ptx = Path(scratch) / 'kernel.ptx'
        ptx.write_text(retargeted)
        done = subprocess.run([_ptxas(), '-arch=sm_100a', '-O3', '-v', '-o', str(output), str(ptx)], check=True, capture_output=True, text=True)
    used = re.search(r'Used (\d+) registers', done.stderr)
    return {'registers': int(used.group(1)) if used else None}


def build_committed_ptx(root: Path, output: Path = OUTPUT) -> Path | None:
    source = root / COMMITTED_PTX
    if not source.is_file():
        return None
    text = source.read_text()
    if '.entry matmul_tiled_128(' not in text:
        raise RuntimeError(f'{source}: not the PTX this recipe expects')
    if re.search(r'\bbra\b', text):
        raise RuntimeError(f'{source}: contains branches; it was straight-line code when this recipe was written')
    _assemble(text, output)
    return output


def _example_module(root: Path, name: str):
    spec = importlib.util.spec_from_file_location(f'_reference_example_{name}', root / 'examples' / f'{name}.py')
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def reference_cases(root: Path) -> dict:
    """name -> (graph, meta, options keyword arguments) of every kernel to build."""
    sys.path.insert(0, str(HERE.parent))
    from deuteron_b200 import schedules
    cases: dict = {}
    committed_graph = json.loads((root / 'examples/tensor_matmul/matmul_tiled_128.ir.json').read_text())
    committed_meta = json.loads((root / 'examples/tensor_matmul/meta.json').read_text())
    for mode in ('bf16x3', 'tf32x3', 'f32'):
        for n in GEMM_SIZES:
            if mode == 'f32' and n > 2048:
                continue
            pair = (committed_graph, committed_meta) if n == 128 else schedules.matmul_example(n, n, n)
            cases[f'gemm_{mode}_{n}'] = (*pair, {'contraction_precision': mode})
    attention = _example_module(root, 'attention')
    for name, configuration in ATTENTION_CASES.items():
        cases[name] = (*attention.example(**configuration), {})
    storage = _example_module(root, 'f16_storage')
    for kind in F16_KINDS:
        cases[f'f16_{kind}'] = (*storage.example(kind), {})
    cases['vector_add'] = (json.loads((root / 'examples/vector_add/vector_add.ir.json').read_text()),
                           json.loads((root / 'examples/vector_add/meta.json').read_text()), {})
    for name, pair in schedules.open_workloads().items():
        cases[f'open_{name}'] = (*pair, {})
    # the memory-bound kernels at their benchmark sizes
    cases['vector_add_2p28'] = (*schedules.vector_add_example(1 << 28), {})
    for kind in ('copy', 'widen', 'narrow'):
        cases[f'f16_{kind}_2p28'] = (*storage.example(kind, count=1 << 28, width=4), {})
    for op in ('sum', 'max'):
        cases[f'row_{op}_65536x4096'] = (*schedules.row_reduce_example(65536, 4096, op), {})
    return cases


def build_compiled(root: Path, only: str | None = None) -> dict:
    """Runs the reference compiler on every case and assembles what it emits. Returns the manifest."""
    for path in (str(HERE / 'emmy_standin'), str(root)):
        if path not in sys.path:
            sys.path.insert(0, path)
    from compiler import Options, compile_kernel     # the reference's own package
    manifest = json.loads(MANIFEST.read_text()) if MANIFEST.exists() else {}
    kernels = manifest.setdefault('kernels', {})
    for name, (graph, meta, option_fields) in reference_cases(root).items():
        if only and only not in name:
            continue
        launch = meta['kernels'][0]
        with tempfile.TemporaryDirectory() as scratch:
            source = Path(scratch) / 'kernel.ir.json'
            source.write_text(json.dumps(graph))
            source.with_name('meta.json').write_text(json.dumps(meta))
            compilation = compile_kernel(source, arch='sm_100', opt_level=3, options=Options(**option_fields))
        resources = _assemble(compilation.ptx, OUT / f'{name}.cubin')
        # the IR and meta the kernel was compiled from travel with it, so that the same pair can be handed to this
        # build's compile_kernel on the GPU box
        (OUT / f'{name}.case.json').write_text(json.dumps({'graph': graph, 'meta': meta, 'options': option_fields}))
        kernels[name] = {'cubin': f'{name}.cubin', 'entry': launch['entry'], 'grid': launch['grid'], 'block': launch['block'],
                         'smem_bytes': launch.get('smem_bytes', 0), 'arg_order': launch['arg_order'], 'args': launch['args'],
                         'zero_outputs': launch.get('zero_outputs', []), 'rtol': meta.get('rtol'), 'atol': meta.get('atol'),
                         'options': option_fields, 'registers': resources['registers'],
                         'ptx_sha256': hashlib.sha256(compilation.ptx.encode()).hexdigest(),
                         'mma_sync': compilation.ptx.count('mma.sync')}
    manifest['how'] = 'unmodified reference compiler (arch sm_100, opt_level 3) + oracle/emmy_standin, ptxas -arch=sm_100a -O3'
    OUT.mkdir(parents=True, exist_ok=True)
    MANIFEST.write_text(json.dumps(manifest, indent=1) + '\n')
    return manifest


def build(reference: str | Path | None = None, only: str | None = None) -> Path | None:
    """Builds everything that can be built. Returns the path of the committed-PTX cubin (None when neither the
    reference checkout nor an earlier build is there). A missing checkout leaves earlier outputs in place."""
    root = reference_root(reference)
    if root is None or _ptxas() is None:
        return OUTPUT if OUTPUT.exists() else None
    built = build_committed_ptx(root)
    try:
        import llvmlite  # noqa: F401  (the reference compiler's code generator)
    except ImportError:
        return built
    build_compiled(root, only)
    return built


if __name__ == '__main__':
    arguments = [a for a in sys.argv[1:] if not a.startswith('--only=')]
    chosen = next((a.split('=', 1)[1] for a in sys.argv[1:] if a.startswith('--only=')), None)
    result = build(arguments[0] if arguments else None, chosen)
    print(result if result else 'reference checkout or ptxas not found; nothing built')
    if MANIFEST.exists():
        print(f'{len(json.loads(MANIFEST.read_text())["kernels"])} compiled kernels in {MANIFEST}')
