"""Regenerates the golden fixtures in this directory from the reference checkout.

Run where the reference (stashuk-olek/deuteron) is available:

    python tests/golden/make_golden.py /path/to/deuteron

It copies the reference's own known-answer data (no source code):
  * examples/tensor_matmul/expected.npz and examples/vector_add/expected.npz (float64 product and exact
    FP32 sum of the seeded inputs), stored compressed;
  * from benchmarks/features-rtx5090-2026-10-24-r6.json, for each example kernel the reference ran on
    a GPU: its max absolute error against the float64 expectation and the SHA-256 of the output bytes;
  * the launch geometry recorded in the examples' meta.json files.
The tests never read the reference checkout; they read these files.
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def main(reference: Path) -> None:
    with np.load(reference / 'examples/tensor_matmul/expected.npz') as data:
        np.savez_compressed(HERE / 'tensor_matmul_expected.npz', result=data['result'])
    with np.load(reference / 'examples/vector_add/expected.npz') as data:
        np.savez_compressed(HERE / 'vector_add_expected.npz', sum=data['sum'])
    features = json.loads((reference / 'benchmarks/features-rtx5090-2026-10-24-r6.json').read_text())
    published = {}
    for result in features['results']:
        published[result['name']] = {
            'entry': result['entry'],
            'arch': result['arch'],
            'registers': result['registers'],
            'median_us': result['median_us'],
            'max_absolute_errors': result['max_absolute_errors'],
            'output_sha256': result['output_sha256'],
        }
    metas = {}
    for name in ('tensor_matmul', 'vector_add'):
        metas[name] = json.loads((reference / 'examples' / name / 'meta.json').read_text())
    (HERE / 'reference_published.json').write_text(json.dumps({
        'source': 'benchmarks/features-rtx5090-2026-10-24-r6.json (RTX 5090, sm_120) and examples/*/meta.json',
        'results': published,
        'meta': metas,
    }, indent=1) + '\n')
    for name, source in (('tensor_matmul', 'matmul_tiled_128.ir.json'), ('vector_add', 'vector_add.ir.json')):
        # the scheduled IR of the two self-contained examples is input data for the boundary tests
        (HERE / f'{name}.ir.json').write_text((reference / 'examples' / name / source).read_text())
    print('wrote', sorted(p.name for p in HERE.iterdir()))


if __name__ == '__main__':
    main(Path(sys.argv[1] if len(sys.argv) > 1 else '/root/reference'))
