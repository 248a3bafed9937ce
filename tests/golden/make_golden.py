"""Regenerates the golden fixtures in this directory from the reference checkout.

Run where the reference (stashuk-olek/deuteron) is available:

    python tests/golden/make_golden.py /path/to/deuteron      (or DEUTERON_REFERENCE=/path/to/deuteron)

It copies the reference's own known-answer data (no source code):
  * examples/tensor_matmul/expected.npz and examples/vector_add/expected.npz (float64 product and exact
    FP32 sum of the seeded inputs), stored compressed;
  * from benchmarks/features-rtx5090-2026-10-24-r6.json, for each example kernel the reference ran on
    a GPU: its max absolute error against the float64 expectation and the SHA-256 of the output bytes;
  * the launch geometry recorded in the examples' meta.json files.
  * reference_examples.json: the scheduled IR and meta.json that the reference's own example generators build
    (examples/attention.py `example(...)` at five shapes, examples/f16_storage.py `example(kind)` for the five kinds),
    written exactly as those scripts write them (`repr` of the IR). The generators construct IR from classes of the
    third-party emmy-ml package, absent offline; oracle/emmy_standin stands in for those classes, so the statement
    structure is the reference's and the spelling of a node is the stand-in's dataclass repr (the same spelling as
    in the IR files the reference committed).
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
    sys.path.insert(0, str(HERE.parent.parent))
    from oracle import build_ref
    sys.path.insert(0, str(Path(build_ref.__file__).resolve().parent / 'emmy_standin'))
    sys.path.insert(0, str(reference))
    examples = {}
    attention = build_ref._example_module(reference, 'attention')
    for name, configuration in build_ref.ATTENTION_CASES.items():
        graph, meta = attention.example(**configuration)
        examples[name] = {'generator': f'examples/attention.py example({configuration})', 'graph': graph, 'meta': meta}
    storage = build_ref._example_module(reference, 'f16_storage')
    for kind in build_ref.F16_KINDS:
        for width in (4, 1):
            graph, meta = storage.example(kind, width=width)
            examples[f'f16_{kind}_w{width}'] = {'generator': f'examples/f16_storage.py example({kind!r}, width={width})', 'graph': graph, 'meta': meta}
    (HERE / 'reference_examples.json').write_text(json.dumps(examples, indent=1) + '\n')
    print('wrote', sorted(p.name for p in HERE.iterdir()))


if __name__ == '__main__':
    import os
    where = sys.argv[1] if len(sys.argv) > 1 else os.environ.get('DEUTERON_REFERENCE')
    if not where:
        raise SystemExit('usage: make_golden.py /path/to/deuteron (or set DEUTERON_REFERENCE)')
    main(Path(where))
