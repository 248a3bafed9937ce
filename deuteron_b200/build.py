"""compile_kernel: the reference's compile surface (compiler/build.py:78-149) over native kernels.

The reference lowers scheduled Kernel IR to PTX text. Here the same inputs (IR JSON + sibling
meta.json, target, optimisation level, Options) are parsed and validated the same way and then
*classified*: the result names the hand-written sm_100a kernel in libdeuteron_b200.so that computes
the workload, together with the buffer roles taken from meta.json's arg_order. `Compilation.ptx`
keeps its place in the interface but holds a short textual description of that selection (there is
no PTX text to JIT); `Compilation.plan` is what the runner launches.
"""
from __future__ import annotations

import hashlib
import json
import os
import threading
from collections import OrderedDict
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

from . import cache
from .classify import Plan, classify
from .options import Options
from .validation import parse_kernel, validate_compile_arguments, validate_launch


@dataclass(frozen=True)
class Compilation:
    """Mirror of compiler/build.py:23-27 plus the native plan and the launch it was compiled for."""
    ptx: str
    unoptimized: str
    optimized: str
    plan: Plan = field(compare=False, default=None)
    launch: dict = field(compare=False, default=None)
    arch: str = 'sm_100a'


_COMPILE_LOCK = threading.RLock()
_CACHE: 'OrderedDict[str, Compilation]' = OrderedDict()
_CACHE_ENTRIES = 128


def clear_cache() -> None:
    with _COMPILE_LOCK:
        _CACHE.clear()


def _payloads(source: Any, meta: Any) -> tuple[bytes, bytes]:
    """IR and meta as bytes. `source` is a path (meta.json beside it), JSON text/bytes or a dict."""
    if isinstance(source, (str, os.PathLike)) and not (isinstance(source, str) and source.lstrip().startswith('{')):
        path = Path(source)
        payload = path.read_bytes()
        meta_payload = path.with_name('meta.json').read_bytes() if meta is None else None
    else:
        payload = json.dumps(source).encode() if isinstance(source, dict) else (source.encode() if isinstance(source, str) else bytes(source))
        meta_payload = None
        if meta is None:
            raise ValueError('an IR object needs its meta.json object as the second argument')
    if meta_payload is None:
        if isinstance(meta, (str, os.PathLike)) and not (isinstance(meta, str) and meta.lstrip().startswith('{')):
            meta_payload = Path(meta).read_bytes()
        else:
            meta_payload = json.dumps(meta).encode() if isinstance(meta, dict) else (meta.encode() if isinstance(meta, str) else bytes(meta))
    return payload, meta_payload


def compile_kernel(source: Any, meta: Any = None, *, arch: Any = 'sm_100a', opt_level: int = 2,
                   options: Options | None = None) -> Compilation:
    """Validates the scheduled kernel and selects its native implementation.

    Raises ValueError for malformed input or options, NotImplementedError for schedules outside the
    native subset and OSError for unreadable paths, like the reference. Thread-safe and cached on the
    hash of (IR, meta, arch, opt_level, options) as compiler/build.py:89-97 does.
    """
    with _COMPILE_LOCK:
        options = validate_compile_arguments(arch, opt_level, options)
        payload, meta_payload = _payloads(source, meta)
        digest = hashlib.sha256()
        for part in (payload, meta_payload, arch.encode(), bytes((opt_level,)), repr(sorted(options.__dict__.items())).encode()):
            digest.update(len(part).to_bytes(8, 'big'))
            digest.update(part)
        key = digest.hexdigest()
        hit = _CACHE.get(key)
        if hit is not None:
            _CACHE.move_to_end(key)
            return hit
        root = os.environ.get('DEUTERON_CACHE')   # directory of on-disk records (compiler/build.py:99-104)
        stored = cache.read(root, key)
        if stored is not None:
            plan = Plan(stored['kind'], stored['params'], {role: (name, offset) for role, (name, offset) in stored['buffers'].items()})
            result = Compilation(ptx=stored['text'], unoptimized=stored['text'], optimized=stored['text'], plan=plan,
                                 launch=stored['launch'], arch=stored['arch'])
        else:
            kernel, launch = parse_kernel(payload, meta_payload)
            specs = validate_launch(launch)
            plan = classify(kernel, launch, specs, options.contraction_precision)
            description = (f'// deuteron_b200 native kernel selection for entry {kernel.name}\n'
                           f'// target {arch}, opt_level {opt_level}\n// {plan.describe()}\n')
            result = Compilation(ptx=description, unoptimized=description, optimized=description, plan=plan,
                                 launch=json.loads(json.dumps(launch)), arch=arch)
            cache.write(root, key, {'text': description, 'kind': plan.kind, 'params': json.loads(json.dumps(plan.params)),
                                    'buffers': {role: [name, offset] for role, (name, offset) in plan.buffers.items()},
                                    'launch': result.launch, 'arch': arch})
        _CACHE[key] = result
        if len(_CACHE) > _CACHE_ENTRIES:
            _CACHE.popitem(last=False)
        return result


def compile_many(jobs: Any, workers: int | None = None) -> list[Compilation]:
    """compiler/build.py:59-76: a list of (source, arch, opt_level, options) jobs. Classification is
    cheap, so the jobs run in this process whatever `workers` says."""
    if workers is not None and (type(workers) is not int or workers < 1):
        raise ValueError('workers must be a positive integer or None')
    try:
        jobs = list(jobs)
    except TypeError as exc:
        raise ValueError('jobs must be an iterable of (path, arch, opt_level, options)') from exc
    for index, job in enumerate(jobs):
        if not isinstance(job, (tuple, list)) or len(job) != 4:
            raise ValueError(f'job {index}: expected (path, arch, opt_level, options)')
    return [compile_kernel(path, arch=arch, opt_level=opt_level, options=options) for path, arch, opt_level, options in jobs]
