"""On-disk records of compile results, the counterpart of compiler/cache.py.

The reference keeps (ptx, unoptimized, optimized) under DEUTERON_CACHE as `<key>.json`, written
atomically and re-validated on every read so that a damaged or foreign file is ignored rather than
trusted (compiler/cache.py:34-54, 89-128). The record here holds what a native compile produces: the
selection text and the plan (kernel kind, parameters, buffer roles) with the launch it was made for.
Keys are the SHA-256 of (IR, meta, arch, opt_level, options), as in compiler/build.py:89-97.
"""
from __future__ import annotations

import hashlib
import json
import os
import re
import tempfile
from pathlib import Path
from typing import Any

VERSION = 1
MAX_RECORD_BYTES = 64 * 1024 * 1024
_KEY = re.compile(r'[0-9a-f]{64}')
_FIELDS = ('text', 'kind', 'params', 'buffers', 'launch', 'arch')


def _encode(record: dict) -> bytes:
    return json.dumps(record, sort_keys=True, separators=(',', ':')).encode('utf-8')


def _valid(payload: dict) -> bool:
    return (type(payload.get('text')) is str and payload['text'] != '' and type(payload.get('kind')) is str
            and type(payload.get('params')) is dict and type(payload.get('buffers')) is dict
            and all(type(v) is list and len(v) == 2 and type(v[0]) is str and type(v[1]) is int for v in payload['buffers'].values())
            and type(payload.get('launch')) is dict and type(payload.get('arch')) is str)


def read(root: str | None, key: str) -> dict | None:
    """The record stored for `key` under `root`, or None when it is absent, oversized, damaged, of another
    version or stored under another key."""
    if not root or not _KEY.fullmatch(key):
        return None
    try:
        with (Path(root) / (key + '.json')).open('rb') as stream:
            raw = stream.read(MAX_RECORD_BYTES + 1)
        if len(raw) > MAX_RECORD_BYTES:
            return None
        data = json.loads(raw)
    except (OSError, ValueError, TypeError, RecursionError):
        return None
    if type(data) is not dict or set(data) != {'version', 'key', 'sha256', *_FIELDS}:
        return None
    if type(data['version']) is not int or data['version'] != VERSION or data['key'] != key:
        return None
    payload = {name: value for name, value in data.items() if name != 'sha256'}
    if not _valid(payload) or type(data['sha256']) is not str or hashlib.sha256(_encode(payload)).hexdigest() != data['sha256']:
        return None
    return payload


def write(root: str | None, key: str, payload: dict[str, Any]) -> None:
    """Stores `payload` (the _FIELDS) for `key`: temporary file in the same directory, then an atomic replace.
    Failures to write are not errors (the cache is an optimisation), as in compiler/cache.py:124-125."""
    if not root or not _KEY.fullmatch(key):
        return
    record = {'version': VERSION, 'key': key, **{name: payload[name] for name in _FIELDS}}
    if not _valid(record):
        return
    temporary: str | None = None
    try:
        data = _encode({**record, 'sha256': hashlib.sha256(_encode(record)).hexdigest()})
        if len(data) > MAX_RECORD_BYTES:
            return
        directory = Path(root)
        directory.mkdir(parents=True, exist_ok=True)
        with tempfile.NamedTemporaryFile(mode='wb', prefix='.' + key + '.', suffix='.tmp', dir=directory, delete=False) as stream:
            temporary = stream.name
            stream.write(data)
        os.replace(temporary, directory / (key + '.json'))
        temporary = None
    except (OSError, ValueError, TypeError):
        pass
    finally:
        if temporary is not None:
            try:
                os.unlink(temporary)
            except OSError:
                pass
