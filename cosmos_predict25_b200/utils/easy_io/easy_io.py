"""Unified file API: one set of functions for local paths, ``s3://`` objects and ``http(s)://`` URLs, plus
format-aware ``load`` / ``dump``.

Parity target: cosmos_predict2/_src/imaginaire/utils/easy_io/easy_io.py:30-1086 (same function names and arguments:
``set_s3_backend``, ``get_file_backend``, ``get``, ``get_text``, ``put``, ``put_text``, ``exists``, ``isdir``, ``isfile``,
``join_path``, ``get_local_path``, ``copyfile*``, ``copytree*``, ``remove``, ``rmtree``, ``copy_if_symlink_fails``, ``list_dir``,
``list_dir_or_file``, ``generate_presigned_url``, ``load``, ``dump``).
"""

from __future__ import annotations

import json
from contextlib import contextmanager
from io import BytesIO, StringIO
from pathlib import Path
from typing import Any, Generator, Iterator, Optional, Tuple, Union

from .backends import BaseStorageBackend, backends, prefix_to_backends
from .handlers import BaseFileHandler, file_handlers

backend_instances: dict = {}


def is_filepath(filepath) -> bool:
    return isinstance(filepath, (str, Path))


def _parse_uri_prefix(uri: Union[str, Path]) -> str:
    assert is_filepath(uri)
    uri = str(uri)
    if "://" not in uri:
        return ""
    prefix, _ = uri.split("://", 1)
    return prefix.split(":")[-1] if ":" in prefix else prefix      # e.g. "clusterName:s3://path"


def _get_file_backend(prefix: str, backend_args: dict):
    if "backend" in backend_args:
        args = dict(backend_args)
        return backends[args.pop("backend")](**args)
    return prefix_to_backends[prefix](**backend_args)


def set_s3_backend(backend_args: Optional[dict] = None, backend_key: str = "s3", path_mapping: Optional[dict] = None,
                   s3_credential_path: Optional[str] = None):
    """Install the default S3 backend used for ``s3://`` paths when no ``backend_args`` are given."""
    args = dict(backend_args or {})
    args.setdefault("backend", "s3")
    if path_mapping is not None:
        args["path_mapping"] = path_mapping
    if s3_credential_path is not None:
        args["s3_credential_path"] = s3_credential_path
    backend_instances[backend_key] = _get_file_backend("s3", args)
    return backend_instances[backend_key]


def get_file_backend(uri: Union[str, Path, None] = None, *, backend_args: Optional[dict] = None, enable_singleton: bool = False,
                     backend_key: Optional[str] = None) -> BaseStorageBackend:
    if backend_key is not None and backend_key in backend_instances:
        return backend_instances[backend_key]
    if backend_args is None:
        backend_args = {}
    if uri is None and "backend" not in backend_args and backend_key is None:
        raise ValueError('uri should not be None when "backend" does not exist in backend_args and backend_key is None')
    prefix = _parse_uri_prefix(uri) if uri is not None else ""
    if prefix == "s3" and not backend_args and "s3" in backend_instances:
        return backend_instances["s3"]
    if enable_singleton:
        key = f"{prefix}:{json.dumps(backend_args, sort_keys=True, default=str)}"
        if key not in backend_instances:
            backend_instances[key] = _get_file_backend(prefix, backend_args)
        return backend_instances[key]
    return _get_file_backend(prefix, backend_args)


def _b(filepath, backend_args, backend_key=None):
    return get_file_backend(filepath, backend_args=backend_args, enable_singleton=True, backend_key=backend_key)


def get(filepath, backend_args=None, backend_key=None) -> bytes:
    return _b(filepath, backend_args, backend_key).get(filepath)


def get_text(filepath, encoding="utf-8", backend_args=None, backend_key=None) -> str:
    return _b(filepath, backend_args, backend_key).get_text(filepath, encoding)


def put(obj, filepath, backend_args=None, backend_key=None) -> None:
    _b(filepath, backend_args, backend_key).put(obj, filepath)


def put_text(obj: str, filepath, backend_args=None, backend_key=None) -> None:
    _b(filepath, backend_args, backend_key).put_text(obj, filepath)


def exists(filepath, backend_args=None, backend_key=None) -> bool:
    return _b(filepath, backend_args, backend_key).exists(filepath)


def isdir(filepath, backend_args=None, backend_key=None) -> bool:
    return _b(filepath, backend_args, backend_key).isdir(filepath)


def isfile(filepath, backend_args=None, backend_key=None) -> bool:
    return _b(filepath, backend_args, backend_key).isfile(filepath)


def join_path(filepath, *filepaths, backend_args=None, backend_key=None):
    return _b(filepath, backend_args, backend_key).join_path(filepath, *filepaths)


@contextmanager
def get_local_path(filepath, backend_args=None, backend_key=None) -> Generator[str, None, None]:
    with _b(filepath, backend_args, backend_key).get_local_path(str(filepath)) as p:
        yield p


def copyfile(src, dst, backend_args=None, backend_key=None):
    return _b(src, backend_args, backend_key).copyfile(src, dst)


def copytree(src, dst, backend_args=None, backend_key=None):
    return _b(src, backend_args, backend_key).copytree(src, dst)


def copyfile_from_local(src, dst, backend_args=None, backend_key=None):
    return _b(dst, backend_args, backend_key).copyfile_from_local(src, dst)


def copytree_from_local(src, dst, backend_args=None, backend_key=None):
    return _b(dst, backend_args, backend_key).copytree_from_local(src, dst)


def copyfile_to_local(src, dst, dst_type: str = "file", backend_args=None, backend_key=None):
    return _b(src, backend_args, backend_key).copyfile_to_local(src, dst)


def copytree_to_local(src, dst, backend_args=None, backend_key=None):
    return _b(src, backend_args, backend_key).copytree_to_local(src, dst)


def remove(filepath, backend_args=None, backend_key=None) -> None:
    _b(filepath, backend_args, backend_key).remove(filepath)


def rmtree(dir_path, backend_args=None, backend_key=None) -> None:
    _b(dir_path, backend_args, backend_key).rmtree(dir_path)


def copy_if_symlink_fails(src, dst, backend_args=None, backend_key=None) -> bool:
    return _b(src, backend_args, backend_key).copy_if_symlink_fails(src, dst)


def list_dir(dir_path, backend_args=None, backend_key=None):
    return _b(dir_path, backend_args, backend_key).list_dir(dir_path)


def list_dir_or_file(dir_path, list_dir: bool = True, list_file: bool = True, suffix=None, recursive: bool = False, backend_args=None,
                     backend_key=None) -> Iterator[str]:
    yield from _b(dir_path, backend_args, backend_key).list_dir_or_file(dir_path, list_dir, list_file, suffix, recursive)


def generate_presigned_url(url: str, client_method: str = "get_object", expires_in: int = 3600, backend_args=None, backend_key=None) -> str:
    return _b(url, backend_args, backend_key).generate_presigned_url(url, client_method, expires_in)


def _handler(file, file_format) -> Tuple[str, BaseFileHandler]:
    if isinstance(file, Path):
        file = str(file)
    if file_format is None and isinstance(file, str):
        file_format = file.split(".")[-1].lower()
    if file_format not in file_handlers:
        raise TypeError(f"Unsupported format: {file_format}")
    return file_format, file_handlers[file_format]


def load(file, file_format: Optional[str] = None, file_client_args=None, fast_backend: bool = False, backend_args=None, backend_key=None,
         **kwargs) -> Any:
    """Load ``file`` (a path / URI or an open file object) with the handler of its extension or of ``file_format``."""
    backend_args = backend_args if backend_args is not None else file_client_args
    _, handler = _handler(file, file_format)
    if is_filepath(file):
        backend = _b(str(file), backend_args, backend_key)
        if handler.str_like:
            with StringIO(backend.get_text(str(file))) as f:
                return handler.load_from_fileobj(f, **kwargs)
        with BytesIO(backend.get(str(file))) as f:
            return handler.load_from_fileobj(f, **kwargs)
    if hasattr(file, "read"):
        return handler.load_from_fileobj(file, **kwargs)
    raise TypeError('"file" must be a filepath str or a file-object')


def dump(obj, file=None, file_format: Optional[str] = None, file_client_args=None, fast_backend: bool = False, backend_args=None,
         backend_key=None, **kwargs):
    """Dump ``obj`` to a path / URI / file object, or return it as a string when ``file`` is None."""
    backend_args = backend_args if backend_args is not None else file_client_args
    if file is None and file_format is None:
        raise ValueError("file_format must be specified since file is None")
    _, handler = _handler(file, file_format)
    if file is None:
        return handler.dump_to_str(obj, **kwargs)
    if is_filepath(file):
        backend = _b(str(file), backend_args, backend_key)
        if handler.str_like:
            with StringIO() as f:
                handler.dump_to_fileobj(obj, f, **kwargs)
                backend.put_text(f.getvalue(), str(file))
        else:
            with BytesIO() as f:
                handler.dump_to_fileobj(obj, f, **kwargs)
                backend.put(f.getvalue(), str(file))
        return None
    if hasattr(file, "write"):
        handler.dump_to_fileobj(obj, file, **kwargs)
        return None
    raise TypeError('"file" must be a filename str or a file-object')
