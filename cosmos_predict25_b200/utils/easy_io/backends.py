"""Storage backends behind the unified file API: local disk, HTTP(S) (read-only) and S3 through boto3.

Parity targets: ``BaseStorageBackend`` / ``LocalBackend`` / ``HTTPBackend`` / ``Boto3Backend`` and the backend registry
(cosmos_predict2/_src/imaginaire/utils/easy_io/backends/*.py). A backend is chosen by an explicit ``backend`` argument or
by the URI prefix (``s3://`` -> boto3, ``http(s)://`` -> http, anything else -> local).
"""

from __future__ import annotations

import io
import os
import shutil
import tempfile
from abc import ABCMeta, abstractmethod
from contextlib import contextmanager
from pathlib import Path
from typing import Dict, Generator, Iterator, Optional, Tuple, Type, Union

backends: Dict[str, Type["BaseStorageBackend"]] = {}
prefix_to_backends: Dict[str, Type["BaseStorageBackend"]] = {}


def register_backend(name: str, backend=None, force: bool = False, prefixes=None):
    def _reg(cls):
        if not force and name in backends:
            raise ValueError(f"{name} is already registered as a storage backend")
        backends[name] = cls
        for p in ([prefixes] if isinstance(prefixes, str) else (prefixes or [])):
            if p in prefix_to_backends and not force:
                raise ValueError(f"{p} is already registered as a storage backend prefix")
            prefix_to_backends[p] = cls
        return cls
    return _reg(backend) if backend is not None else _reg


class BaseStorageBackend(metaclass=ABCMeta):
    _allow_symlink = False

    @property
    def allow_symlink(self):
        return self._allow_symlink

    @property
    def name(self):
        return self.__class__.__name__

    @abstractmethod
    def get(self, filepath) -> bytes: ...

    @abstractmethod
    def get_text(self, filepath, encoding="utf-8") -> str: ...


@register_backend("local", prefixes="")
class LocalBackend(BaseStorageBackend):
    _allow_symlink = True

    def get(self, filepath) -> bytes:
        with open(filepath, "rb") as f:
            return f.read()

    def get_text(self, filepath, encoding="utf-8") -> str:
        with open(filepath, encoding=encoding) as f:
            return f.read()

    def put(self, obj: Union[bytes, io.IOBase], filepath) -> None:
        os.makedirs(os.path.dirname(os.path.abspath(filepath)), exist_ok=True)
        if isinstance(obj, io.IOBase):
            obj = obj.read()
        with open(filepath, "wb") as f:
            f.write(obj)

    def put_text(self, obj: str, filepath, encoding="utf-8") -> None:
        os.makedirs(os.path.dirname(os.path.abspath(filepath)), exist_ok=True)
        with open(filepath, "w", encoding=encoding) as f:
            f.write(obj)

    def exists(self, filepath) -> bool:
        return os.path.exists(filepath)

    def isdir(self, filepath) -> bool:
        return os.path.isdir(filepath)

    def isfile(self, filepath) -> bool:
        return os.path.isfile(filepath)

    def join_path(self, filepath, *filepaths) -> str:
        return os.path.join(str(filepath), *[str(p) for p in filepaths])

    @contextmanager
    def get_local_path(self, filepath) -> Generator[str, None, None]:
        yield str(filepath)

    def copyfile(self, src, dst) -> str:
        return shutil.copy(src, dst)

    def copytree(self, src, dst) -> str:
        return shutil.copytree(src, dst)

    copyfile_from_local, copytree_from_local, copyfile_to_local, copytree_to_local = copyfile, copytree, copyfile, copytree

    def remove(self, filepath) -> None:
        if not self.exists(filepath):
            raise FileNotFoundError(f"filepath {filepath} does not exist, it could not be removed.")
        if self.isdir(filepath):
            raise IsADirectoryError(f"filepath {filepath} should be a file")
        os.remove(filepath)

    def rmtree(self, dir_path) -> None:
        shutil.rmtree(dir_path)

    def copy_if_symlink_fails(self, src, dst) -> bool:
        try:
            os.symlink(src, dst)
            return True
        except Exception:
            (self.copyfile if self.isfile(src) else self.copytree)(src, dst)
            return False

    def list_dir(self, dir_path) -> Iterator[str]:
        yield from sorted(os.listdir(dir_path))

    def list_dir_or_file(self, dir_path, list_dir=True, list_file=True, suffix=None, recursive=False) -> Iterator[str]:
        if list_dir and suffix is not None:
            raise TypeError("`suffix` should be None when `list_dir` is True")
        root = str(dir_path)

        def walk(d):
            for e in sorted(os.scandir(d), key=lambda e: e.name):
                rel = os.path.relpath(e.path, root)
                if e.is_file() and not e.name.startswith("."):
                    if list_file and (suffix is None or rel.endswith(suffix)):
                        yield rel
                elif e.is_dir():
                    if list_dir:
                        yield rel
                    if recursive:
                        yield from walk(e.path)
        return walk(root)


@register_backend("http", prefixes=["http", "https"])
class HTTPBackend(BaseStorageBackend):
    """Read-only."""

    def get(self, filepath) -> bytes:
        from urllib.request import urlopen
        return urlopen(str(filepath)).read()

    def get_text(self, filepath, encoding="utf-8") -> str:
        return self.get(filepath).decode(encoding)

    @contextmanager
    def get_local_path(self, filepath) -> Generator[str, None, None]:
        f = tempfile.NamedTemporaryFile(delete=False)
        try:
            f.write(self.get(filepath))
            f.close()
            yield f.name
        finally:
            os.remove(f.name)


@register_backend("s3", prefixes=["s3"])
class Boto3Backend(BaseStorageBackend):
    """S3 (or S3-compatible) object store. ``s3_credential_path`` is a json file with ``aws_access_key_id``,
    ``aws_secret_access_key``, ``endpoint_url`` and ``region_name``; ``path_mapping`` rewrites path prefixes first."""

    def __init__(self, s3_credential_path: Optional[str] = None, path_mapping: Optional[dict] = None, client=None):
        self.path_mapping = path_mapping or {}
        if client is not None:
            self._client = client
            return
        try:
            import boto3
        except ImportError as e:
            raise ImportError("the s3 backend needs `boto3`") from e
        import json
        cred = json.load(open(s3_credential_path)) if s3_credential_path and os.path.exists(s3_credential_path) else {}
        self._client = boto3.client("s3", **{k: v for k, v in cred.items() if k in (
            "aws_access_key_id", "aws_secret_access_key", "endpoint_url", "region_name", "aws_session_token")})

    def _split(self, filepath) -> Tuple[str, str]:
        p = str(filepath)
        for k, v in self.path_mapping.items():
            p = p.replace(k, v, 1)
        p = p[len("s3://"):] if p.startswith("s3://") else p
        bucket, _, key = p.partition("/")
        return bucket, key

    def get(self, filepath) -> bytes:
        b, k = self._split(filepath)
        buf = io.BytesIO()
        self._client.download_fileobj(b, k, buf)
        return buf.getvalue()

    def get_text(self, filepath, encoding="utf-8") -> str:
        return self.get(filepath).decode(encoding)

    def put(self, obj, filepath) -> None:
        b, k = self._split(filepath)
        if isinstance(obj, (bytes, bytearray)):
            obj = io.BytesIO(obj)
        self._client.upload_fileobj(obj, b, k)

    def put_text(self, obj: str, filepath, encoding="utf-8") -> None:
        self.put(obj.encode(encoding), filepath)

    def exists(self, filepath) -> bool:
        return self.isfile(filepath) or self.isdir(filepath)

    def isfile(self, filepath) -> bool:
        b, k = self._split(filepath)
        try:
            self._client.head_object(Bucket=b, Key=k)
            return True
        except Exception:
            return False

    def isdir(self, filepath) -> bool:
        b, k = self._split(filepath)
        k = k if k.endswith("/") else k + "/"
        r = self._client.list_objects_v2(Bucket=b, Prefix=k, MaxKeys=1)
        return r.get("KeyCount", 0) > 0

    def join_path(self, filepath, *filepaths) -> str:
        parts = [str(filepath).rstrip("/")] + [str(p).strip("/") for p in filepaths]
        return "/".join(parts)

    @contextmanager
    def get_local_path(self, filepath) -> Generator[str, None, None]:
        f = tempfile.NamedTemporaryFile(delete=False, suffix=Path(str(filepath)).suffix)
        try:
            f.write(self.get(filepath))
            f.close()
            yield f.name
        finally:
            os.remove(f.name)

    def remove(self, filepath) -> None:
        b, k = self._split(filepath)
        self._client.delete_object(Bucket=b, Key=k)

    def copyfile_from_local(self, src, dst) -> str:
        with open(src, "rb") as f:
            self.put(f, dst)
        return str(dst)

    def copyfile_to_local(self, src, dst) -> str:
        os.makedirs(os.path.dirname(os.path.abspath(dst)), exist_ok=True)
        with open(dst, "wb") as f:
            f.write(self.get(src))
        return str(dst)

    def copyfile(self, src, dst) -> str:
        sb, sk = self._split(src)
        db, dk = self._split(dst)
        self._client.copy({"Bucket": sb, "Key": sk}, db, dk)
        return str(dst)

    def list_dir_or_file(self, dir_path, list_dir=True, list_file=True, suffix=None, recursive=False) -> Iterator[str]:
        b, k = self._split(dir_path)
        k = k if (k.endswith("/") or not k) else k + "/"
        pag = self._client.get_paginator("list_objects_v2")
        kw = dict(Bucket=b, Prefix=k)
        if not recursive:
            kw["Delimiter"] = "/"
        for page in pag.paginate(**kw):
            if list_dir:
                for cp in page.get("CommonPrefixes", []):
                    yield cp["Prefix"][len(k):].rstrip("/")
            if list_file:
                for o in page.get("Contents", []):
                    rel = o["Key"][len(k):]
                    if rel and (suffix is None or rel.endswith(suffix)):
                        yield rel

    def list_dir(self, dir_path):
        return self.list_dir_or_file(dir_path)

    def generate_presigned_url(self, url: str, client_method: str = "get_object", expires_in: int = 3600) -> str:
        b, k = self._split(url)
        return self._client.generate_presigned_url(client_method, Params={"Bucket": b, "Key": k}, ExpiresIn=expires_in)
