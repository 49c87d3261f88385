"""Thin object-store client: typed save/load of Python objects under a bucket prefix.

Parity target: ``ObjectStore`` (cosmos_predict2/_src/imaginaire/utils/object_store.py:54-470): ``save_object`` /
``load_object`` with a ``type`` in {torch, pickle, json, image, video, numpy, text, bytes}, ``object_exists``, and a
context manager that retries transient failures. It sits on the unified file API, so the same code writes to a local
directory (tests, single box) or to S3.
"""

from __future__ import annotations

import time
from typing import Any, Optional

from . import log
from .easy_io import easy_io

_FORMAT = {"torch": "pt", "pickle": "pkl", "json": "json", "numpy": "npy", "image": "png", "video": "mp4", "text": "txt", "bytes": "bin",
           "yaml": "yaml"}


class ObjectStore:
    def __init__(self, bucket: str = "", credentials: Optional[str] = None, root: Optional[str] = None, max_retries: int = 3,
                 retry_wait_s: float = 1.0):
        """``root`` (a local directory) takes precedence; otherwise objects live under ``s3://<bucket>/``."""
        self.root = root.rstrip("/") if root else f"s3://{bucket}"
        self.backend_args = None
        if root is None:
            self.backend_args = {"backend": "s3", "s3_credential_path": credentials}
        self.max_retries, self.retry_wait_s = max_retries, retry_wait_s

    def _path(self, key: str) -> str:
        return f"{self.root}/{key.lstrip('/')}"

    def _retry(self, fn):
        last = None
        for attempt in range(self.max_retries):
            try:
                return fn()
            except (OSError, ConnectionError, TimeoutError) as e:   # transient
                last = e
                log.warning(f"object store attempt {attempt + 1}/{self.max_retries} failed: {e}")
                time.sleep(self.retry_wait_s * (attempt + 1))
        raise last

    def save_object(self, obj: Any, key: str, type: str = "torch", **kwargs) -> None:
        fmt = _FORMAT[type]
        self._retry(lambda: easy_io.dump(obj, self._path(key), file_format=fmt, backend_args=self.backend_args, **kwargs))

    def load_object(self, key: str, type: str = "torch", **kwargs) -> Any:
        fmt = _FORMAT[type]
        return self._retry(lambda: easy_io.load(self._path(key), file_format=fmt, backend_args=self.backend_args, **kwargs))

    def object_exists(self, key: str) -> bool:
        return easy_io.exists(self._path(key), backend_args=self.backend_args)

    def delete_object(self, key: str) -> None:
        easy_io.remove(self._path(key), backend_args=self.backend_args)

    def list_objects(self, prefix: str = "", suffix: Optional[str] = None, recursive: bool = True):
        return list(easy_io.list_dir_or_file(self._path(prefix), list_dir=False, list_file=True, suffix=suffix, recursive=recursive,
                                             backend_args=self.backend_args))
