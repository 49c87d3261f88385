"""Legacy object-style client over the unified file API (parity: .../easy_io/file_client.py ``FileClient``)."""

from __future__ import annotations

from typing import Optional

from . import easy_io


class FileClient:
    def __init__(self, backend: Optional[str] = None, prefix: Optional[str] = None, **kwargs):
        args = dict(kwargs)
        if backend is not None:
            args["backend"] = backend
        uri = f"{prefix}://" if prefix else ""
        self.client = easy_io.get_file_backend(uri or None, backend_args=args if (args or not uri) else None) \
            if (backend or prefix) else easy_io.get_file_backend("", backend_args={})

    @classmethod
    def infer_client(cls, file_client_args: Optional[dict] = None, uri: Optional[str] = None) -> "FileClient":
        if file_client_args:
            return cls(**file_client_args)
        return cls(prefix=easy_io._parse_uri_prefix(uri or "") or None)

    def __getattr__(self, name):
        return getattr(self.client, name)
