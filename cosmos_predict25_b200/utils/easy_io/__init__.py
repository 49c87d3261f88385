"""Unified file I/O (local / S3 / HTTP backends, format handlers). Use as ``from ...utils.easy_io import easy_io``."""

from . import easy_io  # noqa: F401
from .backends import BaseStorageBackend, Boto3Backend, HTTPBackend, LocalBackend, register_backend  # noqa: F401
from .handlers import BaseFileHandler, file_handlers, register_handler  # noqa: F401
