"""Serving: a long-lived pool of model workers (one process per GPU, launched with torchrun) driven by a front-end
process through file-based command / status channels, plus an HTTP front-end."""

from .ipc import WorkerCommand, WorkerException, WorkerStatus  # noqa: F401
from .server import ModelServer  # noqa: F401
from .worker import ModelWorker, worker_main  # noqa: F401
