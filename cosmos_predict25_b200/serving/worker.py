"""Worker side of the serving pool.

Parity target: ``ModelWorker`` / ``worker_main`` (packages/cosmos-gradio/cosmos_gradio/model_ipc/model_worker.py:30-150).
A worker builds its pipeline with the factory named in ``FACTORY_MODULE`` / ``FACTORY_FUNCTION``, reports readiness, then
loops: wait for a command, run ``infer`` (every rank runs the same request: the pipelines are context-parallel), report
the result or the traceback. ``shutdown`` ends the loop.
"""

from __future__ import annotations

import importlib
import os
import traceback
from abc import ABC, abstractmethod

from ..utils import log
from .ipc import WorkerCommand, WorkerStatus


class ModelWorker(ABC):
    """Load checkpoints in ``__init__``; ``infer(args)`` handles one request and returns a json-serialisable dict."""

    @abstractmethod
    def infer(self, args: dict) -> dict: ...


class EchoWorker(ModelWorker):
    """Used by tests and as a template: returns its arguments and its rank."""

    def infer(self, args: dict) -> dict:
        if args.get("fail"):
            raise RuntimeError("requested failure")
        return {"echo": args, "rank": int(os.environ.get("LOCAL_RANK", 0)), "world_size": int(os.environ.get("WORLD_SIZE", 1))}


def create_worker() -> ModelWorker:
    return EchoWorker()


def create_worker_pipeline(factory_module: str, factory_function: str) -> ModelWorker:
    module = importlib.import_module(factory_module)
    return getattr(module, factory_function)()


def worker_main():
    rank = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    cmd, status = WorkerCommand(world), WorkerStatus(world)
    pipeline = None
    try:
        pipeline = create_worker_pipeline(os.environ.get("FACTORY_MODULE", __name__), os.environ.get("FACTORY_FUNCTION", "create_worker"))
        status.signal_status(rank, "success", "Worker initialized successfully")
        while True:
            try:
                data = cmd.wait_for_command(rank)
                command, params = data.get("command"), data.get("params", {})
                if command == "inference":
                    status.signal_status(rank, "success", pipeline.infer(params))
                elif command == "shutdown":
                    break
                else:
                    status.signal_status(rank, "error", f"Unknown command: {command}")
            except Exception as e:
                log.error(f"worker {rank}: {e}\n{traceback.format_exc()}")
                status.signal_status(rank, "error", f"{e}\n{traceback.format_exc()}")
    except Exception as e:
        log.error(f"worker {rank} failed to initialise: {e}\n{traceback.format_exc()}")
        status.signal_status(rank, "error", f"{e}\n{traceback.format_exc()}")
    finally:
        del pipeline
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    worker_main()
