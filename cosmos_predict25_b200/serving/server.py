"""Front-end side of the serving pool.

Parity target: ``ModelServer`` (packages/cosmos-gradio/cosmos_gradio/model_ipc/model_server.py:24-200): start
``num_gpus`` workers with torchrun, block until all report readiness, ``infer`` = broadcast one request and wait for the
compound status, context-manager shutdown (broadcast ``shutdown``, then terminate the launcher).
"""

from __future__ import annotations

import importlib
import os
import subprocess
import sys
import time
from typing import Any, Dict, Optional

from ..utils import log
from .ipc import WorkerCommand, WorkerStatus


class ModelServer:
    def __init__(self, num_gpus: int = 1, factory_module: str = "cosmos_predict25_b200.serving.worker", factory_function: str = "create_worker",
                 ipc_directory: Optional[str] = None, master_port: int = 29571, startup_timeout: float = 1800, shutdown_grace_s: float = 2.0):
        self.num_workers = num_gpus
        self.process: Optional[subprocess.Popen] = None
        self.dir = ipc_directory or os.environ.get("COSMOS_IPC_DIR", "/tmp")
        self.worker_command = WorkerCommand(num_gpus, self.dir)
        self.worker_status = WorkerStatus(num_gpus, self.dir)
        self.master_port, self.startup_timeout, self.shutdown_grace_s = master_port, startup_timeout, shutdown_grace_s
        self.start_workers(num_gpus, factory_module, factory_function)

    def start_workers(self, num_gpus: int, factory_module: str, factory_function: str):
        module = importlib.import_module(factory_module)      # fail early on a wrong factory
        getattr(module, factory_function)
        env = os.environ.copy()
        env.update(FACTORY_MODULE=factory_module, FACTORY_FUNCTION=factory_function, COSMOS_IPC_DIR=self.dir)
        self.worker_command.cleanup()
        self.worker_status.cleanup()
        cmd = [sys.executable, "-m", "torch.distributed.run", f"--nproc-per-node={num_gpus}", "--nnodes=1", "--master-addr", "127.0.0.1",
               "--master-port", str(self.master_port), "-m", "cosmos_predict25_b200.serving.worker"]
        log.info(f"starting {num_gpus} workers: {' '.join(cmd)}")
        try:
            self.process = subprocess.Popen(cmd, env=env, text=True, start_new_session=True)
            self.worker_status.wait_for_status(self.startup_timeout)
        except Exception:
            self.stop_workers()
            raise

    def stop_workers(self):
        self.worker_command.broadcast("shutdown", {})
        if self.process is None:
            return
        t0 = time.time()
        while self.process.poll() is None and time.time() - t0 < self.shutdown_grace_s:
            time.sleep(0.1)
        if self.process.poll() is None:
            self.process.terminate()
            try:
                self.process.wait(timeout=10)
            except subprocess.TimeoutExpired:
                log.warning("the worker launcher did not terminate")
        self.process = None
        self.worker_command.cleanup()
        self.worker_status.cleanup()

    def infer(self, args: Dict[str, Any], timeout: float = 1800) -> Dict[str, Any]:
        self.worker_command.broadcast("inference", args)
        return self.worker_status.wait_for_status(timeout)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.stop_workers()

    def __del__(self):
        try:
            if self.process is not None:
                self.stop_workers()
        except Exception:
            pass
