"""File-based command / status channels between the serving front-end and its workers.

Parity target: ``WorkerCommand`` / ``WorkerStatus`` / ``WorkerException``
(packages/cosmos-gradio/cosmos_gradio/model_ipc/command_ipc.py:25-160): one json file per worker and direction,
``<dir>/worker_<rank>_commands.json`` and ``<dir>/worker_<rank>_status.json``; the reader polls for the file, parses it and
deletes it, which makes every exchange a blocking rendezvous. Files are written to a temporary name and renamed, so a
reader never sees a partially written message. The directory defaults to ``/tmp`` (``COSMOS_IPC_DIR`` overrides it so
several servers can share a machine).
"""

from __future__ import annotations

import json
import os
import time
from typing import Any, Dict, Optional

from ..utils import log

POLL_S = 0.1


def ipc_dir() -> str:
    return os.environ.get("COSMOS_IPC_DIR", "/tmp")


def _atomic_write(path: str, payload: Dict[str, Any]) -> None:
    tmp = f"{path}.{os.getpid()}.tmp"
    with open(tmp, "w") as f:
        json.dump(payload, f)
    os.replace(tmp, path)


class WorkerCommand:
    def __init__(self, num_workers: int, directory: Optional[str] = None):
        self.num_workers, self.dir = num_workers, directory or ipc_dir()

    def _file(self, rank: int) -> str:
        return os.path.join(self.dir, f"worker_{rank}_commands.json")

    def cleanup(self):
        for r in range(self.num_workers):
            if os.path.exists(self._file(r)):
                os.remove(self._file(r))

    def _send_command_to_worker(self, rank: int, command: str, params: Optional[Dict[str, Any]] = None):
        _atomic_write(self._file(rank), {"command": command, "params": params or {}})

    def broadcast(self, task_name: str, task_params: Dict[str, Any]):
        for r in range(self.num_workers):
            self._send_command_to_worker(r, task_name, task_params)

    def wait_for_command(self, rank: int, timeout: Optional[float] = None) -> Optional[Dict[str, Any]]:
        """Blocks until a command arrives (forever by default: a worker idles until a user sends a request)."""
        path, t0 = self._file(rank), time.time()
        while not os.path.exists(path):
            if timeout is not None and time.time() - t0 > timeout:
                return None
            time.sleep(POLL_S)
        with open(path) as f:
            data = json.load(f)
        os.remove(path)
        return data


class WorkerException(Exception):
    def __init__(self, message, status_dict=None):
        super().__init__(message)
        self.details = status_dict or {}

    def __str__(self):
        return f"{super().__str__()}\nexception on worker({self.details.get('rank', 'unknown')}): {self.details.get('result', 'no result json')}"


class WorkerStatus:
    def __init__(self, num_workers: int, directory: Optional[str] = None):
        self.num_workers, self.dir = num_workers, directory or ipc_dir()

    def _file(self, rank: int) -> str:
        return os.path.join(self.dir, f"worker_{rank}_status.json")

    def cleanup(self):
        for r in range(self.num_workers):
            if os.path.exists(self._file(r)):
                os.remove(self._file(r))

    def signal_status(self, rank: int, status: str, results_json) -> None:
        """status: "success" | "error"; results_json: a dict or a message string."""
        _atomic_write(self._file(rank), {"rank": rank, "status": status, "result": results_json})

    def _get_worker_status(self, rank: int, timeout: float = 1800) -> Dict[str, Any]:
        path, t0 = self._file(rank), time.time()
        while not os.path.exists(path):
            if time.time() - t0 > timeout:
                return {"status": "timeout", "rank": rank}
            time.sleep(POLL_S)
        try:
            with open(path) as f:
                status = json.load(f)
            os.remove(path)
            return status
        except Exception:
            log.error(f"failed to read the status file of worker {rank}")
            return {"status": "unknown", "rank": rank}

    def wait_for_status(self, timeout: float = 1800):
        """Blocks until every worker has reported; raises ``WorkerException`` if any did not succeed. Returns rank 0's status."""
        statuses = {r: self._get_worker_status(r, timeout) for r in range(self.num_workers)}
        for r, st in statuses.items():
            if st.get("status") != "success":
                raise WorkerException(f"Worker {r} failed with status: {st.get('status', 'unknown')}", st)
        return statuses[0]
