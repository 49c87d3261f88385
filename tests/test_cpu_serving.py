"""Serving: IPC channels, worker pool via torchrun (CPU echo workers), HTTP front-end handlers."""
import json
import os
import threading

import pytest

from cosmos_predict25_b200.serving import ModelServer, WorkerCommand, WorkerException, WorkerStatus
from cosmos_predict25_b200.serving.app import ServingApp, get_outputs, tail_log


def test_ipc_channels(tmp_path):
    cmd, st = WorkerCommand(2, str(tmp_path)), WorkerStatus(2, str(tmp_path))
    cmd.broadcast("inference", {"a": 1})
    assert cmd.wait_for_command(1, timeout=1) == {"command": "inference", "params": {"a": 1}}
    assert not os.path.exists(tmp_path / "worker_1_commands.json")          # consumed
    assert cmd.wait_for_command(1, timeout=0.2) is None
    st.signal_status(0, "success", {"x": 1})
    st.signal_status(1, "error", "boom")
    with pytest.raises(WorkerException) as e:
        st.wait_for_status(timeout=1)
    assert "boom" in str(e.value)
    st.signal_status(0, "success", {"x": 1})
    with pytest.raises(WorkerException):                                     # rank 1 never answers -> timeout status
        st.wait_for_status(timeout=0.3)
    # late writer thread: the reader blocks until the file appears
    threading.Timer(0.2, lambda: [st.signal_status(r, "success", {"r": r}) for r in (0, 1)]).start()
    assert st.wait_for_status(timeout=5)["result"] == {"r": 0}


@pytest.mark.timeout(180)
def test_model_server_two_cpu_workers(tmp_path):
    with ModelServer(2, ipc_directory=str(tmp_path), master_port=29683, startup_timeout=120) as server:
        r = server.infer({"prompt": "hello", "seed": 3}, timeout=60)
        assert r["status"] == "success" and r["result"]["echo"] == {"prompt": "hello", "seed": 3} and r["result"]["world_size"] == 2
        with pytest.raises(WorkerException):
            server.infer({"fail": True}, timeout=60)
        assert server.infer({"again": 1}, timeout=60)["status"] == "success"   # workers survive a failed request
        proc = server.process
    assert proc.poll() is not None or proc.wait(timeout=20) is not None


def test_serving_app_handlers(tmp_path):
    class FakeServer:
        num_workers, process = 1, None

        def infer(self, args):
            open(os.path.join(args["output_dir"], "out.mp4"), "wb").write(b"x")
            return {"status": "success", "result": {"message": "done"}}

    def validator(a):
        if "prompt" not in a:
            raise ValueError("prompt is required")
        return a

    log_file = tmp_path / "log.txt"
    log_file.write_text("\n".join(f"line {i}" for i in range(300)))
    app = ServingApp(FakeServer(), validator, str(tmp_path / "out"), str(tmp_path / "up"), str(log_file))
    assert app.infer("{bad json")["status"] == "error"
    assert "prompt is required" in app.infer({})["message"]
    r = app.infer(json.dumps({"prompt": "p"}))
    assert r["status"] == "success" and len(r["videos"]) == 1 and get_outputs(r["output_folder"])["videos"] == r["videos"]
    p = app.save_upload("../../evil.png", b"123")
    assert os.path.dirname(os.path.dirname(p)) == str(tmp_path / "up") and os.path.basename(p) == "evil.png"
    rel = os.path.relpath(r["videos"][0], str(tmp_path / "out"))
    assert app.resolve_file(rel) == os.path.realpath(r["videos"][0])
    assert app.resolve_file("../log.txt") is None                            # no escape from the served directories
    assert tail_log(str(log_file), 3).splitlines() == ["line 297", "line 298", "line 299"]
    from fastapi.testclient import TestClient
    try:
        client = TestClient(app.fastapi())
    except Exception:
        pytest.skip("starlette test client unavailable (httpx missing)")
    assert client.post("/infer", json={"prompt": "q"}).json()["status"] == "success"
    assert client.get("/files/" + rel).content == b"x" and client.get("/files/../log.txt").status_code == 404
