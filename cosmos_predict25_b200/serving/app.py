"""HTTP front-end of the serving pool.

Parity target: the gradio application of the reference (packages/cosmos-gradio/cosmos_gradio/gradio_app/{gradio_app,
gradio_file_server,gradio_log_file_viewer,gradio_ui,util}.py and ``gradio_bootstrapper.py:38,51``): validate a json request,
hand it to the ``ModelServer``, return the paths of the generated files, let the user upload inputs into a per-server
directory, browse / download outputs, and read the tail of the log file. gradio is not required: the same functions are
exposed as a FastAPI application, and ``build_gradio_ui`` wraps them in a gradio Blocks UI when gradio is installed.
"""


import json
import os
import time
from datetime import datetime
from typing import Any, Callable, Dict, List, Optional

from ..utils import log
from .server import ModelServer


def get_output_folder(output_dir: str) -> str:
    """A fresh time-stamped sub-folder per request."""
    d = os.path.join(output_dir, f"generation_{datetime.now().strftime('%Y%m%d_%H%M%S_%f')}")
    os.makedirs(d, exist_ok=True)
    return d


def get_outputs(output_folder: str) -> Dict[str, List[str]]:
    vids, imgs = [], []
    for root, _, files in os.walk(output_folder):
        for f in sorted(files):
            p = os.path.join(root, f)
            if f.lower().endswith((".mp4", ".webm", ".mov")):
                vids.append(p)
            elif f.lower().endswith((".png", ".jpg", ".jpeg", ".webp")):
                imgs.append(p)
    return {"videos": vids, "images": imgs}


def tail_log(path: str, num_lines: int = 100) -> str:
    if not os.path.exists(path):
        return f"log file {path} does not exist"
    with open(path, "rb") as f:
        f.seek(0, os.SEEK_END)
        size = f.tell()
        f.seek(max(0, size - 200 * num_lines))
        lines = f.read().decode(errors="replace").splitlines()
    return "\n".join(lines[-num_lines:])


class ServingApp:
    def __init__(self, server: Optional[ModelServer], validator: Optional[Callable[[dict], dict]] = None, output_dir: str = "outputs/serving",
                 uploads_dir: str = "uploads", log_file: Optional[str] = None, default_request: Optional[dict] = None):
        self.server, self.validator = server, validator
        self.output_dir, self.uploads_dir, self.log_file = output_dir, uploads_dir, log_file
        self.default_request = default_request or {}
        os.makedirs(output_dir, exist_ok=True)
        os.makedirs(uploads_dir, exist_ok=True)

    # ---- request handling --------------------------------------------------------------------------------
    def infer(self, request: Any) -> Dict[str, Any]:
        """``request``: a dict or its json text. Returns {"status", "message", "output_folder", "videos", "images"}."""
        try:
            args = json.loads(request) if isinstance(request, str) else dict(request)
        except Exception as e:
            return {"status": "error", "message": f"invalid json: {e}"}
        try:
            if self.validator is not None:
                args = self.validator(args)
        except Exception as e:
            return {"status": "error", "message": f"invalid request: {e}"}
        out = get_output_folder(self.output_dir)
        args = dict(args, output_dir=out)
        t0 = time.time()
        try:
            st = self.server.infer(args)
        except Exception as e:
            log.error(f"inference failed: {e}")
            return {"status": "error", "message": str(e), "output_folder": out}
        res = {"status": "success", "message": st.get("result"), "output_folder": out, "seconds": time.time() - t0}
        res.update(get_outputs(out))
        return res

    def save_upload(self, filename: str, data: bytes) -> str:
        safe = os.path.basename(filename)
        d = os.path.join(self.uploads_dir, f"upload_{datetime.now().strftime('%Y%m%d_%H%M%S')}")
        os.makedirs(d, exist_ok=True)
        p = os.path.join(d, safe)
        with open(p, "wb") as f:
            f.write(data)
        return p

    def resolve_file(self, rel: str) -> Optional[str]:
        """Only files under the output / upload directories are served."""
        for base in (self.output_dir, self.uploads_dir):
            p = os.path.realpath(os.path.join(base, rel))
            if p.startswith(os.path.realpath(base) + os.sep) and os.path.isfile(p):
                return p
        return None

    # ---- FastAPI ---------------------------------------------------------------------------------------------
    def fastapi(self):
        from fastapi import FastAPI, File, HTTPException, Request, UploadFile
        from fastapi.responses import FileResponse, PlainTextResponse
        app = FastAPI(title="cosmos-predict2.5 B200 serving")

        @app.get("/health")
        def health():
            alive = self.server is not None and self.server.process is not None and self.server.process.poll() is None
            return {"workers": getattr(self.server, "num_workers", 0), "alive": alive}

        @app.get("/default_request")
        def default_request():
            return self.default_request

        @app.post("/infer")
        async def infer(req: Request):
            return self.infer(await req.json())

        @app.post("/upload")
        async def upload(file: UploadFile = File(...)):
            return {"path": self.save_upload(file.filename, await file.read())}

        @app.get("/files/{rel:path}")
        def files(rel: str):
            p = self.resolve_file(rel)
            if p is None:
                raise HTTPException(status_code=404, detail="not found")
            return FileResponse(p)

        @app.get("/logs", response_class=PlainTextResponse)
        def logs(lines: int = 100):
            return tail_log(self.log_file, lines) if self.log_file else "no log file configured"

        return app


def build_gradio_ui(app: ServingApp, header: str = "Cosmos-Predict2.5", help_text: str = ""):
    """Blocks UI over the same handlers (requires the optional ``gradio`` package)."""
    try:
        import gradio as gr
    except ImportError as e:
        raise ImportError("`gradio` is not installed; use ServingApp.fastapi() instead") from e
    with gr.Blocks(title=header) as ui:
        gr.Markdown(f"# {header}\n{help_text}")
        req = gr.Textbox(label="request (json)", value=json.dumps(app.default_request, indent=2), lines=12)
        btn = gr.Button("Generate")
        video, status = gr.Video(label="output"), gr.Textbox(label="status", lines=6)

        def run(text):
            r = app.infer(text)
            return (r.get("videos") or [None])[0], json.dumps({k: v for k, v in r.items() if k != "videos"}, indent=2, default=str)

        btn.click(run, inputs=[req], outputs=[video, status])
        if app.log_file:
            logbox = gr.Textbox(label="log", lines=20)
            gr.Button("Refresh log").click(lambda: tail_log(app.log_file), outputs=[logbox])
    return ui


def launch(factory_module: str = "cosmos_predict25_b200.serving.workers", factory_function: str = "create_video2world_worker",
           num_gpus: int = 1, host: str = "0.0.0.0", port: int = 8080, output_dir: str = "outputs/serving", validator=None):
    """Start the worker pool and serve HTTP until interrupted (the bootstrapper of the reference)."""
    import uvicorn
    with ModelServer(num_gpus, factory_module, factory_function) as server:
        uvicorn.run(ServingApp(server, validator, output_dir).fastapi(), host=host, port=port)


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--factory-module", default="cosmos_predict25_b200.serving.workers")
    ap.add_argument("--factory-function", default="create_video2world_worker")
    ap.add_argument("--num-gpus", type=int, default=int(os.environ.get("NUM_GPUS", "1")))
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=8080)
    ap.add_argument("--output-dir", default="outputs/serving")
    a = ap.parse_args()
    launch(a.factory_module, a.factory_function, a.num_gpus, a.host, a.port, a.output_dir)
