"""File-format handlers of the unified file API (one per extension family).

Parity target: cosmos_predict2/_src/imaginaire/utils/easy_io/handlers/*.py. A handler turns a file object into a Python
object (``load_from_fileobj``) and back (``dump_to_fileobj`` / ``dump_to_str``); ``str_like`` says whether the file is text.
"""

from __future__ import annotations

import csv
import gzip
import io
import json
import pickle
import tarfile
from typing import Any, Dict

import numpy as np


class BaseFileHandler:
    str_like = True

    def load_from_fileobj(self, file, **kw): raise NotImplementedError
    def dump_to_fileobj(self, obj, file, **kw): raise NotImplementedError

    def dump_to_str(self, obj, **kw):
        raise NotImplementedError(f"{type(self).__name__} cannot dump to a string")


def _np_default(o):
    if isinstance(o, (set, range)):
        return list(o)
    if isinstance(o, np.ndarray):
        return o.tolist()
    if isinstance(o, np.generic):
        return o.item()
    raise TypeError(f"{type(o)} is unsupported for json dump")


class JsonHandler(BaseFileHandler):
    def load_from_fileobj(self, file, **kw): return json.load(file)
    def dump_to_fileobj(self, obj, file, **kw): kw.setdefault("default", _np_default); json.dump(obj, file, **kw)
    def dump_to_str(self, obj, **kw): kw.setdefault("default", _np_default); return json.dumps(obj, **kw)


class JsonlHandler(BaseFileHandler):
    def load_from_fileobj(self, file, **kw): return [json.loads(l) for l in file if l.strip()]
    def dump_to_fileobj(self, obj, file, **kw): file.write(self.dump_to_str(obj, **kw))
    def dump_to_str(self, obj, **kw): return "".join(json.dumps(o, default=_np_default, **kw) + "\n" for o in obj)


class YamlHandler(BaseFileHandler):
    def load_from_fileobj(self, file, **kw):
        import yaml
        return yaml.load(file, Loader=kw.pop("Loader", yaml.SafeLoader))

    def dump_to_fileobj(self, obj, file, **kw):
        import yaml
        yaml.dump(obj, file, Dumper=kw.pop("Dumper", yaml.SafeDumper), **kw)

    def dump_to_str(self, obj, **kw):
        import yaml
        return yaml.dump(obj, Dumper=kw.pop("Dumper", yaml.SafeDumper), **kw)


class PickleHandler(BaseFileHandler):
    str_like = False
    def load_from_fileobj(self, file, **kw): return pickle.load(file, **kw)
    def dump_to_fileobj(self, obj, file, **kw): kw.setdefault("protocol", 2); pickle.dump(obj, file, **kw)
    def dump_to_str(self, obj, **kw): kw.setdefault("protocol", 2); return pickle.dumps(obj, **kw)


class TorchHandler(BaseFileHandler):
    str_like = False

    def load_from_fileobj(self, file, **kw):
        import torch
        kw.setdefault("weights_only", False)
        return torch.load(file, **kw)

    def dump_to_fileobj(self, obj, file, **kw):
        import torch
        torch.save(obj, file, **kw)


class TorchJitHandler(BaseFileHandler):
    str_like = False

    def load_from_fileobj(self, file, **kw):
        import torch
        return torch.jit.load(file, **kw)

    def dump_to_fileobj(self, obj, file, **kw):
        import torch
        torch.jit.save(obj, file, **kw)


class NumpyHandler(BaseFileHandler):
    str_like = False
    def load_from_fileobj(self, file, **kw): return np.load(io.BytesIO(file.read()), allow_pickle=kw.pop("allow_pickle", True), **kw)
    def dump_to_fileobj(self, obj, file, **kw): np.save(file, obj, **kw)


class TxtHandler(BaseFileHandler):
    def load_from_fileobj(self, file, **kw): return file.read()
    def dump_to_fileobj(self, obj, file, **kw): file.write(obj if isinstance(obj, str) else str(obj))
    def dump_to_str(self, obj, **kw): return obj if isinstance(obj, str) else str(obj)


class ByteHandler(BaseFileHandler):
    str_like = False
    def load_from_fileobj(self, file, **kw): return file.read()
    def dump_to_fileobj(self, obj, file, **kw): file.write(obj)


class CsvHandler(BaseFileHandler):
    """Rows as lists of strings, header row included (the reference's convention: csv_handler.py:22-42 there); rows given as
    dicts are written as a header plus values."""

    def load_from_fileobj(self, file, **kw): return list(csv.reader(file))

    def dump_to_fileobj(self, obj, file, **kw):
        rows = list(obj)
        if rows and all(isinstance(r, dict) for r in rows):
            rows = [list(rows[0].keys())] + [list(r.values()) for r in rows]
        if not all(isinstance(r, (list, tuple)) for r in rows):
            raise ValueError("Each row must be a list")
        csv.writer(file).writerows(rows)

    def dump_to_str(self, obj, **kw):
        s = io.StringIO()
        self.dump_to_fileobj(obj, s, **kw)
        return s.getvalue()


class PandasHandler(BaseFileHandler):
    """parquet tables."""
    str_like = False

    def load_from_fileobj(self, file, **kw):
        import pandas as pd
        return pd.read_parquet(io.BytesIO(file.read()), **kw)

    def dump_to_fileobj(self, obj, file, **kw):
        obj.to_parquet(file, **kw)


class GzipHandler(PickleHandler):
    """gzip-compressed pickle."""
    def load_from_fileobj(self, file, **kw): return pickle.loads(gzip.decompress(file.read()), **kw)
    def dump_to_fileobj(self, obj, file, **kw): file.write(gzip.compress(pickle.dumps(obj, **kw)))


class TarHandler(BaseFileHandler):
    """load: an open ``TarFile``; dump: {member name: bytes}."""
    str_like = False

    def load_from_fileobj(self, file, **kw):
        return tarfile.open(fileobj=io.BytesIO(file.read()), mode=kw.pop("mode", "r:*"), **kw)

    def dump_to_fileobj(self, obj: Dict[str, bytes], file, **kw):
        with tarfile.open(fileobj=file, mode=kw.pop("mode", "w")) as tf:
            for name, data in obj.items():
                info = tarfile.TarInfo(name)
                info.size = len(data)
                tf.addfile(info, io.BytesIO(data))


class PILHandler(BaseFileHandler):
    str_like = False
    format = "png"

    def load_from_fileobj(self, file, fmt: str = "pil", size=None, **kw):
        from PIL import Image
        img = Image.open(io.BytesIO(file.read()))
        img.load()
        if size is not None:
            img = img.resize(tuple(size))
        return np.array(img) if fmt in ("np", "npy", "numpy") else img

    def dump_to_fileobj(self, obj, file, **kw):
        from PIL import Image
        if isinstance(obj, np.ndarray):
            obj = Image.fromarray(obj)
        obj.save(file, format=kw.pop("format", self.format), **kw)


class VideoHandler(BaseFileHandler):
    """mp4: load -> (uint8 frames [T,H,W,3], {"fps": ...}); dump <- frames (+ ``fps``), through OpenCV."""
    str_like = False

    def load_from_fileobj(self, file, **kw):
        import os
        import tempfile

        import cv2
        with tempfile.NamedTemporaryFile(suffix=".mp4", delete=False) as f:
            f.write(file.read())
        try:
            cap = cv2.VideoCapture(f.name)
            fps = cap.get(cv2.CAP_PROP_FPS)
            frames = []
            while True:
                ok, fr = cap.read()
                if not ok:
                    break
                frames.append(cv2.cvtColor(fr, cv2.COLOR_BGR2RGB))
            cap.release()
        finally:
            os.unlink(f.name)
        return (np.stack(frames) if frames else np.zeros((0, 0, 0, 3), np.uint8)), {"fps": fps}

    def dump_to_fileobj(self, obj, file, fps: float = 24.0, **kw):
        import os
        import tempfile

        import cv2
        frames = np.asarray(obj)
        with tempfile.NamedTemporaryFile(suffix=".mp4", delete=False) as f:
            name = f.name
        try:
            h, w = frames.shape[1:3]
            wr = cv2.VideoWriter(name, cv2.VideoWriter_fourcc(*"mp4v"), float(fps), (w, h))
            for fr in frames:
                wr.write(cv2.cvtColor(fr, cv2.COLOR_RGB2BGR))
            wr.release()
            file.write(open(name, "rb").read())
        finally:
            os.unlink(name)


file_handlers: Dict[str, BaseFileHandler] = {}


def register_handler(exts, handler: BaseFileHandler):
    for e in ([exts] if isinstance(exts, str) else exts):
        file_handlers[e] = handler


register_handler("json", JsonHandler())
register_handler("jsonl", JsonlHandler())
register_handler(["yaml", "yml"], YamlHandler())
register_handler(["pickle", "pkl"], PickleHandler())
register_handler(["pt", "pth", "ckpt"], TorchHandler())
register_handler("jit", TorchJitHandler())
register_handler(["npy", "npz"], NumpyHandler())
register_handler(["txt", "md"], TxtHandler())
register_handler(["bin", "byte"], ByteHandler())
register_handler("csv", CsvHandler())
register_handler("parquet", PandasHandler())
register_handler("gz", GzipHandler())
register_handler("tar", TarHandler())
for _ext in ("png", "jpg", "jpeg", "bmp", "webp"):
    h = PILHandler()
    h.format = {"jpg": "jpeg"}.get(_ext, _ext)
    register_handler(_ext, h)
register_handler(["mp4", "avi", "mov", "webm"], VideoHandler())
