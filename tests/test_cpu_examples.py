"""The end-to-end post-training example on the offline tiny preset: train, convert, sample, resume skips finished stages."""

import importlib.util
import os
import sys


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def test_posttraining_pipeline_tiny(tmp_path, monkeypatch):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    monkeypatch.setenv("IMAGINAIRE_OUTPUT_ROOT", str(tmp_path / "jobs"))
    monkeypatch.delenv("MAX_ITERS", raising=False)
    mod = _load(os.path.join(root, "examples", "posttraining", "pipeline.py"), "posttraining_pipeline_example")
    pipe = mod.PostTrainingPipeline("tiny", str(tmp_path / "work"), max_iters=2, save_iter=2)
    state = pipe.run(num_steps=2)
    assert all(state[s] for s in mod.STAGES)
    assert os.path.exists(state["converted"]["model"]) and os.path.exists(state["sample"])
    again = mod.PostTrainingPipeline("tiny", str(tmp_path / "work"), max_iters=2, save_iter=2)
    assert again.state["train"] and again.job_dir == state["job_dir"]
    ran = []
    for s in mod.STAGES:
        setattr(again, s, lambda s=s, **k: ran.append(s))
    again.run()
    assert ran == []                                     # everything was marked done: nothing runs again


def test_multiview_example_parses_arguments(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    mod = _load(os.path.join(root, "examples", "multiview.py"), "multiview_example")
    assert callable(mod.main)
