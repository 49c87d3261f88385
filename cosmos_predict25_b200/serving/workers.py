"""Worker factories for the shipped pipelines (the ``factory_module`` / ``factory_function`` of ``ModelServer``).

Parity target: the per-model ``create_worker`` factories the reference's gradio apps pass to ``GradioApp``
(cosmos_predict2/gradio/*). A request is the json form of the public ``InferenceArguments`` of the pipeline.
"""

from __future__ import annotations

import os

from .worker import ModelWorker


class Video2WorldWorker(ModelWorker):
    def __init__(self):
        from ..config import SetupArguments
        from ..inference import Inference
        out = os.environ.get("COSMOS_OUTPUT_DIR", "outputs/serving")
        kw = {"output_dir": out}
        for env, key in (("COSMOS_MODEL", "model"), ("COSMOS_EXPERIMENT", "experiment"), ("COSMOS_CHECKPOINT", "checkpoint_path")):
            if os.environ.get(env):
                kw[key] = os.environ[env]
        if os.environ.get("COSMOS_DISABLE_GUARDRAILS", "0") == "1":
            kw["disable_guardrails"] = True
        self.setup = SetupArguments(**kw)
        self.pipe = Inference(self.setup)

    def infer(self, args: dict) -> dict:
        from ..config import InferenceArguments
        sample = InferenceArguments(**args)
        paths = self.pipe.generate([sample], self.setup.output_dir)
        return {"videos": [str(p) for p in paths], "message": "done"}


def create_video2world_worker() -> ModelWorker:
    return Video2WorldWorker()


class MultiviewWorker(ModelWorker):
    def __init__(self):
        from ..multiview import MultiviewInference
        from ..multiview_config import MultiviewSetupArguments
        self.setup = MultiviewSetupArguments(output_dir=os.environ.get("COSMOS_OUTPUT_DIR", "outputs/serving"))
        self.pipe = MultiviewInference(self.setup)

    def infer(self, args: dict) -> dict:
        from ..multiview_config import MultiviewInferenceArguments
        return {"videos": self.pipe.generate(MultiviewInferenceArguments(**args)), "message": "done"}


def create_multiview_worker() -> ModelWorker:
    return MultiviewWorker()
