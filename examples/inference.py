"""``python examples/inference.py PARAMS.json OUTPUT_DIR [--model 2B/post-trained] [--checkpoint-path P] [--experiment E]
[--context-parallel-size N] [--disable-guardrails]`` (or under torchrun for context parallelism). Parity:
examples/inference.py:25-53 of the reference."""

import argparse
import os
import sys
from pathlib import Path

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from cosmos_predict25_b200.config import InferenceArguments, SetupArguments, init_script  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("params_file", type=Path)
    ap.add_argument("output_dir", type=Path)
    ap.add_argument("--model", default="2B/post-trained")
    ap.add_argument("--checkpoint-path", default=None)
    ap.add_argument("--experiment", default=None)
    ap.add_argument("--context-parallel-size", type=int, default=None)
    ap.add_argument("--disable-guardrails", action="store_true")
    ap.add_argument("--offload-guardrail-models", action="store_true")
    a = ap.parse_args()
    init_script()
    from cosmos_predict25_b200.inference import Inference
    setup = SetupArguments(output_dir=a.output_dir, model=a.model, checkpoint_path=a.checkpoint_path, experiment=a.experiment,
                           context_parallel_size=a.context_parallel_size, disable_guardrails=a.disable_guardrails,
                           offload_guardrail_models=a.offload_guardrail_models)
    args = InferenceArguments.from_file(a.params_file)
    inference = Inference(setup)
    inference.generate(args, a.output_dir)
    inference.cleanup()


if __name__ == "__main__":
    main()
