"""``python examples/multiview.py PARAMS.json OUTPUT_DIR [--model auto/multiview] [--checkpoint-path P] [--experiment E]
[--context-parallel-size N]`` (or under torchrun): seven-camera driving video generation. Parity: examples/multiview.py:16-53
of the reference."""

import argparse
import os
import sys
from pathlib import Path

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from cosmos_predict25_b200.config import init_script  # noqa: E402
from cosmos_predict25_b200.multiview_config import MultiviewInferenceArguments, MultiviewSetupArguments  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("params_file", type=Path, help="inference parameters (json / yaml)")
    ap.add_argument("output_dir", type=Path)
    ap.add_argument("--model", default=None)
    ap.add_argument("--checkpoint-path", default=None)
    ap.add_argument("--experiment", default=None)
    ap.add_argument("--context-parallel-size", type=int, default=None)
    a = ap.parse_args(argv)
    init_script()
    kw = dict(output_dir=a.output_dir, checkpoint_path=a.checkpoint_path, experiment=a.experiment,
              context_parallel_size=a.context_parallel_size)
    if a.model is not None:
        kw["model"] = a.model
    setup = MultiviewSetupArguments(**kw)
    args = MultiviewInferenceArguments.from_file(a.params_file)
    from cosmos_predict25_b200.multiview import MultiviewInference
    from cosmos_predict25_b200.utils import log
    log.info(f"{setup}")
    log.info(f"{args}")
    return MultiviewInference(setup).generate(args)


if __name__ == "__main__":
    main()
