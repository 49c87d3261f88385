"""Sparse (neighbourhood) self-attention experiments of the Video2World network.

Every block of the DiT either keeps dense self-attention or attends inside a (strided, optionally dilated) neighbourhood of the
44 x 80 token grid of a 720p frame; all frames are always visible. Two families, as in the reference
(cosmos_predict2/_src/predict2/configs/video2world/experiment/resume_text2world/sparse_2B.py and sparse_14B.py):

* uniform: one neighbourhood for all sparse blocks and ``n_dense_blocks`` dense ones spread evenly over the depth;
* per-layer schedules ("comb" presets): a neighbourhood per block, chosen by layer-wise sensitivity; here a schedule is a string
  with one letter per block (``LAYER_KINDS``), ``-`` keeps the block dense.

The experiments start from the dense rectified-flow base experiment of the same size and change the network's two sparse fields,
the optimiser / schedule of the sparse fine-tuning runs and the context-parallel size.
"""

from __future__ import annotations

from typing import Dict, List, Optional

from ..utils.config import ConfigStore
from .video2world import BASE_2B, BASE_14B

cs = ConfigStore.instance()

BASE_SIZE = (-1, 44, 80)          # token grid the window sizes refer to; other resolutions scale the windows

# letter -> (window, stride, dilation); -1 along time = all frames
LAYER_KINDS: Dict[str, tuple] = {
    "a": ((-1, 12, 24), (1, 4, 8), None),            # ~90 % of the key / value positions skipped
    "b": ((-1, 20, 40), (1, 4, 8), None),            # ~75 %
    "c": ((-1, 28, 56), (1, 4, 8), None),            # ~50 %
    "d": ((-1, 4, 16), (1, 1, 1), (1, 11, 5)),       # dilated: a coarse view of the whole frame
    "e": ((-1, 12, 16), (1, 4, 1), (1, 1, 5)),       # dilated along the width only
    "f": ((-1, 4, 24), (1, 1, 8), (1, 11, 1)),       # dilated along the height only
}

SCHEDULES: Dict[str, str] = {
    "2B_comb01": "acaaaaaaacacccc-cc--ccc-cccc",
    "2B_comb02": "ddeaaeaaaaebbbbbbbbbbbbcbbba",     # the schedule chosen for the 2B model
    "2B_comb03": "ddeaaeaaabbcccccccccccc-cccb",
    "2B_comb04": "aaaaaaaaaaabbbbbbbbbbbbcbbba",
    "2B_comb05": "dfeaaeaaaeeb--ccbcbcccccbcca",
    "14B_comb01": "dddddddddddeeaaaaaabaabccbc-cccccccc",
    "14B_comb02": "dddddddddddeeaaaaaaaaaabcbc-cbbccbcb",
}


def layer_parameters(kind: str) -> Optional[dict]:
    if kind == "-":
        return None
    window, stride, dilation = LAYER_KINDS[kind]
    p = {"window_size": window, "stride": stride, "base_size": BASE_SIZE}
    if dilation is not None:
        p["dilation"] = dilation
    return p


def schedule_parameters(name: str) -> List[Optional[dict]]:
    """Per-block parameter list of a named schedule (``None`` = dense block)."""
    return [layer_parameters(k) for k in SCHEDULES[name]]


def skipped_fraction(name: str) -> float:
    """Share of the dense attention work that a schedule skips at the base resolution (window area / frame area per block)."""
    kept = 0.0
    for k in SCHEDULES[name]:
        if k == "-":
            kept += 1.0
        else:
            (_, wh, ww), _, _ = LAYER_KINDS[k]
            kept += (wh * ww) / float(BASE_SIZE[1] * BASE_SIZE[2])
    return 1.0 - kept / len(SCHEDULES[name])


UNIFORM = layer_parameters("a")


def _sparse_experiment(name: str, base: str, n_dense_blocks: int, natten_parameters, cp: int, lr: float = 2 ** -14.5, **extra) -> None:
    node = dict(
        defaults=[f"/experiment/{base}", "_self_"],
        job=dict(group="official_runs_video2world", name=name),
        model=dict(config=dict(net=dict(n_dense_blocks=n_dense_blocks, natten_parameters=natten_parameters))),
        model_parallel=dict(context_parallel_size=cp),
        optimizer=dict(lr=lr, weight_decay=0.1),
        scheduler=dict(f_max=(0.6,), f_min=(0.3,), warm_up_steps=(2_000,), cycle_lengths=(400_000,)),
        trainer=dict(max_iter=100_000, logging_iter=200),
        checkpoint=dict(save_iter=2_000, load_training_state=False, strict_resume=False),
    )
    node.update(extra)
    cs.store(group="experiment", package="_global_", name=name, node=node)


_P2B = "Stage-c_pt_4-Index-{i}-Size-2B-Res-720-Fps-16-Note-HQ_V3_from_22_sparse-attn_{note}"
_P14B = "Stage-c_pt_4-Index-{i}-Size-14B-Res-720-Fps-16-Note-T24_HQV2_1_from_43_sparse-attn_{note}"

# uniform neighbourhood, n dense blocks spread over the depth
for _i, _n in ((200, 7), (201, 6), (202, 4), (203, 9), (204, 12)):
    _sparse_experiment(_P2B.format(i=_i, note=f"{_n}dense"), BASE_2B, _n, UNIFORM, cp=2)
_sparse_experiment("Stage-c_pt_4-Index-200-Size-14B-Res-720-Fps-16-Note-T24_HQV3pt1_from_40_sparse-attn_9dense", BASE_14B, 9, UNIFORM, cp=8)

# per-layer schedules (the number in the note = dense blocks left by the schedule)
for _i, _s in ((206, "2B_comb01"), (207, "2B_comb02"), (208, "2B_comb03"), (209, "2B_comb04"), (210, "2B_comb05")):
    _note = f"comb{_s[-2:]}-{SCHEDULES[_s].count('-')}dense"
    _sparse_experiment(_P2B.format(i=_i, note=_note), BASE_2B, 0, schedule_parameters(_s), cp=2)
for _i, _s in ((201, "14B_comb01"), (202, "14B_comb02")):
    _note = f"comb{_s[-2:]}-{SCHEDULES[_s].count('-')}dense"
    _sparse_experiment(_P14B.format(i=_i, note=_note), BASE_14B, 0, schedule_parameters(_s), cp=8)

SPARSE_2B = _P2B.format(i=207, note="comb02-0dense")
SPARSE_14B = _P14B.format(i=202, note="comb02-1dense")

# small configuration for tests: the tiny network with a per-layer schedule on a 8 x 8 token grid
cs.store(group="experiment", package="_global_", name="tiny_video2world_sparse_cpu", node=dict(
    defaults=["/experiment/tiny_video2world_cpu", "_self_"],
    job=dict(group="tests", name="tiny_video2world_sparse_cpu"),
    model=dict(config=dict(net=dict(n_dense_blocks=0, natten_parameters=[
        {"window_size": (-1, 4, 4), "stride": (1, 2, 2), "base_size": (-1, 8, 8)}, None]))),
))
