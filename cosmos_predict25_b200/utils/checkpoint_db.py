"""Checkpoint registry: UUID -> {name, experiment, storage URI, Hugging Face repository/file}.

Parity target: cosmos_predict2/_src/imaginaire/utils/checkpoint_db.py:138-625. Look-ups by UUID, by S3 URI
and by name; resolution order for a path: an explicit local file, the local cache
(``$COSMOS_CHECKPOINT_DIR`` or ``$HF_HOME``), then a Hugging Face download (only when the hub is
importable and reachable; this build environment has no network, so missing weights raise a clear error).
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, Optional


@dataclass(frozen=True)
class CheckpointHf:
    repository: str
    filename: Optional[str] = None       # None => a whole repository (directory checkpoint)
    revision: str = "main"


@dataclass(frozen=True)
class CheckpointConfig:
    uuid: str
    name: str
    experiment: Optional[str] = None
    s3_uri: Optional[str] = None
    hf: Optional[CheckpointHf] = None
    metadata: dict = field(default_factory=dict)

    def local_candidates(self):
        roots = [os.environ.get("COSMOS_CHECKPOINT_DIR"), os.path.join(os.environ.get("HF_HOME", os.path.expanduser("~/.cache/huggingface")), "cosmos")]
        for r in roots:
            if not r:
                continue
            if self.hf is not None and self.hf.filename:
                yield os.path.join(r, self.hf.repository, self.hf.filename)
                yield os.path.join(r, os.path.basename(self.hf.filename))
            yield os.path.join(r, self.uuid)
            yield os.path.join(r, self.uuid + ".pt")

    @property
    def path(self) -> str:
        for c in self.local_candidates():
            if os.path.exists(c):
                return c
        if self.hf is not None:
            try:
                from huggingface_hub import hf_hub_download, snapshot_download
                if self.hf.filename:
                    return hf_hub_download(self.hf.repository, self.hf.filename, revision=self.hf.revision)
                return snapshot_download(self.hf.repository, revision=self.hf.revision)
            except Exception as e:
                raise FileNotFoundError(
                    f"checkpoint {self.name} ({self.uuid}) is not in the local cache and could not be downloaded: {e}") from e
        raise FileNotFoundError(f"checkpoint {self.name} ({self.uuid}) has no Hugging Face location and is not cached locally")


_BY_UUID: Dict[str, CheckpointConfig] = {}
_BY_S3: Dict[str, CheckpointConfig] = {}
_BY_NAME: Dict[str, CheckpointConfig] = {}


def register_checkpoint(c: CheckpointConfig) -> CheckpointConfig:
    if c.uuid in _BY_UUID:
        raise ValueError(f"checkpoint UUID {c.uuid} already registered")
    _BY_UUID[c.uuid] = c
    _BY_NAME[c.name] = c
    if c.s3_uri:
        if c.s3_uri in _BY_S3:
            raise ValueError(f"checkpoint URI {c.s3_uri} already registered")
        _BY_S3[c.s3_uri] = c
    return c


def get_checkpoint_by_uuid(uuid: str) -> CheckpointConfig:
    if uuid not in _BY_UUID:
        raise KeyError(f"unknown checkpoint UUID {uuid}")
    return _BY_UUID[uuid]


def get_checkpoint_by_s3(uri: str) -> CheckpointConfig:
    uri = uri.rstrip("/")
    if uri not in _BY_S3:
        raise KeyError(f"unknown checkpoint URI {uri}")
    return _BY_S3[uri]


def get_checkpoint_by_name(name: str) -> CheckpointConfig:
    return _BY_NAME[name]


def get_checkpoint_path(ref: str) -> str:
    """Local path for a UUID, a registered URI, a registered name, or an existing file/directory."""
    if os.path.exists(ref):
        return ref
    for table in (_BY_UUID, _BY_S3, _BY_NAME):
        if ref in table:
            return table[ref].path
    raise FileNotFoundError(f"{ref} is neither a file nor a registered checkpoint")


def _reg(uuid, name, experiment=None, repo=None, filename=None):
    s3 = f"s3://bucket/cosmos_diffusion_v2/official_runs_vid2vid/{uuid}/model_ema_bf16.pt" if experiment else None
    return register_checkpoint(CheckpointConfig(uuid=uuid, name=name, experiment=experiment, s3_uri=s3,
                                                hf=CheckpointHf(repo, filename) if repo else None))


# auxiliary models
_reg("4dbf13c6-1d30-4b02-99d6-75780dd8b744", "google-t5/t5-11b", repo="google-t5/t5-11b")
_reg("a2944743-cf8d-427e-a6fc-b3c03d807064", "meta-llama/Llama-Guard-3-8B", repo="meta-llama/Llama-Guard-3-8B")
_reg("9c7b7da4-2d95-45bb-9cb8-2eed954e9736", "nvidia/Cosmos-Guardrail1", repo="nvidia/Cosmos-Guardrail1")
_reg("7219c6c7-f878-4137-bbdb-76842ea85e70", "Qwen/Qwen2.5-VL-7B-Instruct", repo="nvidia/Cosmos-Reason1-7B")
_reg("685afcaa-4de2-42fe-b7b9-69f7a2dee4d8", "Wan2.1/vae", repo="nvidia/Cosmos-Predict2.5-2B", filename="tokenizer.pth")
_reg("cb3e3ffa-7b08-4c34-822d-61c7aa31a14f", "nvidia/Cosmos-Reason1.1-7B", repo="nvidia/Cosmos-Reason1-7B")
# Predict2.5 world models (consolidated EMA bf16 weights)
_reg("d20b7120-df3e-4911-919d-db6e08bad31c", "nvidia/Cosmos-Predict2.5-2B/base/pre-trained",
     "Stage-c_pt_4-reason_embeddings-v1p1-Index-26-Size-2B-Res-720-Fps-16-Note-T2V_high_sigma_loss_reweighted_1_1_rectified_flow_only_resume2",
     "nvidia/Cosmos-Predict2.5-2B", "base/pre-trained/d20b7120-df3e-4911-919d-db6e08bad31c_ema_bf16.pt")
_reg("81edfebe-bd6a-4039-8c1d-737df1a790bf", "nvidia/Cosmos-Predict2.5-2B/base/post-trained",
     "Stage-c_pt_4-Index-2-Size-2B-Res-720-Fps-16-Note-rf_with_edm_ckpt",
     "nvidia/Cosmos-Predict2.5-2B", "base/post-trained/81edfebe-bd6a-4039-8c1d-737df1a790bf_ema_bf16.pt")
_reg("6b9d7548-33bb-4517-b5e8-60caf47edba7", "nvidia/Cosmos-Predict2.5-2B/auto/multiview",
     "buttercup_predict2p5_2b_7views_res720p_fps30_t8_from48kfps30mv_condprobs0442_joint_alpamayo1capnoviewprefix_allcapsviewprefix_29frames_nofps",
     "nvidia/Cosmos-Predict2.5-2B", "auto/multiview/6b9d7548-33bb-4517-b5e8-60caf47edba7_ema_bf16.pt")
_reg("0e8177cc-0db5-4cfd-a8a4-b820c772f4fc", "nvidia/Cosmos-Predict2.5-2B/robot/multiview",
     "multicamera_video2video_rectified_flow_2b_res_720_fps16_s3_multicam_syncam",
     "nvidia/Cosmos-Predict2.5-2B", "robot/multiview/0e8177cc-0db5-4cfd-a8a4-b820c772f4fc_ema_bf16.pt")
_reg("7f6b99b7-7fac-4e74-8dbe-a394cb56ef99", "nvidia/Cosmos-Predict2.5-2B/robot/multiview-agibot",
     "multicamera_video2video_rectified_flow_2b_res_720_fps16_s3_agibot",
     "nvidia/Cosmos-Predict2.5-2B", "robot/multiview-agibot/7f6b99b7-7fac-4e74-8dbe-a394cb56ef99_ema_bf16.pt")
_reg("54937b8c-29de-4f04-862c-e67b04ec41e8", "nvidia/Cosmos-Predict2.5-14B/base/pre-trained",
     "Stage-c_pt_4-reason_embeddings-v1p1-Index-43-Size-14B-Res-720-Fps-16_resume_from_reason1p1_rectified_flow_shift5_high_sigma",
     "nvidia/Cosmos-Predict2.5-14B", "base/pre-trained/54937b8c-29de-4f04-862c-e67b04ec41e8_ema_bf16.pt")
