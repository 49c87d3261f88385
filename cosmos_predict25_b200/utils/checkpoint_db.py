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
    filename: Optional[str] = None       # None => a whole repository, or ``subdirectory`` of it (directory checkpoint)
    revision: str = "main"
    subdirectory: Optional[str] = None
    exclude: tuple = ()                  # file patterns not to download

    @property
    def path(self) -> str:
        """Download (or find in the hub cache) and return the local file / directory."""
        from huggingface_hub import hf_hub_download, snapshot_download
        if self.filename:
            return hf_hub_download(self.repository, self.filename, revision=self.revision)
        allow = [self.subdirectory.rstrip("/") + "/*"] if self.subdirectory else None
        root = snapshot_download(self.repository, revision=self.revision, allow_patterns=allow, ignore_patterns=list(self.exclude) or None)
        return os.path.join(root, self.subdirectory) if self.subdirectory else root


@dataclass(frozen=True)
class CheckpointS3:
    uri: str


@dataclass(frozen=True)
class CheckpointConfig:
    uuid: str
    name: str
    experiment: Optional[str] = None
    s3_uri: Optional[str] = None
    hf: Optional[CheckpointHf] = None
    metadata: dict = field(default_factory=dict)

    @property
    def s3(self) -> Optional["CheckpointS3"]:
        """Object-store location as a record with a ``uri`` (None when the checkpoint has none), the attribute name the reference
        uses (checkpoint_db.py:138-170 there)."""
        return CheckpointS3(self.s3_uri) if self.s3_uri else None

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
                return self.hf.path
            except Exception as e:
                raise FileNotFoundError(
                    f"checkpoint {self.name} ({self.uuid}) is not in the local cache and could not be downloaded: {e}") from e
        raise FileNotFoundError(f"checkpoint {self.name} ({self.uuid}) has no Hugging Face location and is not cached locally")


_BY_UUID: Dict[str, CheckpointConfig] = {}
_CHECKPOINTS_BY_UUID = _BY_UUID                                # the reference's name of the table
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


# (uuid, name, experiment, object-store URI, Hugging Face repository, file in it, sub-directory of it, revision, excluded patterns):
# the public identifiers of the released checkpoints; a parameter file or an experiment that names one of them resolves here as it
# does in the reference (checkpoint_db.py:185-625 there)
_RELEASED = [
    ('4dbf13c6-1d30-4b02-99d6-75780dd8b744', 'google-t5/t5-11b', None, None, 'google-t5/t5-11b', None, None, '90f37703b3334dfe9d2b009bfcbfbf1ac9d28ea3', ('tf_model.h5',)),
    ('a2944743-cf8d-427e-a6fc-b3c03d807064', 'meta-llama/Llama-Guard-3-8B', None, None, 'meta-llama/Llama-Guard-3-8B', None, None, '7327bd9f6efbbe6101dc6cc4736302b3cbb6e425', ('original/*',)),
    ('9c7b7da4-2d95-45bb-9cb8-2eed954e9736', 'nvidia/Cosmos-Guardrail1', None, None, 'nvidia/Cosmos-Guardrail1', None, None, 'd6d4bfa899a71454a700907664f3e88f503950cf', ()),
    ('7219c6c7-f878-4137-bbdb-76842ea85e70', 'Qwen/Qwen2.5-VL-7B-Instruct', None, 's3://bucket/cosmos_reasoning1/pretrained/Qwen_tokenizer/Qwen/Qwen2.5-VL-7B-Instruct', 'nvidia/Cosmos-Experimental', None, '7219c6c7-f878-4137-bbdb-76842ea85e70', '736a20b6cfbc38e42ba3f7e7d8efa1d886c20db1', ()),
    ('685afcaa-4de2-42fe-b7b9-69f7a2dee4d8', 'Wan2.1/vae', None, 's3://bucket/cosmos_diffusion_v2/pretrain_weights/tokenizer/wan2pt1/Wan2.1_VAE.pth', 'nvidia/Cosmos-Experimental', 'tokenizer.pth', None, '736a20b6cfbc38e42ba3f7e7d8efa1d886c20db1', ()),
    ('cb3e3ffa-7b08-4c34-822d-61c7aa31a14f', 'nvidia/Cosmos-Reason1.1-7B', None, 's3://bucket/cosmos_reasoning1/sft_exp700/sft_exp721-1_qwen7b_tl_721_5vs5_s3_balanced_n32_resume_16k/checkpoints/iter_000016000/model', 'nvidia/Cosmos-Experimental', None, None, '736a20b6cfbc38e42ba3f7e7d8efa1d886c20db1', ()),
    ('d20b7120-df3e-4911-919d-db6e08bad31c', 'nvidia/Cosmos-Predict2.5-2B/base/pre-trained', 'Stage-c_pt_4-reason_embeddings-v1p1-Index-26-Size-2B-Res-720-Fps-16-Note-T2V_high_sigma_loss_reweighted_1_1_rectified_flow_only_resume2', 's3://bucket/cosmos_diffusion_v2/official_runs_vid2vid/Stage-c_pt_4-reason_embeddings-v1p1-Index-26-Size-2B-Res-720-Fps-16-Note-T2V_high_sigma_loss_reweighted_1_1_rectified_flow_only_resume2/checkpoints/iter_000023000/model', 'nvidia/Cosmos-Experimental', 'd20b7120-df3e-4911-919d-db6e08bad31c/model_ema_bf16.pt', None, 'main', ()),
    ('81edfebe-bd6a-4039-8c1d-737df1a790bf', 'nvidia/Cosmos-Predict2.5-2B/base/post-trained', 'Stage-c_pt_4-Index-2-Size-2B-Res-720-Fps-16-Note-rf_with_edm_ckpt', 's3://bucket/cosmos_diffusion_v2/official_runs_vid2vid/Stage-c_GRPO-reason_embeddings-Index-26-Size-2B-Res-720-Fps-16-posttrain_data-HQ_V7_RF_MERGE_LOCAL_ag_every2_guidance0_scorekeyoverall_reward_databeta0.01_mincon0/checkpoints/iter_000000288/model', 'nvidia/Cosmos-Experimental', '81edfebe-bd6a-4039-8c1d-737df1a790bf/model_ema_bf16.pt', None, 'main', ()),
    ('6b9d7548-33bb-4517-b5e8-60caf47edba7', 'nvidia/Cosmos-Predict2.5-2B/auto/multiview', 'buttercup_predict2p5_2b_7views_res720p_fps30_t8_from48kfps30mv_condprobs0442_joint_alpamayo1capnoviewprefix_allcapsviewprefix_29frames_nofps', 's3://bucket/cosmos_predict2_multiview/cosmos2_mv/buttercup_predict2p5_2b_7views_res720p_fps30_t8_from48kfps30mv_condprobs0442_joint_alpamayo1capnoviewprefix_allcapsviewprefix_29frames_nofps-0/checkpoints/iter_000005000/model', 'nvidia/Cosmos-Experimental', '6b9d7548-33bb-4517-b5e8-60caf47edba7/model_ema_bf16.pt', None, 'main', ()),
    ('0e8177cc-0db5-4cfd-a8a4-b820c772f4fc', 'nvidia/Cosmos-Predict2.5-2B/robot/multiview', 'multicamera_video2video_rectified_flow_2b_res_720_fps16_s3_multicam_syncam', 's3://bucket/cosmos_diffusion_v2/official_runs_vid2vid/multicamera_video2video_rectified_flow_2b_res_720_fps16_s3_multicam_syncam/checkpoints/iter_000002000/model', 'nvidia/Cosmos-Experimental', '0e8177cc-0db5-4cfd-a8a4-b820c772f4fc/model_ema_bf16.pt', None, 'main', ()),
    ('7f6b99b7-7fac-4e74-8dbe-a394cb56ef99', 'nvidia/Cosmos-Predict2.5-2B/robot/multiview-agibot', 'multicamera_video2video_rectified_flow_2b_res_720_fps16_s3_agibot', 's3://bucket/cosmos_diffusion_v2/official_runs_vid2vid/multicamera_video2video_rectified_flow_2b_res_720_fps16_s3_agibot/checkpoints/iter_000003000/model', 'nvidia/Cosmos-Experimental', '7f6b99b7-7fac-4e74-8dbe-a394cb56ef99/model_ema_bf16.pt', None, 'main', ()),
    ('24a3b7b8-6a3d-432d-b7d1-5d30b9229465', 'nvidia/Cosmos-Predict2.5-2B/transfer2.5', 'Stage-c_pt_4-reason_embeddings-v1p1-Index-26-Size-2B-Res-720-Fps-16-Note-T2V_high_sigma_loss_reweighted_1_1_rectified_flow_only', 's3://bucket/cosmos_diffusion_v2/official_runs_text2world/Stage-c_pt_4-reason_embeddings-v1p1-Index-26-Size-2B-Res-720-Fps-16-Note-T2V_high_sigma_loss_reweighted_1_1_rectified_flow_only/checkpoints/iter_000037000/model', 'nvidia/Cosmos-Experimental', '24a3b7b8-6a3d-432d-b7d1-5d30b9229465/model_ema_bf16.pt', None, 'main', ()),
    ('54937b8c-29de-4f04-862c-e67b04ec41e8', 'nvidia/Cosmos-Predict2.5-14B/base/pre-trained', 'Stage-c_pt_4-reason_embeddings-v1p1-Index-43-Size-14B-Res-720-Fps-16_resume_from_reason1p1_rectified_flow_shift5_high_sigma', 's3://bucket/cosmos_diffusion_v2/official_runs_text2world/Stage-c_pt_4-reason_embeddings-v1p1-Index-43-Size-14B-Res-720-Fps-16_resume_from_reason1p1_rectified_flow_shift5_high_sigma/checkpoints/iter_000012500/model', 'nvidia/Cosmos-Experimental', '54937b8c-29de-4f04-862c-e67b04ec41e8/model_ema_bf16.pt', None, 'main', ()),
    ('ecd0ba00-d598-4f94-aa09-e8627899c431', 'nvidia/Cosmos-Transfer2.5-2B/general/edge', 'edge_720p_t24_spaced_layer4_cr1pt1_sdev2_lowsigma0.05_nonuniform_hqv3p1_20250714_64N_rectified_flow_mock_data', 's3://bucket/cosmos_transfer2/vid2vid_2B_control/edge_720p_t24_spaced_layer4_cr1pt1_sdev2_lowsigma0.05_nonuniform_hqv3p1_20250714_64N_rectified_flow/checkpoints/iter_000029000/model', 'nvidia/Cosmos-Experimental', 'ecd0ba00-d598-4f94-aa09-e8627899c431/model_ema_bf16.pt', None, 'main', ()),
    ('fcab44fe-6fe7-492e-b9c6-67ef8c1a52ab', 'nvidia/Cosmos-Transfer2.5-2B/general/seg', 'seg_720p_t24_spaced_layer4_cr1pt1_sdev2_lowsigma0.05_nonuniform_hqv4p2_20250823_64N_rectified_flow', 's3://bucket/cosmos_transfer2/vid2vid_2B_control/seg_720p_t24_spaced_layer4_cr1pt1_sdev2_lowsigma0.05_nonuniform_hqv4p2_20250823_64N_rectified_flow/checkpoints/iter_000031000/model', 'nvidia/Cosmos-Experimental', 'fcab44fe-6fe7-492e-b9c6-67ef8c1a52ab/model_ema_bf16.pt', None, 'main', ()),
    ('20d9fd0b-af4c-4cca-ad0b-f9b45f0805f1', 'nvidia/Cosmos-Transfer2.5-2B/general/blur', 'vis_720p_t24_spaced_layer4_cr1pt1_sdev2_lowsigma0.05_nonuniform_hqv3p1_20250714_64N_rectified_flow', 's3://bucket/cosmos_transfer2/vid2vid_2B_control/vis_720p_t24_spaced_layer4_cr1pt1_sdev2_lowsigma0.05_nonuniform_hqv3p1_20250714_64N_rectified_flow/checkpoints/iter_000043000/model', 'nvidia/Cosmos-Experimental', '20d9fd0b-af4c-4cca-ad0b-f9b45f0805f1/model_ema_bf16.pt', None, 'main', ()),
    ('0f214f66-ae98-43cf-ab25-d65d09a7e68f', 'nvidia/Cosmos-Transfer2.5-2B/general/depth', 'depth_720p_t24_spaced_layer4_cr1pt1_sdev2_lowsigma0.05_nonuniform_hqv4p1_20250823_64N_rectified_flow', 's3://bucket/cosmos_transfer2/vid2vid_2B_control/depth_720p_t24_spaced_layer4_cr1pt1_sdev2_lowsigma0.05_nonuniform_hqv4p1_20250823_64N_rectified_flow/checkpoints/iter_000028000/model', 'nvidia/Cosmos-Experimental', '0f214f66-ae98-43cf-ab25-d65d09a7e68f/model_ema_bf16.pt', None, 'main', ()),
    ('b5ab002d-a120-4fbf-a7f9-04af8615710b', 'nvidia/Cosmos-Transfer2.5-2B/auto/multiview', 'buttercup_transfer2p5_2b_mv_7views_res720p_fps10_t8_frombase5knofps_mads720pmulticaps29frames_world_scenario_resumefrom21k', 's3://bucket/cosmos_transfer2_multiview/cosmos2_mv/buttercup_transfer2p5_2b_mv_7views_res720p_fps10_t8_frombase5knofps_mads720pmulticaps29frames_world_scenario_resumefrom21k-0/checkpoints/iter_000010000/model', 'nvidia/Cosmos-Experimental', 'b5ab002d-a120-4fbf-a7f9-04af8615710b/model_ema_bf16.pt', None, 'main', ()),
]
for _u, _n, _e, _s3, _repo, _file, _sub, _rev, _ex in _RELEASED:
    register_checkpoint(CheckpointConfig(uuid=_u, name=_n, experiment=_e, s3_uri=_s3,
                                         hf=CheckpointHf(_repo, _file, _rev, _sub, _ex) if _repo else None))
