"""Validators, env parsers, camera / quaternion math, volume rendering, straggler detector, profiling contexts (CPU)."""
import math
import os

import numpy as np
import pytest
import torch

from cosmos_predict25_b200.modules.camera import Camera, Quaternion
from cosmos_predict25_b200.modules import volume_render as vr
from cosmos_predict25_b200.utils import validator as V
from cosmos_predict25_b200.utils.env_parsers import CredentialEnvParser, EnvParser, InferenceEnvParser


def _rand_pose(*batch):
    q = Quaternion.normalize(torch.randn(*batch, 4))
    return torch.cat([Quaternion.to_rotation_matrix(q), torch.randn(*batch, 3, 1)], dim=-1)


def test_quaternion_roundtrip_and_product():
    torch.manual_seed(0)
    q = Quaternion.normalize(torch.randn(64, 4))
    q = torch.where(q[:, 3:] < 0, -q, q)
    R = Quaternion.to_rotation_matrix(q)
    assert torch.allclose(R @ R.transpose(-1, -2), torch.eye(3).expand(64, 3, 3), atol=1e-5)
    assert torch.allclose(torch.linalg.det(R), torch.ones(64), atol=1e-5)
    back = Quaternion.from_rotation_matrix(R)                     # q and -q are the same rotation; the sign rule is the reference's
    assert torch.allclose(back * torch.sign((back * q).sum(-1, keepdim=True)), q, atol=1e-5)
    # 180-degree rotations exercise the non-trace branches
    for axis in range(3):
        qq = torch.zeros(4); qq[axis] = 1.0
        back = Quaternion.from_rotation_matrix(Quaternion.to_rotation_matrix(qq))
        assert torch.allclose(back.abs(), qq.abs(), atol=1e-6)
    a, b = Quaternion.normalize(torch.randn(8, 4)), Quaternion.normalize(torch.randn(8, 4))
    assert torch.allclose(Quaternion.to_rotation_matrix(Quaternion.multiply(a, b)),
                          Quaternion.to_rotation_matrix(a) @ Quaternion.to_rotation_matrix(b), atol=1e-5)
    ident = Quaternion.multiply(a, Quaternion.invert(a))
    assert torch.allclose(ident, torch.tensor([0, 0, 0, 1.0]).expand(8, 4), atol=1e-5)


def test_camera_transforms():
    torch.manual_seed(1)
    P = _rand_pose(5)
    x = torch.randn(5, 7, 3)
    xc = Camera.world2camera(x, P)
    assert torch.allclose(xc, x @ P[..., :3].transpose(-1, -2) + P[..., 3].unsqueeze(-2), atol=1e-5)
    assert torch.allclose(Camera.camera2world(xc, P), x, atol=1e-4)
    inv = Camera.invert_pose(P)
    ident = Camera.compose_poses([P, inv])
    assert torch.allclose(ident, torch.eye(3, 4).expand(5, 3, 4), atol=1e-5)
    c = Camera.get_camera_center(P)
    assert torch.allclose(Camera.world2camera(c.unsqueeze(-2), P), torch.zeros(5, 1, 3), atol=1e-5)
    K = Camera.intrinsic_params_to_matrices(torch.tensor([[100.0, 110.0, 16.0, 12.0]]).expand(5, 4))
    assert torch.allclose(Camera.intrinsic_matrices_to_params(K)[0], torch.tensor([100.0, 110.0, 16.0, 12.0]))
    rays = Camera.get_camera_rays(P, K, (24, 32))
    assert rays.shape == (5, 768, 3) and torch.allclose(rays.norm(dim=-1), torch.ones(5, 768), atol=1e-5)
    # a point along a ray projects back to its pixel centre
    pix = 5 * 32 + 9
    pw = c + 3.0 * rays[:, pix]
    uvw = Camera.camera2image(Camera.world2camera(pw.unsqueeze(-2), P), K)[:, 0]
    assert torch.allclose(uvw[:, :2] / uvw[:, 2:], torch.tensor([9.5, 5.5]).expand(5, 2), atol=1e-2)
    pl = Camera.get_plucker_rays(P, K, (24, 32))
    assert pl.shape == (5, 768, 6) and torch.allclose((pl[..., :3] * pl[..., 3:]).sum(-1), torch.zeros(5, 768), atol=1e-4)
    rel = Camera.get_relative_poses_wrt_frame0(_rand_pose(2, 4))
    assert torch.allclose(rel[:, 0], torch.eye(3, 4).expand(2, 3, 4), atol=1e-5)
    prm = Camera.extrinsic_matrices_to_params(P)
    assert torch.allclose(Camera.extrinsic_params_to_matrices(prm), P, atol=1e-5)
    assert isinstance(Camera.invert_pose(P.numpy()), np.ndarray)            # numpy in -> numpy out


def test_volume_rendering():
    near, far = torch.full((4, 1), 1.0), torch.full((4, 1), 3.0)
    d = vr.sample_dists(near, far, 4)
    assert torch.allclose(d[0], torch.tensor([1.25, 1.75, 2.25, 2.75]))
    ds = vr.sample_dists(near, far, 64, stratified=True)
    assert (ds >= 1).all() and (ds <= 3).all() and (ds[:, 1:] > ds[:, :-1]).all()

    class Field(torch.nn.Module):
        def forward(self, pts, dirs):
            return torch.ones_like(pts) * 0.5, torch.full_like(pts[..., :1], 2.0)

    rgb, opacity, w, pts, dists = vr.volume_render_rays(Field(), torch.zeros(4, 3), torch.tensor([0, 0, 1.0]).expand(4, 3), near, far, 256)
    # constant density sigma over [1.0039, 3]: opacity = 1 - exp(-sigma * length)
    assert torch.allclose(opacity, torch.full((4, 1), 1 - math.exp(-2.0 * (3.0 - float(dists[0, 0])))), atol=1e-4)
    assert torch.allclose(rgb, 0.5 * opacity.expand(4, 3), atol=1e-5)
    _, op_solid, *_ = vr.volume_render_rays(Field(), torch.zeros(4, 3), torch.tensor([0, 0, 1.0]).expand(4, 3), near, far, 16, solid_background=True)
    assert torch.allclose(op_solid, torch.ones(4, 1), atol=1e-5)


def test_validators():
    class Req:
        steps = V.Int(default=35, min=1, max=100)
        guidance = V.Float(default=7.0, min=0, max=20)
        flag = V.Bool(default=False)
        mode = V.OneOf(default="a", options=["a", "b"])
        width = V.MultipleOf(default=16, multiple_of=16)
        name = V.String(min=2, max=5)
        extra = V.JsonDict(default={})

    r = Req()
    assert r.steps == 35 and r.flag is False
    r.steps, r.guidance, r.flag, r.extra = "50", 3, "true", '{"a": 1}'
    assert r.steps == 50 and r.guidance == 3.0 and r.flag is True and r.extra == {"a": 1}
    for attr, bad in (("steps", 0), ("steps", 1.5), ("guidance", 21), ("mode", "c"), ("width", 17), ("name", "x"), ("flag", "maybe")):
        with pytest.raises((ValueError, TypeError)):
            setattr(r, attr, bad)
    with pytest.raises(ValueError):
        _ = r.name                                   # mandatory and unset
    assert list(Req.steps.get_range_iterator())[:3] == [1, 2, 3] and sorted(Req.mode.get_range_iterator()) == ["a", "b"]
    assert Req.steps.json()["max"] == 100 and Req.mode.json()["values"] == ["a", "b"]
    assert V.BytesIOType().validate("YWJj").read() == b"abc"


def test_env_parsers(tmp_path, monkeypatch):
    monkeypatch.setenv("NUM_GPUS", "4")
    monkeypatch.setenv("MODEL_NAME", "2B/post-trained")
    p = InferenceEnvParser()
    assert p.NUM_GPUS == 4 and p.MODEL_NAME == "2B/post-trained" and p.DISABLE_GUARDRAILS is False
    q = InferenceEnvParser(p.to_b64())
    assert q.to_dict() == p.to_dict()
    p.to_json(str(tmp_path / "env.json"))
    monkeypatch.delenv("NUM_GPUS")
    r = InferenceEnvParser()
    assert r.NUM_GPUS == 1
    r.from_json(str(tmp_path / "env.json"))
    assert r.NUM_GPUS == 4 and r.to_string_dict()["NUM_GPUS"] == "4"
    monkeypatch.setenv("NUM_GPUS", "99")
    with pytest.raises(ValueError):
        InferenceEnvParser()
    monkeypatch.delenv("NUM_GPUS")

    class Mandatory(EnvParser):
        TOKEN = V.String()

    with pytest.raises(ValueError):
        Mandatory()
    assert CredentialEnvParser().credentials("PROD_FT_AWS_CREDS")["region_name"] == "us-west-2"


def test_straggler_detector_single_process():
    from cosmos_predict25_b200.utils.straggler import BufferCnt, StragglerDetector
    import time
    det = StragglerDetector(report_freq=2, raise_error=False)
    for it in range(1, 5):
        with det.profile_section("fwd", profile_cuda=False):
            time.sleep(0.002 * (3 if it > 2 else 1))
        rep = det.generate_report(it)
        assert (rep is None) == (it % 2 == 1)
    assert rep.gpu_relative_perf_scores == {0: 1.0} and rep.gpu_individual_perf_scores[0] < 0.7   # 3x slower than its best
    assert rep.identify_stragglers()["straggler_gpus_individual"] == [0]
    c = BufferCnt(thres=2, reset_over_thres=True)
    assert [c(True), c(True), c(True), c(False)] == [False, True, False, False]


def test_profiling_contexts(tmp_path):
    from cosmos_predict25_b200.utils.profiling import ProfilingConfig, maybe_enable_memory_snapshot, maybe_enable_profiling
    with maybe_enable_profiling(ProfilingConfig(), str(tmp_path)) as p:
        assert p is None
    cfg = ProfilingConfig(enable_profiling=True, profile_freq=4)
    with maybe_enable_profiling(cfg, str(tmp_path), global_step=0) as prof:
        for _ in range(4):
            torch.randn(8, 8) @ torch.randn(8, 8)
            prof.step()
    assert any(f.endswith("trace.json.gz") for _, _, fs in os.walk(tmp_path / "torch_trace") for f in fs)
    with maybe_enable_memory_snapshot(ProfilingConfig(enable_memory_snapshot=True, profile_freq=2), str(tmp_path)) as mp:
        mp.step(); mp.step()
    assert os.path.exists(tmp_path / "memory_snapshot" / "iteration_2" / "rank0_memory_snapshot.pickle")


def test_config_yaml_round_trip_with_type_markers(tmp_path):
    import enum

    import torch

    from cosmos_predict25_b200.config import InferenceType
    from cosmos_predict25_b200.trainer.optim import OptimizerConfig
    from cosmos_predict25_b200.utils.lazy_config import LazyCall as L
    from cosmos_predict25_b200.utils.lazy_config import LazyConfig, instantiate
    cfg = {"precision": torch.bfloat16, "kind": InferenceType.VIDEO2WORLD, "optimizer": OptimizerConfig(lr=3e-4, weight_decay=0.1),
           "net": L(torch.nn.Linear)(in_features=4, out_features=2, bias=False), "nested": {"sizes": (1, 2, 3), "none": None, "flag": True}}
    path = str(tmp_path / "config.yaml")
    LazyConfig.save_yaml(cfg, path)
    text = open(path).read()
    assert "__type__: torch.dtype" in text and "torch.nn.modules.linear.Linear" in text
    back = LazyConfig.load_yaml(path)
    assert back["precision"] is torch.bfloat16 and back["kind"] is InferenceType.VIDEO2WORLD
    assert isinstance(back["optimizer"], OptimizerConfig) and back["optimizer"].lr == 3e-4 and back["optimizer"].weight_decay == 0.1
    assert back["nested"]["sizes"] == [1, 2, 3] and back["nested"]["none"] is None and back["nested"]["flag"] is True
    lin = instantiate(back["net"])
    assert isinstance(lin, torch.nn.Linear) and lin.weight.shape == (2, 4) and lin.bias is None
