"""Camera and quaternion math on batched tensors (numpy accepted: converted in, converted back out).

Parity target: ``Camera`` / ``Quaternion`` (cosmos_predict2/_src/imaginaire/modules/camera.py:82-700). Conventions: a pose
is a world-to-camera extrinsic ``[R|t]`` of shape [...,3,4] in OpenCV axes, ``x_cam = R x_world + t``; points are row
vectors, so transforms apply as ``points_hom @ pose^T``; intrinsics are [...,3,3] or the parameter vector
``(fx, fy, cx, cy)``; quaternions are ``(x, y, z, w)``. Rotation algebra runs in float32 and is cast back.
"""

from __future__ import annotations

import functools
import inspect
from typing import List, Sequence, Tuple

import numpy as np
import torch


def _to_numpy(x):
    if isinstance(x, torch.Tensor):
        return x.detach().cpu().numpy()
    if isinstance(x, (list, tuple)):
        return type(x)(_to_numpy(v) for v in x)
    return x


def supports_numpy(arg_names: Sequence[str], use_no_grad: bool = True):
    """If any of the named arguments is a numpy array (or a list of them) the call runs on torch copies and returns numpy."""
    def deco(fn):
        sig = inspect.signature(fn)

        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            bound = sig.bind(*args, **kwargs)
            was_np = False
            for name in arg_names:
                if name not in bound.arguments:
                    continue
                v = bound.arguments[name]
                if isinstance(v, np.ndarray):
                    bound.arguments[name], was_np = torch.from_numpy(v), True
                elif isinstance(v, (list, tuple)) and any(isinstance(e, np.ndarray) for e in v):
                    bound.arguments[name] = [torch.from_numpy(e) if isinstance(e, np.ndarray) else e for e in v]
                    was_np = True
            if was_np and use_no_grad:
                with torch.no_grad():
                    return _to_numpy(fn(*bound.args, **bound.kwargs))
            out = fn(*bound.args, **bound.kwargs)
            return _to_numpy(out) if was_np else out
        return wrapper
    return deco


class Camera:
    @staticmethod
    @supports_numpy(["cam_pose"])
    def _check_valid_pose(cam_pose) -> None:
        assert cam_pose.shape[-2:] == (3, 4), "Camera pose is not of shape (3,4)."
        det = torch.linalg.det(cam_pose[..., :3].to(torch.float32))
        tol = (1e-2, 1e-2) if cam_pose.dtype in (torch.bfloat16, torch.float16) else (1e-4, 1e-6)
        ok = bool(torch.isfinite(det).all()) and torch.allclose(det, torch.ones_like(det), rtol=tol[0], atol=tol[1])
        assert ok, f"Rotation component in camera pose is invalid (det != 1 within tol); det_mean={det.mean().item():.6f}"

    @staticmethod
    @supports_numpy(["cam_pose"])
    def invert_pose(cam_pose):
        Camera._check_valid_pose(cam_pose)
        Rt = cam_pose[..., :3].float().transpose(-1, -2)
        return torch.cat([Rt, -Rt @ cam_pose[..., 3:].float()], dim=-1).to(cam_pose.dtype)

    @staticmethod
    @supports_numpy(["cam_poses"])
    def compose_poses(cam_poses: List):
        """``compose([p1, ..., pN])(x) = pN o ... o p1 (x)``."""
        first = cam_poses[0]
        Camera._check_valid_pose(first)
        R, t = first[..., :3].float(), first[..., 3:].float()
        for p in cam_poses[1:]:
            Camera._check_valid_pose(p)
            Rp, tp = p[..., :3].float(), p[..., 3:].float()
            R, t = Rp @ R, Rp @ t + tp
        return torch.cat([R, t], dim=-1).to(first.dtype)

    @staticmethod
    @supports_numpy(["cam_pose"])
    def get_camera_center(cam_pose):
        """World position of the optical centre: ``-R^T t``."""
        R, t = cam_pose[..., :3].float(), cam_pose[..., 3:].float()
        return (-R.transpose(-1, -2) @ t)[..., 0].to(cam_pose.dtype)

    @staticmethod
    @supports_numpy(["points"])
    def to_homogeneous(points):
        return torch.cat([points, torch.ones_like(points[..., :1])], dim=-1)

    @staticmethod
    @supports_numpy(["points", "cam_pose"])
    def world2camera(points, cam_pose):
        """points [...,N,3] -> camera frame."""
        return Camera.to_homogeneous(points) @ cam_pose.transpose(-1, -2)

    @staticmethod
    @supports_numpy(["points", "cam_pose"])
    def camera2world(points, cam_pose):
        return Camera.to_homogeneous(points) @ Camera.invert_pose(cam_pose).transpose(-1, -2)

    @staticmethod
    @supports_numpy(["points", "cam_intr"])
    def camera2image(points, cam_intr):
        """Camera-frame points [...,N,3] -> homogeneous pixel coordinates [...,N,3] (divide by the last entry for pixels)."""
        return points @ cam_intr.transpose(-1, -2)

    @staticmethod
    @supports_numpy(["points", "cam_intr"])
    def image2camera(points, cam_intr):
        """Homogeneous pixel coordinates -> camera-frame points on the depth given by the homogeneous scale."""
        return points @ torch.linalg.inv(cam_intr.float()).to(points.dtype).transpose(-1, -2)

    @staticmethod
    @supports_numpy(["cam_pose", "cam_intr"])
    def get_camera_rays(cam_pose, cam_intr, image_size: Tuple[int, int]):
        """Unit world-space directions through every pixel centre, [...,HW,3]."""
        H, W = image_size
        dev = cam_pose.device
        ys, xs = torch.meshgrid(torch.arange(H, dtype=torch.float32, device=dev) + 0.5,
                                torch.arange(W, dtype=torch.float32, device=dev) + 0.5, indexing="ij")
        xy = torch.stack([xs, ys], dim=-1).view(-1, 2).repeat(*cam_pose.shape[:-2], 1, 1)
        Camera._check_valid_pose(cam_pose)                    # with the tolerance of the pose's own dtype; the math below is fp32
        grid_cam = Camera.image2camera(Camera.to_homogeneous(xy), cam_intr.float())
        R, t = cam_pose[..., :3].float(), cam_pose[..., 3:].float()
        Rt = R.transpose(-1, -2)
        inv = torch.cat([Rt, -Rt @ t], dim=-1)                # cam2world
        grid_world = Camera.to_homogeneous(grid_cam) @ inv.transpose(-1, -2)
        center = (-Rt @ t)[..., 0].unsqueeze(-2)
        return torch.nn.functional.normalize(grid_world - center, dim=-1).to(cam_pose.dtype)

    @staticmethod
    @supports_numpy(["cam_pose", "cam_intr"])
    def get_plucker_rays(cam_pose, cam_intr, image_size: Tuple[int, int]):
        """Pluecker coordinates ``[o x d | d]`` per pixel, [...,HW,6]."""
        d = Camera.get_camera_rays(cam_pose, cam_intr, image_size)
        o = Camera.get_camera_center(cam_pose).unsqueeze(-2).expand_as(d)
        return torch.cat([torch.linalg.cross(o, d), d], dim=-1)

    @staticmethod
    @supports_numpy(["cam_pose"])
    def get_relative_poses_wrt_frame0(cam_pose):
        """[...,V,3,4] -> the same cameras expressed in the first camera's frame (the first becomes ``[I|0]``)."""
        ref_inv = Camera.invert_pose(cam_pose.select(dim=-3, index=0)).unsqueeze(-3).expand_as(cam_pose)
        return Camera.compose_poses([ref_inv, cam_pose])

    @staticmethod
    @supports_numpy(["params"])
    def intrinsic_params_to_matrices(params):
        """(fx, fy, cx, cy) [...,4] -> [...,3,3]."""
        fx, fy, cx, cy = params.unbind(-1)
        z, o = torch.zeros_like(fx), torch.ones_like(fx)
        return torch.stack([torch.stack([fx, z, cx], -1), torch.stack([z, fy, cy], -1), torch.stack([z, z, o], -1)], -2)

    @staticmethod
    @supports_numpy(["cam_intr"])
    def intrinsic_matrices_to_params(cam_intr):
        return torch.stack([cam_intr[..., 0, 0], cam_intr[..., 1, 1], cam_intr[..., 0, 2], cam_intr[..., 1, 2]], dim=-1)

    @staticmethod
    @supports_numpy(["qxyzw_t"])
    def extrinsic_params_to_matrices(qxyzw_t):
        """(qx, qy, qz, qw, tx, ty, tz) [...,7] -> [...,3,4]."""
        return torch.cat([Quaternion.to_rotation_matrix(qxyzw_t[..., :4]), qxyzw_t[..., 4:, None]], dim=-1)

    @staticmethod
    @supports_numpy(["cam_pose"])
    def extrinsic_matrices_to_params(cam_pose):
        return torch.cat([Quaternion.from_rotation_matrix(cam_pose[..., :3]), cam_pose[..., 3]], dim=-1)


class Quaternion:
    """(x, y, z, w) quaternions."""

    @staticmethod
    @supports_numpy(["q"])
    def normalize(q, eps: float = 1e-8):
        return q / q.norm(dim=-1, keepdim=True).clamp_min(eps)

    @staticmethod
    @supports_numpy(["q"])
    def to_rotation_matrix(q):
        x, y, z, w = Quaternion.normalize(q.float()).unbind(-1)
        R = torch.stack([
            torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w)], -1),
            torch.stack([2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w)], -1),
            torch.stack([2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)], -1)], -2)
        return R.to(q.dtype)

    @staticmethod
    @supports_numpy(["R"])
    def from_rotation_matrix(R, eps: float = 1e-8):
        """Numerically stable: per matrix, the branch whose pivot is the trace (when positive) or the largest diagonal entry."""
        m = R.float()
        m00, m11, m22 = m[..., 0, 0], m[..., 1, 1], m[..., 2, 2]
        cand = torch.stack([
            torch.stack([m[..., 2, 1] - m[..., 1, 2], m[..., 0, 2] - m[..., 2, 0], m[..., 1, 0] - m[..., 0, 1], 1 + m00 + m11 + m22], -1),
            torch.stack([1 + m00 - m11 - m22, m[..., 0, 1] + m[..., 1, 0], m[..., 0, 2] + m[..., 2, 0], m[..., 2, 1] - m[..., 1, 2]], -1),
            torch.stack([m[..., 0, 1] + m[..., 1, 0], 1 - m00 + m11 - m22, m[..., 1, 2] + m[..., 2, 1], m[..., 0, 2] - m[..., 2, 0]], -1),
            torch.stack([m[..., 0, 2] + m[..., 2, 0], m[..., 1, 2] + m[..., 2, 1], 1 - m00 - m11 + m22, m[..., 1, 0] - m[..., 0, 1]], -1),
        ], -2)                                                     # [...,4 branches,4]; branch b has pivot cand[b, pivot_idx[b]]
        # branch rule and sign of the reference (camera.py:556-617 there), so that serialised poses agree number by number: the
        # trace branch when the trace is positive, else the branch of the largest diagonal entry; the pivot component is positive
        best = torch.where(m00 + m11 + m22 > 0, 0, torch.where((m00 > m11) & (m00 > m22), 1, torch.where(m11 > m22, 2, 3)))
        q = torch.gather(cand, -2, best[..., None, None].expand(*best.shape, 1, 4))[..., 0, :]
        return Quaternion.normalize(q, eps).to(R.dtype)

    @staticmethod
    @supports_numpy(["q"])
    def invert(q, eps: float = 1e-8):
        conj = torch.cat([-q[..., :3], q[..., 3:]], dim=-1)
        return conj / (q * q).sum(-1, keepdim=True).clamp_min(eps)

    @staticmethod
    @supports_numpy(["q1", "q2"])
    def multiply(q1, q2):
        """Hamilton product: the rotation ``q1 * q2`` applies ``q2`` first."""
        x1, y1, z1, w1 = q1.unbind(-1)
        x2, y2, z2, w2 = q2.unbind(-1)
        return torch.stack([w1 * x2 + x1 * w2 + y1 * z2 - z1 * y2, w1 * y2 - x1 * z2 + y1 * w2 + z1 * x2,
                            w1 * z2 + x1 * y2 - y1 * x2 + z1 * w2, w1 * w2 - x1 * x2 - y1 * y2 - z1 * z2], dim=-1)
