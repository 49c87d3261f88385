"""Volume rendering along rays (quadrature of the emission-absorption integral).

Parity target: cosmos_predict2/_src/imaginaire/modules/volume_render.py:19-150 (``volume_render_rays``,
``volume_rendering_alphas``, ``alpha_compositing_weights``, ``composite``, ``sample_dists``).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch


@torch.no_grad()
def sample_dists(near: torch.Tensor, far: torch.Tensor, num_samples: int, stratified: bool = False) -> torch.Tensor:
    """near / far [...,1] -> distances [...,N]: bin midpoints, or one uniform draw per bin when ``stratified``."""
    offs = torch.rand(*near.shape[:-1], num_samples, device=near.device, dtype=near.dtype) if stratified else 0.5
    frac = (torch.arange(num_samples, device=near.device, dtype=near.dtype) + offs) / num_samples
    return near + (far - near) * frac


def volume_rendering_alphas(densities: torch.Tensor, dists: torch.Tensor, dist_far: Optional[torch.Tensor] = None) -> torch.Tensor:
    """alpha_i = 1 - exp(-sigma_i * (d_{i+1} - d_i)); the last interval ends at ``dist_far`` (default: effectively infinity,
    which makes the alphas along a ray sum to full opacity)."""
    if dist_far is None:
        dist_far = torch.full_like(dists[..., :1, :], 1e10)
    edges = torch.cat([dists, dist_far], dim=-2)
    return 1 - torch.exp(-densities * (edges[..., 1:, :] - edges[..., :-1, :]))


def alpha_compositing_weights(alphas: torch.Tensor) -> torch.Tensor:
    """w_i = alpha_i * prod_{j<i} (1 - alpha_j), accumulated in fp32."""
    front = torch.cat([torch.zeros_like(alphas[..., :1, :]), alphas[..., :-1, :]], dim=-2)
    visibility = (1 - front.float()).cumprod(dim=-2).to(alphas.dtype)
    return alphas * visibility


def composite(quantities, weights: torch.Tensor) -> torch.Tensor:
    return (quantities * weights).sum(dim=-2)


def volume_render_rays(nerf: torch.nn.Module, center: torch.Tensor, ray_unit: torch.Tensor, near: torch.Tensor, far: torch.Tensor,
                       num_samples: int, stratified: bool = False, solid_background: bool = False
                       ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """``nerf(points [...,N,3], ray dirs [...,N,3]) -> (rgb [...,N,3], density [...,N,1])``.
    Returns (rgb [...,3], opacity [...,1], weights [...,N,1], points [...,N,3], dists [...,N])."""
    dists = sample_dists(near, far, num_samples, stratified)
    points = center[..., None, :] + ray_unit[..., None, :] * dists[..., None]
    dirs = ray_unit[..., None, :].expand_as(points).contiguous()
    rgbs, densities = nerf(points, dirs)
    alphas = volume_rendering_alphas(densities, dists[..., None], None if solid_background else far[..., None])
    weights = alpha_compositing_weights(alphas)
    return composite(rgbs, weights), composite(1.0, weights), weights, points, dists
