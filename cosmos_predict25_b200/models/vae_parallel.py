"""Row-sharded execution of the causal-Conv3d VAE decoder across a process group.

The reference decodes the whole latent on every rank (or on one) even when the diffusion transformer ran
context-parallel (cosmos_predict2/_src/predict2/models/text2world_model_rectified_flow.py:585,779-795), so on
8 GPUs seven of them idle through the decode. Here every rank decodes a horizontal band of the frame
(``H / P`` latent rows -> ``8 H / P`` pixel rows) and the result is exact, not tiled-with-overlap:

  * every spatial convolution (3x3x3 causal Conv3d, 3x3 Conv2d of the up-samplers) first swaps its boundary rows
    with the two neighbouring ranks and uses them in place of its zero padding along H (the outermost ranks keep
    zeros);
  * the single-head spatial attention of the middle block attends from the local rows to the keys / values of the
    whole frame (all-gather of k and v, 14k tokens x 384 channels per frame at 720p);
  * the encoder's stride-2 convolutions (zero padding on the bottom / right only) take one boundary row from the next rank;
  * everything else (RMS norm over channels, SiLU, nearest 2x up-sampling, causal time convolutions and their
    chunk-to-chunk caches) is local to a pixel column or a row and needs no communication.

The boundary rows are small (two rows per layer and chunk), so the exchange is a pair of point-to-point messages
per layer through ``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests).
"""

from __future__ import annotations

import contextlib
from typing import Optional, Tuple

import torch
import torch.distributed as dist

_active: Optional[Tuple[object, int, int]] = None  # (group, rank in group, group size)


def active() -> Optional[Tuple[object, int, int]]:
    return _active


@contextlib.contextmanager
def row_sharded(group):
    """Inside the context the decoder modules treat their input as this rank's band of rows (dim H)."""
    global _active
    prev = _active
    size = dist.get_world_size(group)
    _active = (group, dist.get_rank(group), size) if size > 1 else None
    try:
        yield
    finally:
        _active = prev


def _global(group, r: int) -> int:
    return dist.get_global_rank(group, r) if group is not None and group is not dist.group.WORLD else r


def exchange_rows(x: torch.Tensor, dim: int, n: int, top: bool = True, bottom: bool = True) -> torch.Tensor:
    """``x`` extended along ``dim`` by the last ``n`` rows of the previous rank (``top``) and the first ``n`` rows of the next
    one (``bottom``); zeros where there is no neighbour (they stand for the convolution's zero padding at the frame border).
    The messages always flow both ways (every rank runs the same exchange); a side that is switched off is just not attached."""
    if _active is None or n == 0:
        return x
    group, r, P = _active
    size = x.shape[dim]
    assert size >= n, "band thinner than the halo"
    first = x.narrow(dim, 0, n).contiguous()
    last = x.narrow(dim, size - n, n).contiguous()
    from_prev = torch.zeros_like(first)
    from_next = torch.zeros_like(last)
    ops = []
    if r > 0:
        ops.append(dist.P2POp(dist.isend, first, _global(group, r - 1), group))
        ops.append(dist.P2POp(dist.irecv, from_prev, _global(group, r - 1), group))
    if r < P - 1:
        ops.append(dist.P2POp(dist.isend, last, _global(group, r + 1), group))
        ops.append(dist.P2POp(dist.irecv, from_next, _global(group, r + 1), group))
    for req in dist.batch_isend_irecv(ops):
        req.wait()
    parts = ([from_prev] if top else []) + [x] + ([from_next] if bottom else [])
    return torch.cat(parts, dim)


def gather_tokens(x: torch.Tensor, dim: int) -> torch.Tensor:
    """Concatenate every rank's ``x`` along ``dim`` in rank order (rows of a frame in row-major order)."""
    if _active is None:
        return x
    group, _, P = _active
    parts = [torch.empty_like(x) for _ in range(P)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim)


def split_rows(x: torch.Tensor, dim: int, group) -> torch.Tensor:
    """This rank's band of ``x`` along ``dim``."""
    P, r = dist.get_world_size(group), dist.get_rank(group)
    assert x.shape[dim] % P == 0, f"{x.shape[dim]} rows do not divide over {P} ranks"
    n = x.shape[dim] // P
    return x.narrow(dim, r * n, n).contiguous()


def can_shard(latent_rows: int, group) -> bool:
    if group is None or not dist.is_available() or not dist.is_initialized():
        return False
    P = dist.get_world_size(group)
    return P > 1 and latent_rows % P == 0 and latent_rows // P >= 1


def encode_row_sharded(encode_fn, video: torch.Tensor, group) -> torch.Tensor:
    """Run ``encode_fn`` (pixels [B,3,T,H,W] -> latent [B,C,T',H/8,W/8]) on this rank's band of pixel rows and gather the
    latent rows on every rank. Band heights must stay even through the three stride-2 stages: H divisible by 8 * ranks."""
    band = split_rows(video, 3, group)
    with row_sharded(group):
        lat = encode_fn(band).contiguous()
    parts = [torch.empty_like(lat) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, lat, group=group)
    return torch.cat(parts, 3)


def decode_row_sharded(decode_fn, latent: torch.Tensor, group, dst: Optional[int] = None) -> Optional[torch.Tensor]:
    """Run ``decode_fn`` (latent [B,C,T,h,w] -> pixels [B,3,T',8h,8w]) on this rank's band of latent rows with halo
    exchange between neighbours, then assemble the frame. With ``dst`` (a rank of the group) only that rank
    receives the video and the others return None; otherwise every rank gets it."""
    P, r = dist.get_world_size(group), dist.get_rank(group)
    band = split_rows(latent, 3, group)
    with row_sharded(group):
        out = decode_fn(band).contiguous()
    if dst is None:
        parts = [torch.empty_like(out) for _ in range(P)]
        dist.all_gather(parts, out, group=group)
        return torch.cat(parts, 3)
    parts = [torch.empty_like(out) for _ in range(P)] if r == dst else None
    dist.gather(out, parts, dst=_global(group, dst), group=group)
    return torch.cat(parts, 3) if r == dst else None
