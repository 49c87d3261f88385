"""Symmetric (peer-mapped) device memory and the device-side barrier used by the fused collectives.

Every rank of a group allocates the same-sized arena; after a rendezvous each rank knows the virtual
address of every peer's arena in its own address space, so kernels can load from / store to a peer's
buffer over NVLink with ordinary ld/st. The handle exchange is done by torch's symmetric-memory
allocator (plumbing); everything that moves data is a kernel of this package
(``ops/csrc/peer.cu``). NVSwitch multicast objects are not created: the kernels use plain peer
accesses only, and a rank that exits never leaves a multicast binding behind.

``PeerContext.barrier()`` enqueues a 1-block kernel on the current stream: it publishes an epoch into
every peer's flag word, then waits - with a bound - until every peer has published the same epoch. If
the bound is hit the kernel records an error code (readable with ``check()``) and returns; the host
raises, the GPU context stays usable.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import native

os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")


@dataclass
class SymmetricTensor:
    """A local tensor carved from a symmetric arena plus the address of the same bytes on every peer."""

    tensor: torch.Tensor
    ptrs: List[int]


CANARY_BYTES = 256
CANARY_VALUE = 0xA5
CANARY_SLOTS = 4096           # head-room (in allocations) that a guarded arena adds to the size its owner asked for


class BumpArena:
    """Bump allocator over one uint8 buffer whose address on every peer is known (256-byte aligned tensors).

    With ``canary`` every allocation is followed by a 256-byte guard filled with 0xA5; ``check_canaries()`` reads the guards back
    and raises if a kernel (this rank's or a peer's: peers store into this memory) wrote past the end of a buffer. The guards
    cost one small device-to-host copy per check and nothing inside the kernels."""

    def __init__(self, buf: torch.Tensor, base_ptrs: List[int], canary: bool = False):
        self.buf = buf
        self.nbytes = buf.numel()
        self.base_ptrs = base_ptrs
        self.canary = canary
        self.offset = 0
        self._guards: List[Tuple[int, int, str]] = []      # (offset of the guard, bytes of the allocation before it, dtype)

    def alloc(self, numel: int, dtype: torch.dtype, zero: bool = True) -> SymmetricTensor:
        esize = torch.empty((), dtype=dtype).element_size()
        nbytes = (numel * esize + 255) // 256 * 256
        need = nbytes + (CANARY_BYTES if self.canary else 0)
        if self.offset + need > self.nbytes:
            raise MemoryError(f"symmetric arena exhausted: need {need} more bytes, {self.nbytes - self.offset} left")
        t = self.buf[self.offset: self.offset + numel * esize].view(dtype)
        if zero:
            t.zero_()
        st = SymmetricTensor(t, [p + self.offset for p in self.base_ptrs])
        self.offset += nbytes
        if self.canary:
            # the guard starts at the 256-byte boundary after the data: the alignment slack before it is not watched
            self.buf[self.offset: self.offset + CANARY_BYTES].fill_(CANARY_VALUE)
            self._guards.append((self.offset, numel * esize, str(dtype)))
            self.offset += CANARY_BYTES
        return st

    def check_canaries(self) -> None:
        if not self._guards:
            return
        idx = torch.tensor([g[0] for g in self._guards], device=self.buf.device)
        words = self.buf[(idx[:, None] + torch.arange(CANARY_BYTES, device=self.buf.device)[None, :])].cpu()
        bad = (words != CANARY_VALUE).any(dim=1).nonzero().flatten().tolist()
        if bad:
            i = bad[0]
            off, nbytes, dtype = self._guards[i]
            first = int((words[i] != CANARY_VALUE).nonzero()[0])
            raise RuntimeError(f"symmetric arena: allocation #{i} ({nbytes} bytes of {dtype}, guard at offset {off}) was overrun: "
                               f"guard byte {first} holds {int(words[i][first]):#x}; {len(bad)} guard(s) damaged in total")


class SymmetricArena(BumpArena):
    """One symmetric allocation per rank, bump-allocated into tensors (256-byte aligned). ``canary`` (default: the environment
    variable ``COSMOS_B200_CANARY=1``) adds guard words behind every tensor, see ``BumpArena``."""

    def __init__(self, nbytes: int, group, device: torch.device, canary: Optional[bool] = None):
        import torch.distributed._symmetric_memory as symm_mem

        if canary is None:
            canary = os.environ.get("COSMOS_B200_CANARY", "0") == "1"
        self.group = group
        self.device = device
        nbytes = (nbytes + 255) // 256 * 256 + (CANARY_BYTES * CANARY_SLOTS if canary else 0)
        buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(buf, group if group is not None else dist.group.WORLD)
        self.rank = self.handle.rank
        self.world = self.handle.world_size
        super().__init__(buf, [int(p) for p in self.handle.buffer_ptrs], canary)
        assert self.base_ptrs[self.rank] == self.buf.data_ptr(), "symmetric arena: local pointer mismatch"


class PeerContext:
    """Rank/size of a group, a flag word array in symmetric memory and the epoch counter of its barrier."""

    def __init__(self, group, device: torch.device, arena: Optional[SymmetricArena] = None, arena_bytes: int = 1 << 20):
        self.group = group if group is not None else dist.group.WORLD
        self.device = device
        self.arena = arena or SymmetricArena(arena_bytes, self.group, device)
        self.rank, self.world = self.arena.rank, self.arena.world
        assert self.world <= 8, "peer kernels support up to 8 ranks (one NVSwitch domain)"
        self.flags = self.arena.alloc(64, torch.int32)
        self.epoch = 0
        self.timeout_s = float(os.environ.get("COSMOS_B200_PEER_TIMEOUT_S", "30"))  # bound of device-side waits
        self.ops = native.load()
        torch.cuda.synchronize(device)
        dist.barrier(self.group)  # flag words are zeroed everywhere before the first device barrier

    def barrier(self) -> None:
        self.epoch += 1
        self.ops.peer_barrier(self.flags.ptrs, self.rank, self.epoch, self.device.index, int(self.timeout_s * 1e6))
        native.count_launch()

    def check(self) -> None:
        """Host-side check of the device error word (synchronises the device)."""
        code = int(self.ops.kernel_error(self.device.index, True))
        self.arena.check_canaries()
        if code != 0:
            raise RuntimeError(f"a peer-memory kernel gave up waiting (error code {code}): rank {code - 100} did not arrive"
                               if code >= 100 else f"kernel error code {code}")


class PeerAllToAll:
    """Ulysses exchanges over peer memory for one context-parallel group.

    seq_to_head: every 16-byte vector of x [B, S_loc, H, D] is stored straight into the staging buffer of
    the rank that owns its head (optionally after per-head RMSNorm + RoPE: the q/k epilogue chain and the
    exchange are one kernel). head_to_seq: each rank reads its token rows of every peer's staged
    attention output. Staging buffers rotate so that a buffer is rewritten only two exchanges later,
    after a barrier every rank has passed."""

    def __init__(self, ctx: PeerContext, max_elems: int, n_slots: int = 8):
        self.ctx = ctx
        self.ops = ctx.ops
        self.slots = [ctx.arena.alloc(max_elems, torch.bfloat16, zero=False) for _ in range(n_slots)]
        self.max_elems = max_elems
        self.cursor = 0

    def _next(self, numel: int) -> SymmetricTensor:
        assert numel <= self.max_elems, f"exchange of {numel} elements exceeds the staging size {self.max_elems}"
        s = self.slots[self.cursor]
        self.cursor = (self.cursor + 1) % len(self.slots)
        return s

    def scatter_heads(self, xs, norm_weights=None, rope=None, eps: float = 1e-6, copy_out: bool = True):
        """Exchange a list of [B, S_loc, H, D] tensors with one barrier. ``norm_weights[i]`` (or None)
        applies per-head RMSNorm (+RoPE when ``rope`` is given) to tensor i on the way out.
        Returns (list of [B, S_loc*P, H/P, D] tensors, list of rstd or None). With ``copy_out`` the results
        are copied out of the rotating staging buffers (needed whenever they are kept for a backward pass);
        without it they alias the staging memory and must be consumed before eight more exchanges."""
        P, r = self.ctx.world, self.ctx.rank
        outs, rstds = [], []
        cos, sin = rope.cos_sin() if rope is not None else (None, None)
        for i, x in enumerate(xs):
            B, S, H, D = x.shape
            slot = self._next(x.numel())
            w = norm_weights[i] if norm_weights is not None else None
            rstd = self.ops.a2a_scatter_heads_peer(x.contiguous(), slot.ptrs, w, cos if w is not None else None,
                                                   sin if w is not None else None, r, eps)
            native.count_launch()
            outs.append(slot.tensor[: x.numel()].view(B, S * P, H // P, D))
            rstds.append(rstd.view(B, S, H) if w is not None else None)
        self.ctx.barrier()
        if copy_out:
            outs = [o.clone() for o in outs]
        return outs, rstds

    def project_scatter_heads(self, x2d: torch.Tensor, weights, norm_weights, rope, B: int, S: int, eps: float = 1e-6,
                              keep_for_backward: bool = False):
        """``x2d [B*S, K] @ w_i^T`` for every projection weight ``w_i [H*128, K]`` with the sequence->head exchange
        as the GEMM epilogue: accumulator rows leave TMEM normalised (``norm_weights[i]``) and rotated (``rope``)
        and are stored straight into the owning rank's staging buffer, so the projected activations never exist
        in sequence layout. One barrier for all projections. The results alias the rotating staging buffers
        (consume them before eight more exchanges). ``keep_for_backward`` (training): the results are copied out of the
        staging buffers, and for every normalised projection the epilogue also stores the raw projection and the reciprocal
        RMS of every (token, head) locally; returns (heads, raws, rstds) then."""
        P, r = self.ctx.world, self.ctx.rank
        cos, sin = rope.cos_sin() if rope is not None else (None, None)
        outs, raws, rstds = [], [], []
        for w, nw in zip(weights, norm_weights):
            H = w.shape[0] // 128
            numel = B * S * w.shape[0]
            slot = self._next(numel)
            raw, rstd = self.ops.gemm_scatter_heads_peer(x2d, w, slot.ptrs, nw, cos if nw is not None else None,
                                                         sin if nw is not None else None, S, r, eps,
                                                         keep_for_backward and nw is not None)
            native.count_launch()
            outs.append(slot.tensor[:numel].view(B, S * P, H // P, 128))
            raws.append(raw.view(B, S, H, 128) if raw.numel() else None)
            rstds.append(rstd.view(B, S, H) if rstd.numel() else None)
        self.ctx.barrier()
        if keep_for_backward:
            return [o.clone() for o in outs], raws, rstds
        return outs

    def attention_scatter_seq(self, qh: torch.Tensor, kh: torch.Tensor, vh: torch.Tensor, scale: float) -> torch.Tensor:
        """Attention on this rank's heads of the gathered sequence ([B, S_loc*P, H/P, 128]) with the head->sequence
        exchange as the kernel's output store: each finished query tile is written straight into the sequence shard
        of the rank that owns its rows. Returns this rank's [B, S_loc, H, 128] (aliases a rotating staging buffer).
        The trailing barrier publishes the peers' stores; the buffer is rewritten two attention calls later, behind
        at least one more barrier, so no barrier is needed after the consumer."""
        P, r = self.ctx.world, self.ctx.rank
        B, SP, Hl, D = qh.shape
        slot = self._next(qh.numel())
        self.ops.fa_fwd_scatter_seq_peer(qh, kh, vh, scale, slot.ptrs, r)
        native.count_launch()
        self.ctx.barrier()
        return slot.tensor[: qh.numel()].view(B, SP // P, Hl * P, D)

    def head_to_seq_many(self, xs):
        """``head_to_seq`` of several tensors with one pair of barriers (the three gradients of a q / k / v exchange)."""
        P, r = self.ctx.world, self.ctx.rank
        slots = []
        for x in xs:
            slot = self._next(x.numel())
            stage = slot.tensor[: x.numel()].view_as(x)
            if stage.data_ptr() != x.data_ptr():
                stage.copy_(x)
            slots.append(slot)
        self.ctx.barrier()
        outs = []
        for x, slot in zip(xs, slots):
            B, SP, Hl, D = x.shape
            outs.append(self.ops.a2a_gather_seq_peer(slot.ptrs, B, SP // P, Hl * P, D, r, x))
            native.count_launch()
        self.ctx.barrier()  # peers have finished reading this rank's stages before they are reused
        return outs

    def seq_to_head(self, x: torch.Tensor, copy_out: bool = True) -> torch.Tensor:
        return self.scatter_heads([x], copy_out=copy_out)[0][0]

    def head_to_seq(self, x: torch.Tensor) -> torch.Tensor:
        """[B, S_loc*P, H/P, D] (all tokens, local heads) -> [B, S_loc, H, D]."""
        P, r = self.ctx.world, self.ctx.rank
        B, SP, Hl, D = x.shape
        slot = self._next(x.numel())
        stage = slot.tensor[: x.numel()].view_as(x)
        if stage.data_ptr() != x.data_ptr():
            stage.copy_(x)
        self.ctx.barrier()
        out = self.ops.a2a_gather_seq_peer(slot.ptrs, B, SP // P, Hl * P, D, r, x)
        native.count_launch()
        self.ctx.barrier()  # peers have finished reading this rank's stage before it is reused
        return out
