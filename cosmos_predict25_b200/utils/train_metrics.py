"""Throughput accounting: parameter / FLOP counts, peak FLOP/s per device, model FLOPs utilisation, memory monitor.

Parity targets: ``get_num_params`` / ``get_num_flop_per_token`` / ``get_peak_flops`` / ``Color``
(cosmos_predict2/_src/reason1/parallelisms/torchtitan_utilts.py:267-350) and ``DeviceMemoryMonitor``
(cosmos_predict2/_src/reason1/parallelisms/metrics.py:48-107). The B200 entry is the dense bf16 figure (2.25 PFLOP/s).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


def get_num_params(model: torch.nn.Module, exclude_embedding: bool = False) -> int:
    n = sum(p.numel() for p in model.parameters())
    if exclude_embedding:
        n -= sum(p.numel() for m in model.modules() if isinstance(m, torch.nn.Embedding) for p in m.parameters())
    return n


def get_num_flop_per_token(num_params: int, num_layers: int, num_heads: int, head_dim: int, seq_len: int) -> int:
    """Training FLOPs per token of a decoder: 6 per parameter (fwd + bwd of every matmul) + 12 * L * H * d * S for attention."""
    return 6 * num_params + 12 * num_layers * num_heads * head_dim * seq_len


def dit_flop_per_sample(model_channels: int, num_blocks: int, seq_len: int, ctx_len: int = 512, mlp_ratio: float = 4.0,
                        training: bool = True) -> float:
    """Analytic FLOPs of the Cosmos DiT for one sample of ``seq_len`` tokens (self-attention dominates at 84k tokens)."""
    D, S = model_channels, seq_len
    proj = 2 * S * D * D * 4 + 2 * S * D * D * 2 + 2 * ctx_len * D * D * 2          # self q,k,v,o + cross q,o + cross k,v
    mlp = 2 * S * D * D * mlp_ratio * 2
    attn = 4 * S * S * D + 4 * S * ctx_len * D
    fwd = num_blocks * (proj + mlp + attn)
    return fwd * (3.0 if training else 1.0)


PEAK_BF16_FLOPS = {"B200": 2.25e15, "GB200": 2.5e15, "H200": 989e12, "H100 NVL": 835e12, "H100 PCIe": 756e12, "H100": 989e12,
                   "A100": 312e12, "L40S": 362e12}


def get_peak_flops(device_name: str) -> float:
    for key, val in PEAK_BF16_FLOPS.items():
        if key in device_name:
            return val
    return 312e12


def mfu(flops_per_step: float, step_seconds: float, n_gpus: int, peak_flops: float) -> float:
    return flops_per_step / (step_seconds * n_gpus * peak_flops)


@dataclass
class DeviceMemStats:
    max_active_gib: float
    max_active_pct: float
    max_reserved_gib: float
    max_reserved_pct: float
    num_alloc_retries: int
    num_ooms: int


class DeviceMemoryMonitor:
    def __init__(self, device: str = "cuda:0"):
        self.device = torch.device(device)
        self.enabled = torch.cuda.is_available() and self.device.type == "cuda"
        if self.enabled:
            self.device_name = torch.cuda.get_device_name(self.device)
            self.device_capacity = torch.cuda.get_device_properties(self.device).total_memory
            torch.cuda.reset_peak_memory_stats(self.device)
            torch.cuda.empty_cache()
        else:
            self.device_name, self.device_capacity = "cpu", 1

    @staticmethod
    def _gib(b: float) -> float:
        return b / (1024 ** 3)

    def get_peak_stats(self) -> DeviceMemStats:
        if not self.enabled:
            return DeviceMemStats(0, 0, 0, 0, 0, 0)
        info = torch.cuda.memory_stats(self.device)
        act, res = info.get("active_bytes.all.peak", 0), info.get("reserved_bytes.all.peak", 0)
        return DeviceMemStats(self._gib(act), 100 * act / self.device_capacity, self._gib(res), 100 * res / self.device_capacity,
                              info.get("num_alloc_retries", 0), info.get("num_ooms", 0))

    def reset_peak_stats(self):
        if self.enabled:
            torch.cuda.reset_peak_memory_stats(self.device)


class Color:
    black, red, green, yellow, blue, magenta, cyan, white, reset = ("\033[30m", "\033[31m", "\033[32m", "\033[33m", "\033[34m", "\033[35m",
                                                                    "\033[36m", "\033[37m", "\033[39m")


class NoColor:
    black = red = green = yellow = blue = magenta = cyan = white = reset = ""
