"""Small debugging helpers (the reference's printGpuArray / cuda_memory_size / syncAndCheck, src/util/cuda_utils.h)."""
from __future__ import annotations

from typing import Dict

import torch


def gpu_memory_report(device=None) -> Dict[str, float]:
    """Free / total / allocated / reserved memory of one GPU in GB."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    free, total = torch.cuda.mem_get_info(dev)
    return {"free_gb": free / 1e9, "total_gb": total / 1e9, "allocated_gb": torch.cuda.memory_allocated(dev) / 1e9,
            "reserved_gb": torch.cuda.memory_reserved(dev) / 1e9}


def describe(t: torch.Tensor, name: str = "tensor", head: int = 8) -> str:
    """One line about a tensor: shape, dtype, finiteness, range and its first values (synchronises)."""
    f = t.detach().float().flatten()
    if f.numel() == 0:
        return f"{name}: empty {tuple(t.shape)} {t.dtype}"
    finite = torch.isfinite(f)
    body = f[finite]
    stats = (f"min {float(body.min()):.4g} max {float(body.max()):.4g} mean {float(body.mean()):.4g} "
             f"rms {float(body.pow(2).mean().sqrt()):.4g}") if body.numel() else "no finite values"
    return (f"{name}: {tuple(t.shape)} {t.dtype} on {t.device}, {int((~finite).sum())} non-finite, {stats}, "
            f"head {[round(float(x), 4) for x in f[:head]]}")


def sync_and_check(where: str = "") -> None:
    """Wait for the device and surface both CUDA errors and the kernels' own status word."""
    from .. import ops
    torch.cuda.synchronize()
    try:
        ops.check_status()
    except RuntimeError as e:
        raise RuntimeError(f"{where}: {e}") from e
