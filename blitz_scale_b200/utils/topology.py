"""GPU / CPU topology of the box: which NUMA node and CPU cores sit next to each GPU, and how GPUs reach each other.

The reference maps each GPU to its nearest RDMA NIC from `nvidia-smi topo -m` + `ibv_devinfo`
(scripts/batch/rank_to_rnic.py:24-86) and binds ranks 0-3 / 4-7 to NUMA node 0 / 1 (src/server/disaggregate.cc).
On an NVSwitch box there is no NIC to choose; what remains useful is the CPU/NUMA affinity of each GPU (the
worker's host threads, pinned staging buffers and the disk loader should live there) and a check that every GPU
pair is connected by NVLink (the peer-memory kernels assume it).
"""
from __future__ import annotations

import os
import re
import subprocess
from dataclasses import dataclass, field
from typing import Dict, List, Optional


@dataclass
class GpuTopology:
    links: Dict[int, Dict[int, str]] = field(default_factory=dict)      # links[i][j] = "NV18", "PIX", "SYS", ...
    cpu_affinity: Dict[int, List[int]] = field(default_factory=dict)    # GPU -> CPU ids
    numa_node: Dict[int, int] = field(default_factory=dict)

    def all_nvlink(self) -> bool:
        return all(v.startswith("NV") for i, row in self.links.items() for j, v in row.items() if i != j)

    def nvlink_count(self, i: int, j: int) -> int:
        m = re.match(r"NV(\d+)", self.links.get(i, {}).get(j, ""))
        return int(m.group(1)) if m else 0


def _cpu_list(spec: str) -> List[int]:
    out: List[int] = []
    for part in spec.split(","):
        part = part.strip()
        if not part or part == "N/A":
            continue
        if "-" in part:
            a, b = part.split("-")
            out += list(range(int(a), int(b) + 1))
        else:
            out.append(int(part))
    return out


def parse_topo_matrix(text: str) -> GpuTopology:
    """Parse the table printed by `nvidia-smi topo -m`."""
    topo = GpuTopology()
    lines = [re.sub(r"\x1b\[[0-9;]*m", "", l) for l in text.splitlines()]
    header = next((l for l in lines if re.match(r"^\s*GPU0\b", l.strip()) or "\tGPU0" in l or l.strip().startswith("GPU0")), None)
    if header is None:
        return topo
    cols = re.split(r"\t+|\s{2,}", header.strip())
    gpu_cols = [c for c in cols if re.fullmatch(r"GPU\d+", c)]
    ncol = len(cols)
    for l in lines:
        m = re.match(r"^\s*GPU(\d+)\s+(.*)$", l)
        if not m or l is header:
            continue
        i = int(m.group(1))
        cells = re.split(r"\t+|\s{2,}", m.group(2).strip())
        topo.links[i] = {}
        for j, c in enumerate(gpu_cols):
            if j < len(cells):
                topo.links[i][int(c[3:])] = cells[j].strip()
        rest = dict(zip(cols[len(gpu_cols):], cells[len(gpu_cols):])) if ncol > len(gpu_cols) else {}
        aff = next((v for k, v in rest.items() if "CPU Affinity" in k), "")
        numa = next((v for k, v in rest.items() if "NUMA Affinity" in k), "")
        if aff:
            topo.cpu_affinity[i] = _cpu_list(aff)
        if numa and numa.strip().isdigit():
            topo.numa_node[i] = int(numa)
    return topo


def query_topology() -> Optional[GpuTopology]:
    try:
        out = subprocess.run(["nvidia-smi", "topo", "-m"], capture_output=True, text=True, timeout=20)
    except (OSError, subprocess.TimeoutExpired):
        return None
    return parse_topo_matrix(out.stdout) if out.returncode == 0 else None


def bind_to_gpu_cpus(gpu: int, topo: Optional[GpuTopology] = None) -> List[int]:
    """Restrict this process (and the threads it starts later) to the CPU cores next to `gpu`.  Returns the cores
    chosen, or [] when the topology is unknown (nothing is changed then)."""
    topo = topo or query_topology()
    cpus = (topo.cpu_affinity.get(gpu) if topo else None) or []
    allowed = set(os.sched_getaffinity(0))
    cpus = [c for c in cpus if c in allowed]
    if cpus:
        os.sched_setaffinity(0, cpus)
    return cpus
