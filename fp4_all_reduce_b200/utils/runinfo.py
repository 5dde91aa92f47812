"""Fields that every measurement record carries so that a number can be traced to its machine and its sources.

The reference project's harness writes tag, node, GPU name, visible devices, NCCL version, time, PCI bus ids and the
memory clock into each JSON line (harness/fp4ar_bench.cu:131-139,423-428); this is the same idea plus the digest of
the native-source manifest.
"""
from __future__ import annotations

import hashlib
import os
import socket
import time
from pathlib import Path


def sources_digest() -> str:
    """First 16 hex digits of the sha256 of csrc/MANIFEST.sha256 ('' when the manifest is absent)."""
    man = Path(__file__).resolve().parent.parent / "csrc" / "MANIFEST.sha256"
    try:
        return hashlib.sha256(man.read_bytes()).hexdigest()[:16]
    except OSError:
        return ""


def run_info(device=None) -> dict:
    info = {"host": socket.gethostname(), "cvd": os.environ.get("CUDA_VISIBLE_DEVICES", ""),
            "time": time.strftime("%Y-%m-%dT%H:%M:%S"), "sources": sources_digest()}
    try:
        import torch

        info["torch"] = torch.__version__
        if torch.cuda.is_available():
            dev = device if device is not None else torch.cuda.current_device()
            p = torch.cuda.get_device_properties(dev)
            info["gpu"] = p.name
            info["sms"] = p.multi_processor_count
            info["pci_bus_id"] = getattr(p, "pci_bus_id", None)
            info["nccl"] = ".".join(map(str, torch.cuda.nccl.version()))
    except Exception:
        pass
    try:
        from .. import _native as N

        info["lib"] = (N.cuda().fp4ar_build_info() or b"").decode()
    except Exception:
        pass
    return info
