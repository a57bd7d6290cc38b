"""Self-describing result records: every JSON names its git commit, environment, seed and command.

Counterpart of ``scripts/bench/record.py:17-72``.
"""

from __future__ import annotations

import datetime as _dt
import json
import os
import platform
import socket
import subprocess
import sys
from importlib import import_module, metadata
from pathlib import Path

REPO = Path(__file__).resolve().parents[2]


def _git(*args: str, repo: Path = REPO) -> str:
    try:
        return subprocess.run(["git", *args], cwd=repo, capture_output=True, text=True, timeout=10).stdout.strip()
    except (OSError, subprocess.SubprocessError):
        return ""


def git_info(repo: Path = REPO) -> dict:
    return {"sha": _git("rev-parse", "HEAD", repo=repo), "dirty": bool(_git("status", "--porcelain", "--untracked-files=no", repo=repo))}


def _version(module: str):
    """Installed version without importing the package (importing an inference engine takes seconds)."""
    try:
        return metadata.version(module)
    except metadata.PackageNotFoundError:
        pass
    try:
        return getattr(import_module(module), "__version__", None) if module == "moeflow_b200" else None
    except Exception:
        return None


def env_info() -> dict:
    info = {
        "hostname": socket.gethostname(),
        "python": platform.python_version(),
        "platform": platform.platform(),
        "job_id": os.environ.get("SLURM_JOB_ID") or os.environ.get("MOEFLOW_JOBID"),
        "cuda_visible_devices": os.environ.get("CUDA_VISIBLE_DEVICES"),
    }
    try:
        import torch

        info.update(torch=torch.__version__, cuda=torch.version.cuda)
        if torch.cuda.is_available():
            info.update(
                gpu=torch.cuda.get_device_name(),
                gpu_count_visible=torch.cuda.device_count(),
                nccl=".".join(str(v) for v in torch.cuda.nccl.version()),
            )
    except ImportError:
        pass
    for mod in ("triton", "vllm", "flashinfer"):
        info[mod] = _version(mod)
    info["moeflow_b200"] = _version("moeflow_b200")
    return info


def make_record(kind: str, config: dict, results: dict, seed: int | None = None, complete: bool = True) -> dict:
    return {
        "kind": kind,
        "created": _dt.datetime.now().astimezone().isoformat(timespec="seconds"),
        "complete": complete,
        "git": git_info(),
        "env": env_info(),
        "seed": seed,
        "command": [sys.executable, *sys.argv],
        "config": config,
        "results": results,
    }


def write_record(path: str | Path, record: dict) -> Path:
    """Write atomically (temp file + rename) so that an incremental record survives a later hang."""
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_suffix(path.suffix + ".tmp")
    tmp.write_text(json.dumps(record, indent=1, default=str))
    tmp.replace(path)
    return path
