"""Result records that describe themselves: what ran (command, configuration, seed), on what (host, GPU,
library versions) and from which source state (git commit, dirty flag), next to the results.

The environment is gathered by a list of small *probes*; each returns a dict of facts or nothing when its
subject is absent (no torch, no GPU, package not installed), so a record can always be written.  Files are
replaced atomically, which lets a benchmark rewrite its record after every data point (``complete: false``
until the end) without ever leaving a half-written file behind.  Same record fields as
``scripts/bench/record.py:17-72`` of the reference, plus ``complete``.
"""

from __future__ import annotations

import json
import os
import platform
import socket
import subprocess
import sys
import tempfile
from datetime import datetime
from functools import lru_cache
from importlib import metadata
from pathlib import Path
from typing import Callable

REPO = Path(__file__).resolve().parents[2]
TRACKED_PACKAGES = ("triton", "vllm", "flashinfer", "moeflow_b200")


# ---- source state -------------------------------------------------------------------------------------
def _git_output(repo: Path, *args: str) -> str:
    try:
        done = subprocess.run(("git", "-C", str(repo), *args), capture_output=True, text=True, timeout=10)
    except (OSError, subprocess.SubprocessError):
        return ""
    return done.stdout.strip() if done.returncode == 0 else ""


def git_info(repo: Path = REPO) -> dict:
    """Commit hash and whether tracked files differ from it (empty hash outside a checkout)."""
    changed = _git_output(repo, "status", "--porcelain", "--untracked-files=no")
    return {"sha": _git_output(repo, "rev-parse", "HEAD"), "dirty": changed != ""}


# ---- environment probes -------------------------------------------------------------------------------
def _host_facts() -> dict:
    return {
        "hostname": socket.gethostname(),
        "python": platform.python_version(),
        "platform": platform.platform(),
        "job_id": os.environ.get("SLURM_JOB_ID") or os.environ.get("MOEFLOW_JOBID"),
        "cuda_visible_devices": os.environ.get("CUDA_VISIBLE_DEVICES"),
    }


def _torch_facts() -> dict:
    try:
        import torch
    except ImportError:
        return {}
    facts = {"torch": torch.__version__, "cuda": torch.version.cuda}
    if torch.cuda.is_available():
        facts["gpu"] = torch.cuda.get_device_name()
        facts["gpu_count_visible"] = torch.cuda.device_count()
        facts["nccl"] = ".".join(str(part) for part in torch.cuda.nccl.version())
    return facts


def _package_version(name: str) -> str | None:
    """From the installed metadata: importing an inference engine just to ask its version takes seconds."""
    try:
        return metadata.version(name)
    except metadata.PackageNotFoundError:
        pass
    if name == "moeflow_b200":  # run from a source tree
        from .. import __version__

        return __version__
    return None


def _package_facts() -> dict:
    return {name: _package_version(name) for name in TRACKED_PACKAGES}


PROBES: tuple[Callable[[], dict], ...] = (_host_facts, _torch_facts, _package_facts)


@lru_cache(maxsize=1)
def _environment() -> tuple:
    facts: dict = {}
    for probe in PROBES:
        facts.update(probe())
    return tuple(facts.items())


def env_info() -> dict:
    """The environment facts (gathered once per process)."""
    return dict(_environment())


# ---- records --------------------------------------------------------------------------------------------
def make_record(kind: str, config: dict, results: dict, seed: int | None = None, complete: bool = True) -> dict:
    header = {"kind": kind, "created": datetime.now().astimezone().isoformat(timespec="seconds"), "complete": complete}
    provenance = {"git": git_info(), "env": env_info(), "seed": seed, "command": [sys.executable, *sys.argv]}
    return {**header, **provenance, "config": config, "results": results}


def write_record(path: str | Path, record: dict) -> Path:
    """Serialise next to the target and rename over it: readers see the old file or the new one, never a part."""
    target = Path(path)
    target.parent.mkdir(parents=True, exist_ok=True)
    handle, scratch = tempfile.mkstemp(prefix=target.name + ".", suffix=".part", dir=target.parent)
    try:
        with os.fdopen(handle, "w") as sink:
            json.dump(record, sink, indent=1, default=str)
        os.replace(scratch, target)
    except BaseException:
        if os.path.exists(scratch):
            os.unlink(scratch)
        raise
    return target
