"""Checkpoint location helpers: local directories and ``repo_id@revision`` tags.

The ``@`` convention follows the reference (OpenTau ``src/opentau/utils/hub.py:45-107``): a bare
integer revision ``repo@40`` means the branch ``step-000040``-style tag is requested.  This build
runs without network access, so hub ids resolve only through the local cache directory
``$HF_OPENTAU_HOME/<repo_id>[/<revision>]``.
"""

from __future__ import annotations

import os
from pathlib import Path

from ..constants import HF_OPENTAU_HOME


def split_repo_revision(name: str) -> tuple[str, str | None]:
    """``"org/repo@rev"`` -> ``("org/repo", "rev")``; paths that exist on disk are never split."""
    if os.path.exists(name) or "@" not in name:
        return name, None
    repo, rev = name.rsplit("@", 1)
    if not repo or not rev:
        raise ValueError(f"malformed repo tag {name!r}: expected 'repo_id@revision'")
    if rev.isdigit():
        rev = f"step-{int(rev):06d}"
    return repo, rev


def resolve_local_or_hub(name: str, filename: str | None = None) -> Path:
    """Returns the local path of ``name`` (a directory, a file, or a cached hub repo)."""
    p = Path(name)
    if p.is_file():
        return p
    if p.is_dir():
        return p / filename if filename else p
    repo, rev = split_repo_revision(name)
    cached = HF_OPENTAU_HOME / repo
    if rev:
        cached = cached / rev
    if cached.is_dir():
        return cached / filename if filename else cached
    raise FileNotFoundError(
        f"{name!r} is not a local path and is not in the local cache ({cached}); "
        "downloading from the hub needs network access, which this installation does not assume")
