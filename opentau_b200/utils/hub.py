"""Checkpoint location helpers: local directories and ``repo_id@revision`` tags.

The ``@`` convention follows the reference (OpenTau ``src/opentau/utils/hub.py:45-107``): a bare
integer revision ``repo@40`` means the branch ``step-000040``-style tag is requested.  This build
runs without network access, so hub ids resolve only through the local cache directory
``$HF_OPENTAU_HOME/<repo_id>[/<revision>]``.
"""

from __future__ import annotations

import os
import re
from pathlib import Path

from ..constants import HF_OPENTAU_HOME


_HUB_REPO_ID = re.compile(r"^[A-Za-z0-9_][A-Za-z0-9._\-]*(?:/[A-Za-z0-9._\-]+)?$")


def split_repo_revision(name, revision: str | None = None) -> tuple[str | None, str | None]:
    """``"org/repo@rev"`` -> ``("org/repo", "rev")`` (reference ``src/opentau/utils/hub.py:45-107``).

    Training runs are published as one repository per run with every saved step as a tag, so ``org/run@6000`` names
    step 6000 and a bare ``org/run`` the latest one.  A file-system path is never split (checkpoint directories may
    contain "@"): an existing path, or a string whose part before the "@" is not a well-formed repository id, comes
    back unchanged, so that a moved checkpoint fails on its real path and not as a repository lookup.  Idempotent
    (``split(*split(x)) == split(x)``): an outer loader may split and hand ``(repo, revision)`` to an inner one.
    A spec that pins ``@rev`` together with a DIFFERENT explicit ``revision`` is an error."""
    if name is None:
        return None, revision
    spec = str(name)
    if not spec or os.path.exists(spec):
        return spec, revision
    head, sep, tail = spec.partition("@")
    if not sep or not tail or not _HUB_REPO_ID.match(head) or os.path.exists(head):
        if sep and not tail and _HUB_REPO_ID.match(head):
            raise ValueError(f"malformed repo tag {spec!r}: expected 'repo_id@revision'")
        return spec, revision
    if revision is not None and revision != tail:
        raise ValueError(f"conflicting revisions for {spec!r}: the path pins '@{tail}' but revision={revision!r} was "
                         "also passed; give only one")
    return head, tail


def format_repo_revision(repo_id, revision: str | None) -> str:
    """Inverse of :func:`split_repo_revision` for messages and logs."""
    return f"{repo_id}@{revision}" if revision else str(repo_id)


def revision_dir_names(revision: str) -> list[str]:
    """Directory names under which a revision may sit in the local cache: the tag as given, and for a bare step
    number also ``step-<six digits>`` (how this framework's own exporter lays steps out)."""
    names = [revision]
    if revision.isdigit():
        names.append(f"step-{int(revision):06d}")
    return names


def cached_revision_dir(repo_dir: Path, revision: str | None) -> Path:
    """``repo_dir`` itself without a revision; else the first existing candidate of :func:`revision_dir_names`, or
    (none existing) the LAST candidate, so that error messages name the canonical directory."""
    if not revision:
        return repo_dir
    cands = [repo_dir / n for n in revision_dir_names(revision)]
    return next((c for c in cands if c.is_dir()), cands[-1])


def resolve_local_or_hub(name: str, filename: str | None = None) -> Path:
    """Returns the local path of ``name`` (a directory, a file, or a cached hub repo)."""
    p = Path(name)
    if p.is_file():
        return p
    if p.is_dir():
        return p / filename if filename else p
    repo, rev = split_repo_revision(name)
    cached = cached_revision_dir(HF_OPENTAU_HOME / repo, rev)
    if cached.is_dir():
        return cached / filename if filename else cached
    raise FileNotFoundError(
        f"{name!r} is not a local path and is not in the local cache ({cached}); "
        "downloading from the hub needs network access, which this installation does not assume")


class HubMixin:
    """``save_pretrained(dir, push_to_hub=...)`` / ``push_to_hub(repo_id, ...)`` for anything that implements
    ``_save_pretrained(dir)`` (policies, configs): lighter than ``huggingface_hub.ModelHubMixin`` and with fewer
    assumptions about the subclass (reference ``src/opentau/utils/hub.py:119-296``).  Uploading needs network access and
    the ``huggingface_hub`` package; the upload call is looked up at call time so tests can substitute it."""

    def save_pretrained(self, save_directory: str | Path, *, repo_id: str | None = None, push_to_hub: bool = False,
                        card_kwargs: dict | None = None, **push_to_hub_kwargs) -> str | None:
        """Writes the object into ``save_directory``; with ``push_to_hub`` also uploads it (``repo_id`` defaults to the
        directory's name) and returns the commit URL."""
        save_directory = Path(save_directory)
        save_directory.mkdir(parents=True, exist_ok=True)
        self._save_pretrained(save_directory)
        if push_to_hub:
            return self.push_to_hub(repo_id=repo_id or save_directory.name, card_kwargs=card_kwargs, **push_to_hub_kwargs)
        return None

    def _save_pretrained(self, save_directory: Path) -> None:
        raise NotImplementedError

    def default_commit_message(self) -> str:
        name = type(self).__name__
        return "Upload policy" if "Policy" in name else "Upload config" if "Config" in name else f"Upload {name}"

    def push_to_hub(self, repo_id: str, *, commit_message: str | None = None, private: bool | None = None,
                    token: str | None = None, branch: str | None = None, create_pr: bool | None = None,
                    allow_patterns=None, ignore_patterns=None, delete_patterns=None, card_kwargs: dict | None = None,
                    api=None) -> str:
        """Saves into a temporary directory and uploads that folder as ONE commit; returns the commit's URL.
        ``allow_patterns`` / ``ignore_patterns`` filter the files, ``delete_patterns`` removes remote files in the same
        commit, ``branch`` / ``create_pr`` choose where it lands.  ``api``: an ``HfApi``-like object (default: a new
        ``huggingface_hub.HfApi(token=token)``)."""
        from tempfile import TemporaryDirectory
        if api is None:
            from huggingface_hub import HfApi
            api = HfApi(token=token)
        created = api.create_repo(repo_id=repo_id, private=private, exist_ok=True)
        repo_id = getattr(created, "repo_id", repo_id)
        with TemporaryDirectory(ignore_cleanup_errors=True) as tmp:
            saved = Path(tmp) / repo_id
            self.save_pretrained(saved, card_kwargs=card_kwargs)
            return api.upload_folder(repo_id=repo_id, repo_type="model", folder_path=saved,
                                     commit_message=commit_message or self.default_commit_message(), revision=branch,
                                     create_pr=create_pr, allow_patterns=allow_patterns, ignore_patterns=ignore_patterns,
                                     delete_patterns=delete_patterns)
