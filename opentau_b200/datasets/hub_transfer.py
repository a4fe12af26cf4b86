"""Moving LeRobot datasets between a local root and the Hugging Face hub
(reference ``src/opentau/datasets/lerobot_dataset.py:457-470, 1949-2117``).

Everything goes through a small client object (:class:`HubClient`) so that the transfer logic (which files, in what
order, what is skipped) can be exercised without a network: tests hand in a recording fake.  The default client wraps
``huggingface_hub``; on a machine without network access its calls fail with the library's own error, and nothing here
is on the training path unless a dataset root is missing files.

Rules that matter at scale:

* an episode SUBSET is fetched file by file with exact paths on a thread pool.  Handing thousands of explicit paths to a
  snapshot download as patterns costs minutes of pattern matching per call, long enough for the other ranks' collective
  to time out while they wait;
* files already on disk are never requested again (one metadata request per present file is enough to hit the hub's
  rate limit on a pre-downloaded dataset), and paths are de-duplicated first: in the v3.0 layout many episodes share one
  consolidated file and two threads must not fetch the same path;
* the WHOLE dataset is one snapshot download without patterns (nothing to match, O(1) listing calls);
* only the main process of each node transfers; the others wait at a barrier.
"""

from __future__ import annotations

import contextlib
import logging
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Any, Protocol

DOWNLOAD_MAX_WORKERS = 16
REPOCARD_NAME = "README.md"


class HubClient(Protocol):
    def snapshot_download(self, repo_id: str, *, revision: str | None, local_dir: Path, allow_patterns=None,
                          ignore_patterns=None) -> Any: ...

    def download_file(self, repo_id: str, filename: str, *, revision: str | None, local_dir: Path) -> Any: ...

    def create_repo(self, repo_id: str, *, private: bool) -> Any: ...

    def create_branch(self, repo_id: str, branch: str, *, revision: str | None) -> Any: ...

    def upload_folder(self, repo_id: str, folder: Path, *, revision: str | None, allow_patterns=None,
                      ignore_patterns=None, large: bool = False) -> Any: ...

    def file_exists(self, repo_id: str, filename: str, *, revision: str | None) -> bool: ...

    def upload_text(self, repo_id: str, filename: str, text: str, *, revision: str | None) -> Any: ...

    def retag(self, repo_id: str, tag: str, *, revision: str | None) -> Any: ...

    def list_refs(self, repo_id: str) -> tuple[list[str], list[str]]:
        """``(branch names, tag names)`` of the repository."""
        ...


class HuggingFaceHubClient:
    """The real thing (dataset repositories)."""

    def __init__(self):
        import huggingface_hub
        self._hub = huggingface_hub
        self._api = huggingface_hub.HfApi()

    def snapshot_download(self, repo_id, *, revision, local_dir, allow_patterns=None, ignore_patterns=None):
        return self._hub.snapshot_download(repo_id, repo_type="dataset", revision=revision, local_dir=local_dir,
                                           allow_patterns=allow_patterns, ignore_patterns=ignore_patterns)

    def download_file(self, repo_id, filename, *, revision, local_dir):
        return self._hub.hf_hub_download(repo_id=repo_id, filename=filename, repo_type="dataset", revision=revision,
                                         local_dir=local_dir)

    def create_repo(self, repo_id, *, private):
        return self._api.create_repo(repo_id=repo_id, private=private, repo_type="dataset", exist_ok=True)

    def create_branch(self, repo_id, branch, *, revision):
        return self._api.create_branch(repo_id=repo_id, branch=branch, revision=revision, repo_type="dataset", exist_ok=True)

    def upload_folder(self, repo_id, folder, *, revision, allow_patterns=None, ignore_patterns=None, large=False):
        kw = dict(repo_id=repo_id, folder_path=folder, repo_type="dataset", revision=revision,
                  allow_patterns=allow_patterns, ignore_patterns=ignore_patterns)
        return self._api.upload_large_folder(**kw) if large else self._api.upload_folder(**kw)

    def file_exists(self, repo_id, filename, *, revision):
        return self._api.file_exists(repo_id, filename, repo_type="dataset", revision=revision)

    def upload_text(self, repo_id, filename, text, *, revision):
        return self._api.upload_file(path_or_fileobj=text.encode(), path_in_repo=filename, repo_id=repo_id,
                                     repo_type="dataset", revision=revision)

    def retag(self, repo_id, tag, *, revision):
        with contextlib.suppress(Exception):           # the tag may not exist yet
            self._api.delete_tag(repo_id, tag=tag, repo_type="dataset")
        return self._api.create_tag(repo_id, tag=tag, revision=revision, repo_type="dataset")

    def list_refs(self, repo_id):
        refs = self._api.list_repo_refs(repo_id, repo_type="dataset")
        return [b.name for b in refs.branches], [t.name for t in refs.tags]


_CLIENT: list[HubClient] = []


def hub_client() -> HubClient:
    if not _CLIENT:
        _CLIENT.append(HuggingFaceHubClient())
    return _CLIENT[0]


def set_hub_client(client: HubClient | None) -> None:
    """Installs another client (tests, a mirror); ``None`` goes back to the default."""
    _CLIENT.clear()
    if client is not None:
        _CLIENT.append(client)


class ForwardCompatibilityError(Exception):
    """The repository only carries formats newer than this loader reads."""


class RevisionNotFoundError(Exception):
    """The repository carries no codebase-version ref (and no default branch to fall back to)."""


DEFAULT_BRANCHES = ("main", "master")


def _parse_version(ref) -> tuple[int, ...] | None:
    """``"v2.1"`` / ``"2.1"`` -> ``(2, 1)``; anything that is not a dotted number (a branch name) -> ``None``."""
    parts = str(ref).lstrip("v").split(".")
    if not parts or not all(p.isdigit() for p in parts):
        return None
    return tuple(int(p) for p in parts)


def _fmt_version(v: tuple[int, ...]) -> str:
    return "v" + ".".join(str(x) for x in v)


def get_repo_versions(repo_id: str) -> list[tuple[int, ...]]:
    """Branches and tags of the repository that parse as versions."""
    branches, tags = hub_client().list_refs(repo_id)
    return [v for v in (_parse_version(r) for r in [*branches, *tags]) if v is not None]


def get_safe_version(repo_id: str, version: str, read_ceiling: str | None = None,
                     allow_branch_fallback: bool = False) -> str:
    """The revision to download when ``version`` was asked for (reference ``src/opentau/datasets/utils.py:1004-1110``):

    1. the version itself when the repository carries it;
    2. else the newest ref of the same major with a minor not above it (with a warning when it is older);
    3. else the newest ref above it that the loader still reads (up to ``read_ceiling``, default: the newest
       supported format), e.g. a repository published only as v3.0 while v2.1 is the default target;
    4. else :class:`BackwardCompatibilityError` (only older majors) or :class:`ForwardCompatibilityError`.

    A repository without any version ref raises :class:`RevisionNotFoundError`, unless ``allow_branch_fallback`` (the
    caller pinned no revision) and a ``main`` / ``master`` branch exists, which is then used with a warning."""
    from .utils import SUPPORTED_VERSIONS, BackwardCompatibilityError
    target = _parse_version(version)
    if target is None:
        raise ValueError(f"{version!r} is not a codebase version")
    ceiling = _parse_version(read_ceiling) if read_ceiling else max(_parse_version(v) for v in SUPPORTED_VERSIONS)
    branches, tags = hub_client().list_refs(repo_id)
    versions = [v for v in (_parse_version(r) for r in [*branches, *tags]) if v is not None]
    if not versions:
        if allow_branch_fallback:
            for name in DEFAULT_BRANCHES:
                if name in branches:
                    logging.warning("%s has no codebase-version tag; defaulting to the %r branch", repo_id, name)
                    return name
        raise RevisionNotFoundError(
            f"{repo_id} must be tagged with its codebase version (the `codebase_version` of meta/info.json): "
            f"create that tag on the dataset repository, or pass an explicit `revision`")
    if target in versions:
        return _fmt_version(target)
    same_major = [v for v in versions if v[0] == target[0] and v[1:] <= target[1:]]
    if same_major:
        best = max(same_major)
        logging.warning("revision %s of %s not found, using %s", version, repo_id, _fmt_version(best))
        return _fmt_version(best)
    readable_newer = [v for v in versions if target < v <= ceiling]
    if readable_newer:
        return _fmt_version(max(readable_newer))
    older = [v for v in versions if v[0] < target[0]]
    if older:
        raise BackwardCompatibilityError(
            f"dataset {repo_id!r} is only published as {_fmt_version(max(older))}, which this loader does not read; "
            f"convert it first (datasets/v2/convert_dataset_v1_to_v2.py)")
    raise ForwardCompatibilityError(
        f"dataset {repo_id!r} is only available as {_fmt_version(min(v for v in versions if v > target))}; this "
        f"loader reads up to {_fmt_version(ceiling)}: update the framework")


def dataset_card(info: dict, tags: list[str] | None = None, license: str | None = "apache-2.0", **extra) -> str:
    """A minimal dataset card: front matter the hub indexes, then the ``info.json`` facts a reader needs first."""
    tag_list = ["LeRobot", *(tags or [])]
    front = ["---", f"license: {license}" if license else None, "task_categories:", "- robotics", "tags:",
             *[f"- {t}" for t in tag_list], "configs:", "- config_name: default", "  data_files: data/*/*.parquet", "---"]
    lines = [x for x in front if x is not None]
    lines += ["", "This dataset follows the LeRobot layout.", "", "| | |", "|---|---|"]
    for k in ("codebase_version", "robot_type", "control_mode", "fps", "total_episodes", "total_frames", "total_tasks"):
        if k in info:
            lines.append(f"| {k} | {info[k]} |")
    for k, v in extra.items():
        lines.append(f"| {k} | {v} |")
    return "\n".join(lines) + "\n"


def _on_main_process_then_barrier(fn):
    def inner(self, *a, **kw):
        from ..parallel import control
        try:
            if control.is_local_main_process():
                return fn(self, *a, **kw)
        finally:
            control.wait_for_everyone()
    inner.__doc__, inner.__name__ = fn.__doc__, fn.__name__
    return inner


class HubTransferMixin:
    """Needs ``repo_id``, ``root``, ``revision`` and, for the episode-wise calls, ``meta`` / ``episodes``."""

    def resolved_revision(self) -> str | None:
        """What is asked of the hub.  A pinned revision is used as it is, if it parses as a version after the same
        compatibility resolution; an unpinned one resolves from the current format, with the default branch as the
        last resort.  A client that cannot list refs (a plain mirror) leaves the revision as it is."""
        from .utils import CODEBASE_VERSION
        pinned = getattr(self, "revision", None)
        if pinned is not None and _parse_version(pinned) is None:
            return pinned                                   # a branch name or a commit hash
        cached = getattr(self, "_resolved_revision", None)
        if cached is not None:
            return cached
        if not hasattr(hub_client(), "list_refs"):
            return pinned
        rev = get_safe_version(self.repo_id, pinned or CODEBASE_VERSION, allow_branch_fallback=pinned is None)
        self._resolved_revision = rev
        return rev

    @_on_main_process_then_barrier
    def pull_from_repo(self, allow_patterns=None, ignore_patterns=None) -> None:
        hub_client().snapshot_download(self.repo_id, revision=self.resolved_revision(), local_dir=Path(self.root),
                                       allow_patterns=allow_patterns, ignore_patterns=ignore_patterns)

    @_on_main_process_then_barrier
    def download_files(self, files: list[str]) -> None:
        """The files of ``files`` that are not on disk yet, one exact-path request each, on a thread pool."""
        missing = list(dict.fromkeys(f for f in files if not (Path(self.root) / f).is_file()))
        if not missing:
            return
        logging.info("%s: %d of %d file(s) are not on disk; fetching them", self.repo_id, len(missing), len(files))
        client, rev, root = hub_client(), self.resolved_revision(), Path(self.root)
        with ThreadPoolExecutor(max_workers=DOWNLOAD_MAX_WORKERS) as pool:
            list(pool.map(lambda f: client.download_file(self.repo_id, f, revision=rev, local_dir=root), missing))

    def get_episodes_file_paths(self) -> list[str]:
        """Data files, then video files, of the selected episodes (relative to the root; v3.0 paths repeat)."""
        episodes = self.episodes if getattr(self, "episodes", None) is not None else sorted(self.meta.episodes)
        out = [str(self.meta.get_data_file_path(e)) for e in episodes]
        for e in episodes:
            out += [str(self.meta.get_video_file_path(e, k)) for k in self.meta.video_keys]
        return out

    def download_episodes(self, download_videos: bool = True, episodes_were_specified: bool | None = None) -> None:
        """The whole dataset as one snapshot, or exactly the selected episodes' files."""
        subset = episodes_were_specified if episodes_were_specified is not None else bool(
            getattr(self, "_episodes_were_specified", False))
        if not subset:
            self.pull_from_repo(ignore_patterns=None if download_videos else "videos/")
            return
        files = self.get_episodes_file_paths()
        self.download_files(files if download_videos else [f for f in files if not f.startswith("videos/")])

    def push_to_hub(self, branch: str | None = None, tags: list | None = None, license: str | None = "apache-2.0",
                    tag_version: bool = True, push_videos: bool = True, private: bool = False, allow_patterns=None,
                    upload_large_folder: bool = False, **card_kwargs) -> None:
        """Uploads the root (without the frame images kept for encoding; ``push_videos=False`` leaves the videos out
        too), writes a dataset card if the repository has none, and moves the codebase-version tag to the upload."""
        from .utils import CODEBASE_VERSION
        client = hub_client()
        ignore = ["images/"] + ([] if push_videos else ["videos/"])
        client.create_repo(self.repo_id, private=private)
        if branch:
            client.create_branch(self.repo_id, branch, revision=getattr(self, "revision", None))
        client.upload_folder(self.repo_id, Path(self.root), revision=branch, allow_patterns=allow_patterns,
                             ignore_patterns=ignore, large=upload_large_folder)
        if not client.file_exists(self.repo_id, REPOCARD_NAME, revision=branch):
            client.upload_text(self.repo_id, REPOCARD_NAME, dataset_card(getattr(self, "meta", self).info, tags, license, **card_kwargs),
                               revision=branch)
        if tag_version:
            client.retag(self.repo_id, CODEBASE_VERSION, revision=branch)
