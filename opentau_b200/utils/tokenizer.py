"""Text and action tokenizers that work without network access.

The reference loads the PaliGemma sentencepiece tokenizer and the FAST action processor from the
hub (OpenTau ``policies/pi05/modeling_pi05.py:300-347``).  Here both are looked up locally first
(``transformers`` cache); when they are not on disk, deterministic stand-ins with the same
interface keep training, tests and benchmarks runnable:

* :class:`HashTokenizer` — whitespace/punctuation pieces hashed into a fixed vocabulary;
* :class:`DctActionTokenizer` — FAST-style discrete cosine transform + uniform quantisation of an
  action chunk, one id per retained coefficient (no BPE merge table).
"""

from __future__ import annotations

import hashlib
import logging
import math
import re
from functools import lru_cache

import numpy as np
import torch
from torch import Tensor

_PIECE = re.compile(r"\w+|[^\w\s]|\s+")


class HashTokenizer:
    """Deterministic offline tokenizer: ids 0=pad, 1=eos, 2=bos, pieces hashed into [3, vocab)."""

    pad_token_id, eos_token_id, bos_token_id = 0, 1, 2
    pad_token, eos_token, bos_token = "<pad>", "<eos>", "<bos>"

    PALIGEMMA_VOCAB, PALIGEMMA_LOC_BASE = 257152, 256000     # <loc0000>.. live at 256000..257023 in that vocabulary

    def __init__(self, vocab_size: int = 257152):
        self.vocab_size = vocab_size
        # pieces hash below the range a PaliGemma-sized vocabulary reserves for location / segmentation tokens
        self._hash_range = (self.PALIGEMMA_LOC_BASE if vocab_size == self.PALIGEMMA_VOCAB else vocab_size) - 3
        # the literal special strings map to their ids, as in the Gemma / PaliGemma tokenizers: prompts spell
        # separators out ("Task: ...<eos>State: ...")
        self.added_tokens: dict[str, int] = {self.pad_token: self.pad_token_id, self.eos_token: self.eos_token_id,
                                             self.bos_token: self.bos_token_id}
        self._added_re: re.Pattern | None = None
        self._compile_added()

    def __len__(self) -> int:
        return self.vocab_size

    def add_tokens(self, tokens, special_tokens: bool = True) -> int:
        """Registers strings that must map to ONE id each.  ``<locNNNN>`` in a PaliGemma-sized vocabulary takes its
        reserved id; anything else is appended.  Returns the number of ids appended (0 when nothing grew)."""
        grown = 0
        for t in tokens:
            t = str(getattr(t, "content", t))
            if t in self.added_tokens:
                continue
            m = re.fullmatch(r"<loc(\d{4})>", t)
            if m and self.vocab_size >= self.PALIGEMMA_VOCAB and int(m.group(1)) < 1024 \
                    and self._hash_range == self.PALIGEMMA_LOC_BASE - 3:
                self.added_tokens[t] = self.PALIGEMMA_LOC_BASE + int(m.group(1))
            else:
                self.added_tokens[t] = self.vocab_size
                self.vocab_size += 1
                grown += 1
        self._compile_added()
        return grown

    def _compile_added(self) -> None:
        self._added_re = re.compile("(" + "|".join(re.escape(t) for t in sorted(self.added_tokens, key=len,
                                                                                reverse=True)) + ")")

    def convert_tokens_to_ids(self, tokens):
        one = isinstance(tokens, str)
        ids = [self.added_tokens[t] if t in self.added_tokens else self._piece_id(t) for t in ([tokens] if one else tokens)]
        return ids[0] if one else ids

    @lru_cache(maxsize=65536)
    def _piece_id(self, piece: str) -> int:
        h = int.from_bytes(hashlib.blake2b(piece.encode("utf-8"), digest_size=8).digest(), "little")
        return 3 + h % self._hash_range

    def encode(self, text: str, add_special_tokens: bool = True) -> list[int]:
        chunks = self._added_re.split(text) if self._added_re is not None else [text]
        ids: list[int] = []
        for c in chunks:
            if c in self.added_tokens:
                ids.append(self.added_tokens[c])
            elif c:
                ids += [self._piece_id(p) for p in _PIECE.findall(c)]
        return ([self.bos_token_id] + ids) if add_special_tokens else ids

    def __call__(self, texts, max_length: int | None = None, padding: str | bool = "max_length",
                 truncation: bool = True, padding_side: str = "right", return_tensors: str = "pt",
                 add_special_tokens: bool = True):
        if isinstance(texts, str):
            texts = [texts]
        rows = [self.encode(t, add_special_tokens) for t in texts]
        L = max_length or max(len(r) for r in rows)
        ids = torch.full((len(rows), L), self.pad_token_id, dtype=torch.long)
        mask = torch.zeros((len(rows), L), dtype=torch.long)
        for i, r in enumerate(rows):
            r = r[:L] if truncation else r
            if padding_side == "right":
                ids[i, :len(r)] = torch.tensor(r, dtype=torch.long)
                mask[i, :len(r)] = 1
            else:
                ids[i, L - len(r):] = torch.tensor(r, dtype=torch.long)
                mask[i, L - len(r):] = 1
        return {"input_ids": ids, "attention_mask": mask}

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        return " ".join(f"<{int(i)}>" for i in ids if not (skip_special_tokens and int(i) < 3))


def load_text_tokenizer(name_or_path: str, vocab_size: int = 257152):
    """Local HF tokenizer when available, else :class:`HashTokenizer`."""
    try:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(name_or_path, local_files_only=True)
        if len(tok) > vocab_size:
            raise ValueError("tokenizer vocabulary exceeds the model's embedding table")
        return tok
    except Exception as e:  # noqa: BLE001 - any failure means "not on disk"
        logging.getLogger(__name__).info(
            "tokenizer %r not available locally (%s); using the offline hash tokenizer", name_or_path,
            type(e).__name__)
        return HashTokenizer(vocab_size)


class DctActionTokenizer:
    """FAST-style action tokenizer: per-dimension DCT-II over time, quantise, flatten low
    frequencies first.  Id 0 is the pad id; coefficient value ``q`` maps to ``1 + clip(q + R)``."""

    def __init__(self, vocab_size: int = 2048, scale: float = 10.0):
        self.vocab_size = vocab_size
        self.scale = scale
        self.radius = (vocab_size - 2) // 2

    @staticmethod
    @lru_cache(maxsize=16)
    def _dct_matrix(n: int) -> np.ndarray:
        k = np.arange(n)[:, None]
        t = np.arange(n)[None, :]
        m = np.cos(math.pi * (t + 0.5) * k / n) * math.sqrt(2.0 / n)
        m[0] /= math.sqrt(2.0)
        return m

    def __call__(self, actions) -> list[list[int]]:
        a = np.asarray(actions.detach().float().cpu() if isinstance(actions, Tensor) else actions, dtype=np.float64)
        if a.ndim == 2:
            a = a[None]
        B, T, D = a.shape
        coef = np.einsum("kt,btd->bkd", self._dct_matrix(T), a)
        q = np.clip(np.rint(coef * self.scale), -self.radius, self.radius).astype(np.int64)
        out = []
        for b in range(B):
            flat = q[b].reshape(-1)               # frequency-major: low frequencies first
            nz = np.nonzero(flat)[0]
            end = int(nz[-1]) + 1 if len(nz) else 0
            out.append((flat[:end] + self.radius + 1).tolist())
        return out

    def decode(self, tokens: list[list[int]], time_horizon: int, action_dim: int) -> np.ndarray:
        out = np.zeros((len(tokens), time_horizon, action_dim))
        m = self._dct_matrix(time_horizon)
        for b, ids in enumerate(tokens):
            flat = np.zeros(time_horizon * action_dim)
            ids = [i for i in ids if i > 0][: flat.size]
            flat[:len(ids)] = np.asarray(ids, dtype=np.float64) - self.radius - 1
            out[b] = m.T @ (flat.reshape(time_horizon, action_dim) / self.scale)
        return out


FITTED_TOKENIZER_FILE = "action_tokenizer.json"


def load_action_tokenizer(name_or_path: str, vocab_size: int = 2048):
    """A tokenizer fitted by ``scripts/fit_fast_tokenizer`` (a directory, or the file itself, holding
    ``action_tokenizer.json``), else a FAST processor from the local transformers cache, else the offline DCT
    tokenizer.  A fitted table larger than the policy's ``discrete_action_vocab_size`` cannot be embedded and is an
    error; a smaller one simply leaves ids unused."""
    from pathlib import Path
    p = Path(str(name_or_path))
    fitted = p / FITTED_TOKENIZER_FILE if p.is_dir() else (p if p.is_file() and p.suffix == ".json" else None)
    if fitted is not None and fitted.is_file():
        tok = BpeDctActionTokenizer.load(fitted)
        if tok.vocab_size > vocab_size:
            raise ValueError(f"the tokenizer at {fitted} has {tok.vocab_size} ids, the policy embeds {vocab_size} "
                             "(discrete_action_vocab_size): refit with a smaller --vocab-size or widen the policy")
        return tok
    try:
        from transformers import AutoProcessor
        return AutoProcessor.from_pretrained(name_or_path, trust_remote_code=True, local_files_only=True)
    except Exception as e:  # noqa: BLE001
        logging.getLogger(__name__).info(
            "action tokenizer %r not available locally (%s); using the offline DCT tokenizer",
            name_or_path, type(e).__name__)
        return DctActionTokenizer(vocab_size)


def pad_tokens(rows: list[list[int]], max_length: int, pad_id: int = 0) -> tuple[Tensor, Tensor]:
    """Right-pads/truncates id lists to ``max_length``; returns ``(ids long, mask bool)``."""
    ids = torch.full((len(rows), max_length), pad_id, dtype=torch.long)
    mask = torch.zeros((len(rows), max_length), dtype=torch.bool)
    for i, r in enumerate(rows):
        r = list(r)[:max_length]
        if r:
            ids[i, :len(r)] = torch.tensor(r, dtype=torch.long)
            mask[i, :len(r)] = True
    return ids, mask


_BPE_LIB: list = []          # [handle or None], filled on first use


def _bpe_lib():
    """The native byte-pair library (``runtime/csrc/bpe.cpp``), or ``None`` when it has not been built."""
    if not _BPE_LIB:
        import ctypes
        from ..ops.build import lib_path
        handle = None
        f = lib_path("bpe")
        if f.exists():
            try:
                handle = ctypes.CDLL(str(f))
                i32p, i64p = ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int64)
                handle.otb_bpe_train.argtypes = [i32p, i64p, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32,
                                                 ctypes.c_int32, i32p]
                handle.otb_bpe_train.restype = ctypes.c_int32
                handle.otb_bpe_encode.argtypes = [i32p, i64p, ctypes.c_int64, i32p, ctypes.c_int32, ctypes.c_int32,
                                                  i32p, i64p, ctypes.c_int32]
                handle.otb_bpe_encode.restype = ctypes.c_int32
            except OSError:
                handle = None
        _BPE_LIB.append(handle)
    return _BPE_LIB[0]


def _flatten(seqs: list[list[int]]):
    import ctypes
    lens = np.fromiter((len(s) for s in seqs), np.int64, len(seqs))
    offsets = np.zeros(len(seqs) + 1, np.int64)
    np.cumsum(lens, out=offsets[1:])
    flat = np.fromiter((x for s in seqs for x in s), np.int32, int(offsets[-1])) if offsets[-1] else np.zeros(1, np.int32)
    ptr = lambda a, t: a.ctypes.data_as(ctypes.POINTER(t))  # noqa: E731
    return flat, offsets, ptr


def _native_train(lib, seqs: list[list[int]], base: int, vocab_size: int, min_count: int) -> list[tuple[int, int]]:
    import ctypes
    room = max(vocab_size - base, 0)
    if room == 0 or not seqs:
        return []
    flat, offsets, ptr = _flatten(seqs)
    out = np.zeros(2 * room, np.int32)
    n = lib.otb_bpe_train(ptr(flat, ctypes.c_int32), ptr(offsets, ctypes.c_int64), len(seqs), base, vocab_size,
                          min_count, ptr(out, ctypes.c_int32))
    if n < 0:
        raise RuntimeError(f"otb_bpe_train refused its arguments ({n})")
    return [(int(out[2 * i]), int(out[2 * i + 1])) for i in range(n)]


def _native_encode(lib, seqs: list[list[int]], merges: list[tuple[int, int]], base: int) -> list[list[int]]:
    import ctypes
    import os
    if not seqs:
        return []
    flat, offsets, ptr = _flatten(seqs)
    table = np.asarray(merges, np.int32).reshape(-1) if merges else np.zeros(2, np.int32)
    out, out_len = np.zeros_like(flat), np.zeros(len(seqs), np.int64)
    threads = min(len(seqs), max(1, (os.cpu_count() or 1) // 2), 16)
    rc = lib.otb_bpe_encode(ptr(flat, ctypes.c_int32), ptr(offsets, ctypes.c_int64), len(seqs),
                            ptr(table, ctypes.c_int32), len(merges), base, ptr(out, ctypes.c_int32),
                            ptr(out_len, ctypes.c_int64), threads)
    if rc != 0:
        raise RuntimeError(f"otb_bpe_encode refused its arguments ({rc})")
    return [out[offsets[i]:offsets[i] + out_len[i]].tolist() for i in range(len(seqs))]


class BpeDctActionTokenizer:
    """FAST-style tokenizer with a learned merge table: DCT-II per action dimension, quantisation, low frequencies
    first, then byte-pair merges fitted on a corpus of action chunks (what
    ``src/opentau/scripts/fit_fast_tokenizer.py`` produces in the reference; there through the FAST processor).

    Base symbols are the quantised coefficients in ``[-radius, radius]`` (ids ``1 .. 2*radius+1``; 0 pads); every
    merge adds one id.  ``save`` / ``load`` use one JSON file.
    """

    def __init__(self, scale: float = 10.0, radius: int = 127, merges: list[tuple[int, int]] | None = None,
                 time_horizon: int | None = None, action_dim: int | None = None):
        self.scale, self.radius = scale, radius
        self.base = 2 * radius + 2
        self.merges = [tuple(m) for m in (merges or [])]
        self.time_horizon, self.action_dim = time_horizon, action_dim
        self._rank = {m: i for i, m in enumerate(self.merges)}

    @property
    def vocab_size(self) -> int:
        return self.base + len(self.merges)

    def _symbols(self, actions) -> list[list[int]]:
        a = np.asarray(actions.detach().float().cpu() if isinstance(actions, Tensor) else actions, dtype=np.float64)
        if a.ndim == 2:
            a = a[None]
        B, T, D = a.shape
        coef = np.einsum("kt,btd->bkd", DctActionTokenizer._dct_matrix(T), a)
        q = np.clip(np.rint(coef * self.scale), -self.radius, self.radius).astype(np.int64)
        out = []
        for b in range(B):
            flat = q[b].reshape(-1)
            nz = np.nonzero(flat)[0]
            end = int(nz[-1]) + 1 if len(nz) else 0
            out.append((flat[:end] + self.radius + 1).tolist())
        return out

    @staticmethod
    def _merge(seq: list[int], pair: tuple[int, int], new_id: int) -> list[int]:
        out, i = [], 0
        while i < len(seq):
            if i + 1 < len(seq) and seq[i] == pair[0] and seq[i + 1] == pair[1]:
                out.append(new_id)
                i += 2
            else:
                out.append(seq[i])
                i += 1
        return out

    def fit(self, chunks, vocab_size: int = 2048, min_count: int = 2, native: bool | None = None) -> "BpeDctActionTokenizer":
        """``chunks (N, T, D)`` normalised action chunks.  The most frequent adjacent pair becomes a new symbol, ties go
        to the smaller left then the smaller right symbol, occurrences merge left to right without overlap; until the
        vocabulary is full or the best pair occurs fewer than ``min_count`` times.  ``native``: the C++ trainer
        (``None`` = when its library is built); both give the same table."""
        arr = np.asarray(chunks)
        self.time_horizon, self.action_dim = int(arr.shape[1]), int(arr.shape[2])
        seqs = self._symbols(arr)
        lib = _bpe_lib() if native in (None, True) else None
        if native and lib is None:
            raise RuntimeError("the native byte-pair library is not built (python -m opentau_b200.ops.build)")
        if lib is not None:
            self.merges = _native_train(lib, seqs, self.base, vocab_size, min_count)
        else:
            self.merges = self._fit_python(seqs, vocab_size, min_count)
        self._rank = {m: i for i, m in enumerate(self.merges)}
        return self

    def _fit_python(self, seqs: list[list[int]], vocab_size: int, min_count: int) -> list[tuple[int, int]]:
        merges: list[tuple[int, int]] = []
        while self.base + len(merges) < vocab_size:
            counts: dict[tuple[int, int], int] = {}
            for s in seqs:
                for a, b in zip(s[:-1], s[1:]):
                    counts[(a, b)] = counts.get((a, b), 0) + 1
            if not counts:
                break
            pair, c = max(counts.items(), key=lambda kv: (kv[1], -kv[0][0], -kv[0][1]))
            if c < min_count:
                break
            new_id = self.base + len(merges)
            merges.append(pair)
            seqs = [self._merge(s, pair, new_id) for s in seqs]
        return merges

    def __call__(self, actions, native: bool | None = None) -> list[list[int]]:
        seqs = self._symbols(actions)
        lib = _bpe_lib() if native in (None, True) else None
        if lib is not None:
            return _native_encode(lib, seqs, self.merges, self.base)
        out = []
        for s in seqs:
            while len(s) > 1:
                best = min(((self._rank.get((a, b), 1 << 30), i) for i, (a, b) in enumerate(zip(s[:-1], s[1:]))))
                if best[0] == 1 << 30:
                    break
                pair = self.merges[best[0]]
                s = self._merge(s, pair, self.base + best[0])
            out.append(s)
        return out

    def _expand(self, tid: int) -> list[int]:
        if tid < self.base:
            return [tid]
        a, b = self.merges[tid - self.base]
        return self._expand(a) + self._expand(b)

    def decode(self, tokens: list[list[int]], time_horizon: int | None = None, action_dim: int | None = None) -> np.ndarray:
        T, D = time_horizon or self.time_horizon, action_dim or self.action_dim
        out = np.zeros((len(tokens), T, D))
        m = DctActionTokenizer._dct_matrix(T)
        for b, ids in enumerate(tokens):
            sym = [x for t in ids if t > 0 for x in self._expand(int(t))][: T * D]
            flat = np.zeros(T * D)
            flat[:len(sym)] = np.asarray(sym, dtype=np.float64) - self.radius - 1
            out[b] = m.T @ (flat.reshape(T, D) / self.scale)
        return out

    def save(self, path) -> None:
        import json
        from pathlib import Path
        Path(path).parent.mkdir(parents=True, exist_ok=True)
        Path(path).write_text(json.dumps({"type": "bpe_dct", "scale": self.scale, "radius": self.radius,
                                          "merges": self.merges, "time_horizon": self.time_horizon,
                                          "action_dim": self.action_dim}))

    @classmethod
    def load(cls, path) -> "BpeDctActionTokenizer":
        import json
        from pathlib import Path
        d = json.loads(Path(path).read_text())
        return cls(d["scale"], d["radius"], [tuple(m) for m in d["merges"]], d["time_horizon"], d["action_dim"])
