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

    PALIGEMMA_VOCAB, PALIGEMMA_LOC_BASE = 257152, 256000     # <loc0000>.. live at 256000..257023 in that vocabulary

    def __init__(self, vocab_size: int = 257152):
        self.vocab_size = vocab_size
        # pieces hash below the range a PaliGemma-sized vocabulary reserves for location / segmentation tokens
        self._hash_range = (self.PALIGEMMA_LOC_BASE if vocab_size == self.PALIGEMMA_VOCAB else vocab_size) - 3
        self.added_tokens: dict[str, int] = {}
        self._added_re: re.Pattern | None = None

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
        self._added_re = re.compile("(" + "|".join(re.escape(t) for t in sorted(self.added_tokens, key=len,
                                                                                reverse=True)) + ")")
        return grown

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


def load_action_tokenizer(name_or_path: str, vocab_size: int = 2048):
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

    def fit(self, chunks, vocab_size: int = 2048, min_count: int = 2) -> "BpeDctActionTokenizer":
        """``chunks (N, T, D)`` normalised action chunks."""
        arr = np.asarray(chunks)
        self.time_horizon, self.action_dim = int(arr.shape[1]), int(arr.shape[2])
        seqs = self._symbols(arr)
        self.merges = []
        while self.base + len(self.merges) < vocab_size:
            counts: dict[tuple[int, int], int] = {}
            for s in seqs:
                for a, b in zip(s[:-1], s[1:]):
                    counts[(a, b)] = counts.get((a, b), 0) + 1
            if not counts:
                break
            pair, c = max(counts.items(), key=lambda kv: (kv[1], -kv[0][0], -kv[0][1]))
            if c < min_count:
                break
            new_id = self.base + len(self.merges)
            self.merges.append(pair)
            seqs = [self._merge(s, pair, new_id) for s in seqs]
        self._rank = {m: i for i, m in enumerate(self.merges)}
        return self

    def __call__(self, actions) -> list[list[int]]:
        out = []
        for s in self._symbols(actions):
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
