"""Samplers: episode-aware frame sampling and the hierarchical (dataset -> sample) mixture sampler.

Every rank iterates the SAME seeded stream and keeps its own slice, so sharding needs no communication
(reference ``src/opentau/datasets/dataset_mixture.py:789-891,1164-1178``, ``datasets/sampler.py``).
"""

from __future__ import annotations

from typing import Iterator, Sequence

import torch


class EpisodeAwareSampler:
    """Iterates frame indices of selected episodes, optionally dropping frames at episode ends."""

    def __init__(self, episode_data_index: dict[str, torch.Tensor], episode_indices_to_use: Sequence[int] | None = None,
                 drop_n_first_frames: int = 0, drop_n_last_frames: int = 0, shuffle: bool = False,
                 generator: torch.Generator | None = None):
        idx: list[int] = []
        starts, ends = episode_data_index["from"], episode_data_index["to"]
        for ep, (s, e) in enumerate(zip(starts.tolist(), ends.tolist())):
            if episode_indices_to_use is None or ep in episode_indices_to_use:
                idx.extend(range(s + drop_n_first_frames, e - drop_n_last_frames))
        self.indices, self.shuffle, self.generator = idx, shuffle, generator

    def __iter__(self) -> Iterator[int]:
        if self.shuffle:
            for i in torch.randperm(len(self.indices), generator=self.generator).tolist():
                yield self.indices[i]
        else:
            yield from self.indices

    def __len__(self) -> int:
        return len(self.indices)


class HierarchicalSampler:
    """Infinite stream of global indices into a concatenation of datasets: first a dataset is drawn with
    probability proportional to its weight, then a uniform sample inside it.  ``rank``/``world`` select
    this rank's share of the common stream (positions ``rank, rank + world, ...``)."""

    def __init__(self, dataset_lengths: Sequence[int], weights: Sequence[float], seed: int, rank: int = 0,
                 world: int = 1, chunk: int = 4096):
        if len(dataset_lengths) != len(weights):
            raise ValueError("one weight per dataset")
        if any(n <= 0 for n in dataset_lengths):
            raise ValueError("every dataset must be non-empty")
        w = torch.tensor(list(weights), dtype=torch.float64)
        if w.sum() <= 0:
            raise ValueError("mixture weights must not all be zero")
        self.probs = w / w.sum()
        self.lengths = torch.tensor(list(dataset_lengths), dtype=torch.int64)
        self.offsets = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(self.lengths, 0)[:-1]])
        self.seed, self.rank, self.world, self.chunk = seed, rank, world, chunk

    def __iter__(self) -> Iterator[int]:
        g = torch.Generator()
        g.manual_seed(self.seed)
        pos = 0
        while True:
            ds = torch.multinomial(self.probs, self.chunk, replacement=True, generator=g)
            u = torch.rand(self.chunk, generator=g, dtype=torch.float64)
            local = (u * self.lengths[ds].double()).long().clamp_max_(self.lengths.max() - 1)
            local = torch.minimum(local, self.lengths[ds] - 1)
            glob = (self.offsets[ds] + local).tolist()
            for gi in glob:
                if pos % self.world == self.rank:
                    yield gi
                pos += 1
