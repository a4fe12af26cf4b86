"""Asynchronous PNG writer used while recording (reference ``src/opentau/datasets/image_writer.py:40-304``):
a pool of worker threads drains a queue of ``(image, path)`` pairs so the control loop never blocks on disk IO."""

from __future__ import annotations

import queue
import threading
from pathlib import Path

import numpy as np
import torch


def image_array_to_pil_image(arr: np.ndarray):
    from PIL import Image
    if arr.ndim != 3:
        raise ValueError(f"expected a 3-D image array, got {arr.ndim} dims")
    if arr.shape[0] in (1, 3) and arr.shape[-1] not in (1, 3):
        arr = arr.transpose(1, 2, 0)
    if arr.dtype != np.uint8:
        if arr.min() < 0.0 or arr.max() > 1.0:
            raise ValueError("float images must be in [0, 1]")
        arr = (arr * 255).round().astype(np.uint8)
    if arr.shape[-1] == 1:
        arr = arr[..., 0]
    return Image.fromarray(arr)


def write_image(image, fpath: Path) -> None:
    try:
        if isinstance(image, torch.Tensor):
            image = image.detach().cpu().numpy()
        img = image_array_to_pil_image(image) if isinstance(image, np.ndarray) else image
        Path(fpath).parent.mkdir(parents=True, exist_ok=True)
        img.save(fpath)
    except Exception as e:  # noqa: BLE001 - a failed frame must not kill a recording session
        print(f"Error writing image {fpath}: {e}")


class AsyncImageWriter:
    def __init__(self, num_processes: int = 0, num_threads: int = 2):
        if num_threads < 1:
            raise ValueError("need at least one writer thread")
        self.queue: queue.Queue = queue.Queue()
        self.threads = [threading.Thread(target=self._worker, daemon=True) for _ in range(num_threads)]
        self._stopped = False
        for t in self.threads:
            t.start()

    def _worker(self) -> None:
        while True:
            item = self.queue.get()
            if item is None:
                self.queue.task_done()
                return
            write_image(*item)
            self.queue.task_done()

    def save_image(self, image, fpath: Path) -> None:
        if isinstance(image, torch.Tensor):
            image = image.detach().cpu().numpy()
        self.queue.put((image, fpath))

    def wait_until_done(self) -> None:
        self.queue.join()

    def stop(self) -> None:
        if self._stopped:
            return
        for _ in self.threads:
            self.queue.put(None)
        for t in self.threads:
            t.join()
        self._stopped = True
