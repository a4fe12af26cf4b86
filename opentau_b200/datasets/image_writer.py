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


def _thread_loop(q) -> None:
    while True:
        item = q.get()
        if item is None:
            q.task_done()
            return
        write_image(*item)
        q.task_done()


def _process_loop(q, num_threads: int) -> None:
    """A worker process: ``num_threads`` threads drain the shared queue; each thread leaves on its own ``None``."""
    threads = [threading.Thread(target=_thread_loop, args=(q,), daemon=True) for _ in range(num_threads)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()


def safe_stop_image_writer(func):
    """Decorator for recording loops: if the wrapped call raises, the dataset's image writer (first argument's
    ``image_writer``, or a ``dataset=`` keyword's) is stopped before the exception travels on, so no worker thread or
    process outlives a crashed session."""
    import functools

    @functools.wraps(func)
    def wrapper(*args, **kwargs):
        try:
            return func(*args, **kwargs)
        except BaseException:
            owner = kwargs.get("dataset", args[0] if args else None)
            writer = getattr(owner, "image_writer", None)
            if writer is not None:
                print("Waiting for the image writer to terminate...")
                writer.stop()
            raise
    return wrapper


class AsyncImageWriter:
    """``num_processes == 0``: ``num_threads`` threads in this process (enough for one or two cameras: most of a PNG
    save is zlib, which releases the interpreter lock).  ``num_processes > 0``: that many worker processes with
    ``num_threads`` threads each, fed through one joinable queue: for many cameras at high frame rates, where the
    Python part of the encoding would otherwise hold up the control loop.  ``wait_until_done`` returns when every queued
    frame is on disk; ``stop`` ends the workers (idempotent)."""

    def __init__(self, num_processes: int = 0, num_threads: int = 2):
        if num_threads < 1 and num_processes < 1:
            raise ValueError("need at least one writer thread or process")
        num_threads = max(1, num_threads)
        self.num_processes, self.num_threads = num_processes, num_threads
        self._stopped = False
        self.processes: list = []
        if num_processes == 0:
            self.queue = queue.Queue()
            self.threads = [threading.Thread(target=_thread_loop, args=(self.queue,), daemon=True)
                            for _ in range(num_threads)]
            for t in self.threads:
                t.start()
        else:
            import multiprocessing as mp
            ctx = mp.get_context("spawn")           # no forked copy of CUDA / thread state in the workers
            self.queue = ctx.JoinableQueue()
            self.threads = []
            for _ in range(num_processes):
                p = ctx.Process(target=_process_loop, args=(self.queue, num_threads), daemon=True)
                p.start()
                self.processes.append(p)

    def save_image(self, image, fpath: Path) -> None:
        if isinstance(image, torch.Tensor):
            image = image.detach().cpu().numpy()       # tensors do not cross the process boundary cheaply
        self.queue.put((image, fpath))

    def wait_until_done(self) -> None:
        self.queue.join()

    def stop(self) -> None:
        if self._stopped:
            return
        self._stopped = True
        for _ in range(max(1, self.num_processes) * self.num_threads):
            self.queue.put(None)
        for t in self.threads:
            t.join()
        for p in self.processes:
            p.join(timeout=10)
            if p.is_alive():
                p.terminate()
        if self.processes:
            self.queue.close()
