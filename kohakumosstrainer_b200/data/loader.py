"""Stateless batch loader: batch i is f(seed, rank, i); resume state is `{seed, start}`.

Same contract as the reference loader (`src/kohakumoss_data/loader/stateless.py:60-146`): the
stream does not depend on the worker count, iteration can stop and restart anywhere, and
`state_dict()` / `load_state_dict()` carry only the seed and the next index.

Built for a host that feeds a B200: worker w of W materialises indices start + w, start + w +
W, ... in its own process (forkserver; decode and caption rendering hold the GIL) or thread
(`workers_mode="thread"`, enough when everything comes from the caches, where the work is
memory-mapped reads and `torch.cat`); finished batches are re-ordered, pinned by the consumer
thread and handed out strictly in index order, `prefetch` batches per worker ahead.
"""

from __future__ import annotations

import multiprocessing as mp
import queue
import threading

import torch


def _serve(dataset, rank, world, start, worker, workers, transform, out, stop):
    torch.set_num_threads(1)
    index = start + worker
    while not stop.is_set():
        try:
            batch = dataset.materialize(index, rank, world)
            if transform is not None:
                batch = transform(batch)
            item = (index, batch, None)
        except BaseException as exc:  # ship the failure to the consumer, which re-raises it
            item = (index, None, f"{type(exc).__name__}: {exc}")
        while not stop.is_set():
            try:
                out.put(item, timeout=0.2)
                break
            except queue.Full:
                continue
        if item[2] is not None:
            return
        index += workers


class Loader:
    def __init__(self, dataset, rank: int = 0, world: int = 1, num_workers: int = 0, prefetch: int = 2, pin_memory: bool = True,
                 start: int = 0, transform=None, workers_mode: str = "process"):
        self.dataset, self.rank, self.world = dataset, rank, world
        self.num_workers, self.prefetch = num_workers, max(1, prefetch)
        self.pin_memory = pin_memory and torch.cuda.is_available()
        self.start, self.served = start, 0
        self.transform = transform
        self.workers_mode = workers_mode
        self._procs, self._stop = [], None

    # -- resume -----------------------------------------------------------------------------------
    def state_dict(self) -> dict:
        return {"seed": self.dataset.cfg.seed, "start": self.start + self.served}

    def load_state_dict(self, state: dict) -> None:
        if state["seed"] != self.dataset.cfg.seed:
            raise ValueError(f"resume seed {state['seed']} != data seed {self.dataset.cfg.seed}")
        self.start, self.served = int(state["start"]), 0

    # -- iteration --------------------------------------------------------------------------------
    def _finish(self, batch):
        return batch.pin_memory() if self.pin_memory and hasattr(batch, "pin_memory") else batch

    def __iter__(self):
        self.start += self.served
        self.served = 0
        if self.num_workers <= 0:
            index = self.start
            while True:
                batch = self.dataset.materialize(index, self.rank, self.world)
                if self.transform is not None:
                    batch = self.transform(batch)
                self.served += 1
                index += 1
                yield self._finish(batch)
        try:
            yield from self._iterate_workers()
        finally:
            self.shutdown()

    def _iterate_workers(self):
        n = self.num_workers
        if self.workers_mode == "thread":
            stop = threading.Event()
            queues = [queue.Queue(self.prefetch) for _ in range(n)]
            make = lambda w: threading.Thread(target=_serve, daemon=True, args=(  # noqa: E731
                self.dataset, self.rank, self.world, self.start, w, n, self.transform, queues[w], stop))
        else:
            ctx = mp.get_context("forkserver")
            stop = ctx.Event()
            queues = [ctx.Queue(self.prefetch) for _ in range(n)]
            make = lambda w: ctx.Process(target=_serve, daemon=True, args=(  # noqa: E731
                self.dataset, self.rank, self.world, self.start, w, n, self.transform, queues[w], stop))
        self._stop = stop
        self._procs = [make(w) for w in range(n)]
        for p in self._procs:
            p.start()
        index = self.start
        while True:
            w = (index - self.start) % n     # one queue per worker keeps index order without a reorder buffer
            while True:
                try:
                    got, batch, err = queues[w].get(timeout=1.0)
                    break
                except queue.Empty:
                    if not self._procs[w].is_alive():
                        raise RuntimeError(f"loader worker {w} died before producing batch {index}")
            if err is not None:
                raise RuntimeError(f"loader worker {w} failed on batch {got}: {err}")
            assert got == index, (got, index)
            self.served += 1
            index += 1
            yield self._finish(batch)

    def shutdown(self) -> None:
        if self._stop is not None:
            self._stop.set()
        for p in self._procs:
            started = p.ident is not None if isinstance(p, threading.Thread) else getattr(p, "_popen", None) is not None
            if not started:
                continue
            p.join(timeout=2.0)
            if hasattr(p, "terminate") and p.is_alive():
                p.terminate()
        self._procs, self._stop = [], None


def build_loader(dataset, cfg=None, rank: int = 0, world: int = 1, start: int = 0, transform=None, workers_mode: str | None = None) -> Loader:
    cfg = cfg or dataset.cfg
    cached = getattr(cfg, "latent_cache", "off") == "offline" and getattr(cfg, "text_cache", "off") == "offline"
    mode = workers_mode or ("thread" if cached else "process")
    return Loader(dataset, rank, world, getattr(cfg, "num_workers", 0), getattr(cfg, "prefetch", 2), getattr(cfg, "pin_memory", True),
                  start, transform, mode)
