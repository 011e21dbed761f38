"""Host-side failure detection: per-rank heartbeats through a key-value store.

Every rank bumps `hb/<rank>` every `interval` seconds from a daemon thread and reads its
peers' counters; a peer whose counter has not moved for `timeout` seconds is reported
dead.  `check()` raises `CommTimeout` naming the dead ranks, so a training loop can stop
launching collectives that would never complete (device-side waits are bounded as well and
report through a status word; see `genesis_b200.distributed.symm`).  Any object with
`set(key, str)` / `get(key)` works as the store (`torch.distributed.TCPStore`, `FileStore`,
`HashStore`).  The reference has no counterpart (its only guard is a 60-try rendezvous
retry, `genesis/distributed/nccl_backend.py:268-301`).
"""
import threading
import time

from .process_group import CommTimeout


class Heartbeat:
    def __init__(self, store, rank, world_size, interval=0.5, timeout=5.0, prefix="hb"):
        self.store, self.rank, self.world = store, rank, world_size
        self.interval, self.timeout, self.prefix = interval, timeout, prefix
        self._stop = threading.Event()
        self._thread = None
        self._count = 0
        self._last = {}        # peer -> (counter, time the counter last changed)
        self._dead = set()
        self._lock = threading.Lock()
        self._paused = False

    def _key(self, r):
        return f"{self.prefix}/{r}"

    def start(self):
        self.store.set(self._key(self.rank), "0")
        now = time.monotonic()
        for r in range(self.world):
            self._last[r] = (None, now)
        # beating and polling run on threads of their own: a store whose `get` blocks on a key that was never set
        # (torch's TCPStore waits for its whole timeout: the "rank never joined" case) must not stop this rank's beats
        self._thread = threading.Thread(target=self._run_beat, name="genesis-heartbeat", daemon=True)
        self._poll_thread = threading.Thread(target=self._run_poll, name="genesis-heartbeat-poll", daemon=True)
        self._thread.start()
        self._poll_thread.start()
        return self

    def pause(self):
        """Stop beating without stopping the monitor (used by tests to emulate a stalled rank)."""
        self._paused = True

    def resume(self):
        self._paused = False

    def _beat(self):
        self._count += 1
        self.store.set(self._key(self.rank), str(self._count))

    def _poll(self):
        now = time.monotonic()
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                check = getattr(self.store, "check", None)       # non-blocking presence test where the store has one
                if check is not None and not check([self._key(r)]):
                    val = None
                else:
                    val = self.store.get(self._key(r))
                    val = val.decode() if isinstance(val, bytes) else str(val)
            except Exception:
                val = None
            prev, t_prev = self._last[r]
            if val is not None and val != prev:
                self._last[r] = (val, now)
                with self._lock:
                    self._dead.discard(r)
            elif now - t_prev > self.timeout:
                with self._lock:
                    self._dead.add(r)

    def _run_beat(self):
        while not self._stop.is_set():
            try:
                if not self._paused:
                    self._beat()
            except Exception:
                pass
            self._stop.wait(self.interval)

    def _run_poll(self):
        while not self._stop.is_set():
            try:
                self._poll()
            except Exception:
                pass
            self._stop.wait(self.interval)

    def dead_ranks(self):
        with self._lock:
            return sorted(self._dead)

    def check(self):
        dead = self.dead_ranks()
        if dead:
            raise CommTimeout(f"rank {self.rank}: no heartbeat from ranks {dead} for more than {self.timeout}s")

    def stop(self):
        self._stop.set()
        for name in ("_thread", "_poll_thread"):
            th = getattr(self, name, None)
            if th is not None:
                th.join(timeout=2.0)
                setattr(self, name, None)
