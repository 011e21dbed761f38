"""Per-step JSONL metrics sink (loss, tokens/s, step ms, loss scale, overflow flag)."""
import json
import os
import time


class JsonlLogger:
    def __init__(self, path=None, rank=0):
        self.path = path
        self.rank = rank
        self._f = None
        if path is not None and rank == 0:
            os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
            self._f = open(path, "a", buffering=1)

    def log(self, **fields):
        fields.setdefault("time", time.time())
        if self._f is not None:
            self._f.write(json.dumps(fields) + "\n")
        return fields

    def close(self):
        if self._f is not None:
            self._f.close()
            self._f = None
