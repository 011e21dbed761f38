"""Token batches for the trainer: tokenizers, text sources and the (inputs, targets) batch stream.

Sources, picked by what `--data` points at:
  * a directory of `*.parquet` shards with a `text` column (FineWeb-Edu layout), `*.txt` files or `*.npy` token arrays;
    files are dealt to the ranks round-robin (file i belongs to rank i mod world), the last shard is the validation split;
  * `synthetic`: uniform random token ids, a different stream per rank (used by the benchmarks: no files needed).
Tokenizers: a HuggingFace `tokenizers` JSON file, a sentencepiece model, or the built-in byte tokenizer.
Reference counterpart: apps/nanochat/dataloader.py:119-180, tokenizer.py.
"""
import glob
import os

import numpy as np


class ByteTokenizer:
    """UTF-8 bytes plus <|bos|>; always available, no training needed."""
    vocab_size = 257
    bos_id = 256

    def encode_batch(self, texts):
        return [[self.bos_id] + list(t.encode("utf-8")) for t in texts]

    def decode(self, ids):
        return bytes(i for i in ids if i < 256).decode("utf-8", errors="replace")


class _HFTokenizer:
    def __init__(self, path):
        from tokenizers import Tokenizer
        self.tk = Tokenizer.from_file(path)
        self.vocab_size = self.tk.get_vocab_size()
        bos = self.tk.token_to_id("<|bos|>")
        self.bos_id = bos if bos is not None else 0

    def encode_batch(self, texts):
        return [[self.bos_id] + e.ids for e in self.tk.encode_batch(texts)]

    def decode(self, ids):
        return self.tk.decode(list(ids))


class _SPTokenizer:
    def __init__(self, path):
        import sentencepiece as spm
        self.sp = spm.SentencePieceProcessor(model_file=path)
        self.vocab_size = self.sp.get_piece_size()
        self.bos_id = max(self.sp.bos_id(), 0)

    def encode_batch(self, texts):
        return [[self.bos_id] + ids for ids in self.sp.encode(list(texts))]

    def decode(self, ids):
        return self.sp.decode(list(ids))


def load_tokenizer(path=None):
    if path is None or path == "bytes":
        return ByteTokenizer()
    if path.endswith(".json"):
        return _HFTokenizer(path)
    if path.endswith(".model"):
        return _SPTokenizer(path)
    raise ValueError(f"unknown tokenizer file: {path}")


def _texts(path, batch):
    if path.endswith(".parquet"):
        import pyarrow.parquet as pq
        pf = pq.ParquetFile(path)
        for g in range(pf.num_row_groups):
            col = pf.read_row_group(g, columns=["text"]).column("text").to_pylist()
            for i in range(0, len(col), batch):
                yield col[i:i + batch]
    else:
        with open(path, encoding="utf-8", errors="replace") as f:
            buf = []
            for line in f:
                if line.strip():
                    buf.append(line)
                if len(buf) == batch:
                    yield buf
                    buf = []
            if buf:
                yield buf


def list_shards(data_dir, split):
    files = sorted(glob.glob(os.path.join(data_dir, "*.parquet")) + glob.glob(os.path.join(data_dir, "*.txt"))
                   + glob.glob(os.path.join(data_dir, "*.npy")))
    if not files:
        raise FileNotFoundError(f"no *.parquet / *.txt / *.npy shards under {data_dir}")
    if len(files) == 1:
        return files
    return files[:-1] if split == "train" else files[-1:]


def token_stream(files, tokenizer, rank=0, world=1, tokenizer_batch=128, loop=True):
    """Endless (with `loop`) stream of token id lists from this rank's share of the files."""
    mine = [f for i, f in enumerate(files) if i % world == rank] or files
    while True:
        for path in mine:
            if path.endswith(".npy"):
                arr = np.load(path, mmap_mode="r")
                for i in range(0, len(arr), 1 << 20):
                    yield np.asarray(arr[i:i + (1 << 20)], dtype=np.int64).tolist()
            else:
                for texts in _texts(path, tokenizer_batch):
                    for ids in tokenizer.encode_batch(texts):
                        yield ids
        if not loop:
            return


def batches(stream, B, T):
    """(inputs, targets) int64 arrays of shape [B, T]; targets are the inputs shifted by one token."""
    need = B * T + 1
    buf = []
    for ids in stream:
        buf.extend(ids)
        while len(buf) >= need:
            chunk = np.asarray(buf[:need], dtype=np.int64)
            buf = buf[B * T:]
            yield chunk[:-1].reshape(B, T), chunk[1:].reshape(B, T)


def synthetic_batches(vocab_size, B, T, seed=0):
    rs = np.random.RandomState(seed)
    while True:
        chunk = rs.randint(0, vocab_size, size=B * T + 1).astype(np.int64)
        yield chunk[:-1].reshape(B, T), chunk[1:].reshape(B, T)


class Prefetcher:
    """Keeps the next batch on the device: pinned host buffers, copies on a side stream."""

    def __init__(self, it, device):
        import torch
        self.torch, self.it, self.device = torch, it, device
        self.cuda = str(device).startswith("cuda") and torch.cuda.is_available()
        self.stream = torch.cuda.Stream() if self.cuda else None
        self.bytes_per_batch = 0
        self._next = None
        self._load()

    def _load(self):
        torch = self.torch
        try:
            x, y = next(self.it)
        except StopIteration:
            self._next = None
            return
        xt, yt = torch.from_numpy(np.ascontiguousarray(x)), torch.from_numpy(np.ascontiguousarray(y))
        self.bytes_per_batch = xt.numel() * 8 * 2
        if self.cuda:
            xt, yt = xt.pin_memory(), yt.pin_memory()
            with torch.cuda.stream(self.stream):
                self._next = (xt.to(self.device, non_blocking=True), yt.to(self.device, non_blocking=True))
        else:
            self._next = (xt, yt)

    def __iter__(self):
        return self

    def __next__(self):
        if self._next is None:
            raise StopIteration
        if self.cuda:
            self.torch.cuda.current_stream().wait_stream(self.stream)
        out = self._next
        if self.cuda:
            for t in out:
                t.record_stream(self.torch.cuda.current_stream())
        self._load()
        return out
