"""The streaming loader of the nanochat app under the names of the reference's `apps/nanochat/dataloader.py`:
`get_dist_info`, `discover_parquet_files`, `parquets_iter_batched`, `tokenizing_distributed_data_loader`.  Built on
`data.py` of this directory (the training script itself uses `data.token_stream` / `data.Prefetcher`, which add `.txt` and
pre-tokenised `.npy` shards and device prefetch)."""
import os
import sys
from pathlib import Path
from typing import Iterator, List, Tuple

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import data as D  # noqa: E402


def get_dist_info() -> Tuple[bool, int, int, int]:
    """(ddp_enabled, rank, local_rank, world_size) from `genesis.distributed` (single process: False, 0, 0, 1)."""
    try:
        import genesis_b200.distributed as dist
        if dist.is_initialized():
            rank = dist.get_rank()
            return True, rank, int(os.environ.get("LOCAL_RANK", rank)), dist.get_world_size()
    except Exception:
        pass
    return False, 0, 0, 1


def discover_parquet_files(data_dir: Path, split: str = "train") -> List[Path]:
    """All but the last parquet shard for `train`, the last one for `val` (a single shard serves both)."""
    files = sorted(Path(data_dir).glob("*.parquet"))
    if not files:
        raise FileNotFoundError(f"no parquet files under {data_dir}")
    if len(files) == 1:
        return files
    return files[:-1] if split == "train" else files[-1:]


def parquets_iter_batched(data_dir: Path, split: str = "train", start: int = 0, step: int = 1,
                          batch: int = 1024) -> Iterator[List[str]]:
    """Lists of documents from this rank's shards (`start` = rank, `step` = world size), endlessly."""
    files = discover_parquet_files(data_dir, split)
    mine = files[start::step] or files
    while True:
        for p in mine:
            yield from D._texts(str(p), batch)


def tokenizing_distributed_data_loader(B: int, T: int, tokenizer_path: Path, data_dir: Path, split: str = "train",
                                       tokenizer_batch_size: int = 128,
                                       device: str = "cuda") -> Iterator[Tuple[np.ndarray, np.ndarray]]:
    """(inputs, targets) int64 arrays of shape [B, T], every document preceded by the BOS token; ranks read disjoint
    shards.  `device` is accepted for signature parity: the arrays stay on the host (the caller moves them)."""
    assert split in ("train", "val"), "split must be 'train' or 'val'"
    from tokenizer import NanoChatBPETokenizer
    _, rank, _, world = get_dist_info()
    tk = NanoChatBPETokenizer.load(tokenizer_path)
    bos = tk._bos_id if tk._bos_id is not None else 0

    def stream():
        for texts in parquets_iter_batched(data_dir, split, rank, world, tokenizer_batch_size):
            for ids in tk.encode_batch(texts, add_special_tokens=False):
                yield [bos] + ids
    yield from D.batches(stream(), B, T)
