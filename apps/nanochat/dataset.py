"""FineWeb-Edu shard fetcher for the nanochat app: fills a data directory with `shard_NNNNN.parquet` files that
`data.list_shards` / `data.token_stream` then read.

    python apps/nanochat/dataset.py --data-dir apps/nanochat/base_data -n 8 [--workers 4]

Shards are fetched on demand, several at a time, each into a `.part` file that is renamed only when complete, with a
capped exponential back-off between attempts; shards that already exist are skipped, so the command can be re-run
after an interruption.  Without network access every attempt fails after its retries and the command reports which
shards are missing (the training script also runs on synthetic tokens or on local text / parquet files).
Same data source and file naming as the reference's `apps/nanochat/dataset.py:22-25`; the download loop is this
file's own (urllib + thread pool instead of requests + process pool).
"""
import argparse
import concurrent.futures as cf
import os
import shutil
import sys
import time
import urllib.error
import urllib.request

SOURCE = "https://huggingface.co/datasets/karpathy/fineweb-edu-100b-shuffle/resolve/main"
LAST_SHARD = 1822


def shard_name(index):
    return f"shard_{index:05d}.parquet"


def fetch_shard(index, data_dir, attempts=5, timeout=30.0, source=SOURCE, opener=None, sleep=time.sleep):
    """Fetches one shard into `data_dir`.  Returns its path, or None when every attempt failed."""
    if not 0 <= index <= LAST_SHARD:
        raise ValueError(f"shard index {index} outside 0..{LAST_SHARD}")
    os.makedirs(data_dir, exist_ok=True)
    path = os.path.join(data_dir, shard_name(index))
    if os.path.exists(path):
        return path
    part = path + ".part"
    url = f"{source}/{shard_name(index)}"
    opener = opener or (lambda u: urllib.request.urlopen(u, timeout=timeout))
    for attempt in range(attempts):
        try:
            with opener(url) as resp, open(part, "wb") as out:
                shutil.copyfileobj(resp, out, length=1 << 20)
            os.replace(part, path)
            return path
        except (urllib.error.URLError, OSError, TimeoutError) as e:
            print(f"{shard_name(index)}: attempt {attempt + 1}/{attempts} failed: {e}", file=sys.stderr)
            if os.path.exists(part):
                os.remove(part)
            if attempt + 1 < attempts:
                sleep(min(2.0 ** (attempt + 1), 30.0))
    return None


def fetch(num_shards, data_dir, workers=4, include_validation=True, **kw):
    """The first `num_shards` training shards, plus the last shard of the set (the validation split of
    `data.list_shards`).  Returns (paths fetched or already present, indices that failed)."""
    wanted = list(range(min(num_shards, LAST_SHARD)))
    if include_validation and LAST_SHARD not in wanted:
        wanted.append(LAST_SHARD)
    done, failed = [], []
    with cf.ThreadPoolExecutor(max_workers=max(1, workers)) as ex:
        for idx, path in zip(wanted, ex.map(lambda i: fetch_shard(i, data_dir, **kw), wanted)):
            (done if path else failed).append(path or idx)
    return done, failed


# ---- the reference's module-level names (`apps/nanochat/dataset.py:34-95`) over the functions above ----------------
DATA_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "base_data")


def list_parquet_files(data_dir=None):
    """Sorted paths of the parquet shards under `data_dir` (default: `DATA_DIR`); unfinished `.part` files excluded."""
    data_dir = DATA_DIR if data_dir is None else data_dir
    if not os.path.isdir(data_dir):
        return []
    return [os.path.join(data_dir, f) for f in sorted(os.listdir(data_dir)) if f.endswith(".parquet")]


def parquets_iter_batched(split, start=0, step=1):
    """Lists of documents, one per parquet row group, from the shards of `split` ("train": all but the last shard,
    "val": the last one); `start` / `step` stride over row groups (rank / world size)."""
    assert split in ("train", "val"), "split must be 'train' or 'val'"
    import pyarrow.parquet as pq
    files = list_parquet_files()
    files = files[:-1] if split == "train" else files[-1:]
    for path in files:
        pf = pq.ParquetFile(path)
        for g in range(start, pf.num_row_groups, step):
            yield pf.read_row_group(g, columns=["text"]).column("text").to_pylist()


def download_single_file(index):
    """Fetches shard `index` into `DATA_DIR`; True when the file is there afterwards."""
    return fetch_shard(index, DATA_DIR) is not None


def main():
    ap = argparse.ArgumentParser(description="Fetch FineWeb-Edu shards for nanochat pretraining")
    ap.add_argument("--data-dir", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "base_data"))
    ap.add_argument("-n", "--num-shards", type=int, default=8)
    ap.add_argument("--workers", type=int, default=4)
    a = ap.parse_args()
    done, failed = fetch(a.num_shards, a.data_dir, a.workers)
    print(f"{len(done)} shards in {a.data_dir}" + (f"; missing: {failed}" if failed else ""))
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
