"""The nanochat trainer end to end on CPU: synthetic data, text shards with the byte tokenizer, resume."""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "apps", "nanochat"))


def _train(argv):
    import importlib
    train = importlib.import_module("train")
    return train.main(argv)


def test_trainer_synthetic_and_resume(tmp_path):
    out = str(tmp_path / "ck")
    metrics = str(tmp_path / "m.jsonl")
    common = ["--model", "tiny", "--data", "synthetic", "--vocab-size", "200", "--batch-size", "2", "--block-size", "16",
              "--device", "cpu", "--out", out, "--log-interval", "2", "--eval-interval", "4", "--eval-batches", "2",
              "--save-interval", "4", "--accumulation-steps", "2", "--clip-grad", "1.0", "--warmup-steps", "2"]
    assert _train(common + ["--max-steps", "4", "--metrics", metrics]) == 4
    rows = [json.loads(l) for l in open(metrics)]
    assert [r["step"] for r in rows] == [2, 4] and all(np.isfinite(r["loss"]) for r in rows)
    ck = os.path.join(out, "checkpoint_4.pth")
    assert os.path.exists(ck) and os.path.exists(os.path.join(out, "checkpoint_final.pth"))
    assert _train(common + ["--max-steps", "6", "--resume", ck]) == 6


def test_trainer_learns_text_shards(tmp_path):
    data = tmp_path / "shards"
    data.mkdir()
    for i in range(2):
        (data / f"shard_{i}.txt").write_text("the quick brown fox jumps over the lazy dog\n" * 200)
    metrics = str(tmp_path / "m.jsonl")
    _train(["--model", "tiny", "--data", str(data), "--tokenizer", "bytes", "--batch-size", "4", "--block-size", "32",
            "--device", "cpu", "--out", str(tmp_path / "ck"), "--max-steps", "30", "--log-interval", "10",
            "--eval-interval", "0", "--save-interval", "0", "--learning-rate", "3e-3", "--metrics", metrics,
            "--amp", "--dtype", "bf16"])
    rows = [json.loads(l) for l in open(metrics)]
    assert rows[-1]["loss"] < rows[0]["loss"] - 0.5, rows


def test_batches_shift_targets_by_one():
    import data as D
    stream = iter([[1, 2, 3, 4, 5], [6, 7, 8, 9, 10, 11, 12]])
    x, y = next(D.batches(stream, 2, 3))
    assert x.tolist() == [[1, 2, 3], [4, 5, 6]] and y.tolist() == [[2, 3, 4], [5, 6, 7]]
    tok = D.ByteTokenizer()
    ids = tok.encode_batch(["hé"])[0]
    assert ids[0] == tok.bos_id and tok.decode(ids) == "hé"


def test_cuda_graph_flag_is_refused_without_cuda(tmp_path):
    import pytest
    with pytest.raises(SystemExit):
        _train(["--model", "tiny", "--data", "synthetic", "--vocab-size", "200", "--batch-size", "2", "--block-size", "16",
                "--device", "cpu", "--out", str(tmp_path / "ck"), "--max-steps", "2", "--cuda-graph"])


def test_shard_fetcher_writes_atomically_retries_and_skips(tmp_path):
    import io
    import importlib.util
    import urllib.error
    spec = importlib.util.spec_from_file_location("nanochat_dataset", os.path.join(ROOT, "apps", "nanochat", "dataset.py"))
    ds = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ds)
    calls = {"n": 0}

    def flaky(url):
        calls["n"] += 1
        if calls["n"] == 1:
            raise urllib.error.URLError("temporary failure")
        return io.BytesIO(b"PAR1" + url.encode())

    p = ds.fetch_shard(3, str(tmp_path), opener=flaky, sleep=lambda s: None)
    assert p.endswith("shard_00003.parquet") and open(p, "rb").read().startswith(b"PAR1")
    assert calls["n"] == 2 and not os.path.exists(p + ".part")
    assert ds.fetch_shard(3, str(tmp_path), opener=flaky) == p and calls["n"] == 2        # already there: no request

    def dead(url):
        raise urllib.error.URLError("no network")
    assert ds.fetch_shard(4, str(tmp_path), attempts=2, opener=dead, sleep=lambda s: None) is None
    done, failed = ds.fetch(2, str(tmp_path), workers=2, opener=dead, attempts=1, sleep=lambda s: None)
    assert failed == [0, 1, ds.LAST_SHARD] and done == []


def test_nanochat_tokenizer_and_loader_under_the_reference_names(tmp_path):
    """`tokenizer.NanoChatBPETokenizer` (train / save / load / encode / decode) and
    `dataloader.tokenizing_distributed_data_loader` over a parquet shard written here."""
    import importlib
    import sys
    import pyarrow as pa
    import pyarrow.parquet as pq
    app = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "apps", "nanochat")
    sys.path.insert(0, app)
    try:
        tokmod = importlib.import_module("tokenizer")
        loader = importlib.import_module("dataloader")
        docs = [f"the quick brown fox {i} jumps over the lazy dog number {i * 7}" for i in range(200)]
        cfg = tokmod.NanoChatTokenizerConfig(vocab_size=400)
        tk = tokmod.NanoChatBPETokenizer.train(iter(docs), config=cfg)
        assert tk.vocab_size <= 400 and tk._bos_id is not None and tk._eos_id is not None
        ids = tk.encode("the quick brown fox")
        assert ids[0] == tk._bos_id and ids[-1] == tk._eos_id
        assert tk.decode(ids) == "the quick brown fox"
        assert tk.encode("lazy dog", add_special_tokens=False) == tk.encode_batch(["lazy dog"], add_special_tokens=False)[0]
        path = tk.save(tmp_path / "tok")
        back = tokmod.NanoChatBPETokenizer.load(path)
        assert back.encode("jumps over") == tk.encode("jumps over") and back.config.vocab_size == 400
        txt = tmp_path / "a.txt"
        txt.write_text("one\n\n two \n")
        assert list(tokmod.iter_file_lines([txt])) == ["one", "two"]
        data = tmp_path / "shards"
        data.mkdir()
        pq.write_table(pa.table({"text": docs}), data / "shard_00000.parquet", row_group_size=64)
        assert loader.get_dist_info() == (False, 0, 0, 1)
        assert [p.name for p in loader.discover_parquet_files(data, "val")] == ["shard_00000.parquet"]
        it = loader.tokenizing_distributed_data_loader(2, 16, path, data, split="train", device="cpu")
        x, y = next(it)
        assert x.shape == (2, 16) and y.shape == (2, 16) and x.dtype == np.int64
        assert np.array_equal(x.reshape(-1)[1:], y.reshape(-1)[:-1]) and x[0, 0] == tk._bos_id
    finally:
        sys.path.remove(app)
        for m in ("tokenizer", "dataloader", "data"):
            sys.modules.pop(m, None)


def test_bench_reference_arm_prints_one_json_line_and_help_lists_the_contract_flags():
    """`bench.py --impl reference` must print exactly one JSON line (here: why the arm is unavailable) and exit 0, on
    any machine; the flags the measurement contract names exist."""
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--gpus", "1",
                        "--steps", "2", "--warmup", "3"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and isinstance(rec.get("unavailable"), str) and rec["unavailable"]
    h = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--help"], capture_output=True, text=True,
                       timeout=300).stdout
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--grad-wire", "--bucket-mb", "--moe", "--no-graph"):
        assert flag in h, flag
