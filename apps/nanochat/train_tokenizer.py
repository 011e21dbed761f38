"""Trains a byte-level BPE tokenizer (HuggingFace `tokenizers`) on the text shards and writes tokenizer.json.

    python apps/nanochat/train_tokenizer.py --data /path/to/shards --vocab-size 65536 --out tokenizer.json
Reference counterpart: apps/nanochat/train_tokenizer.py, tokenizer.py.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--data", required=True)
    ap.add_argument("--vocab-size", type=int, default=65536)
    ap.add_argument("--max-chars", type=int, default=2_000_000_000)
    ap.add_argument("--out", default="tokenizer.json")
    a = ap.parse_args(argv)
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    import data as D

    def texts():
        seen = 0
        for path in D.list_shards(a.data, "train"):
            if path.endswith(".npy"):
                continue
            for batch in D._texts(path, 256):
                for t in batch:
                    seen += len(t)
                    yield t
                if seen >= a.max_chars:
                    return

    tk = Tokenizer(models.BPE())
    tk.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tk.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=a.vocab_size, special_tokens=["<|bos|>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tk.train_from_iterator(texts(), trainer)
    tk.save(a.out)
    print(f"wrote {a.out} (vocab {tk.get_vocab_size()})")


if __name__ == "__main__":
    main()
