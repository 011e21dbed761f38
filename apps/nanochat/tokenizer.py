"""Byte-level BPE tokenizer of the nanochat app under the names of the reference's `apps/nanochat/tokenizer.py`
(`NanoChatTokenizerConfig`, `NanoChatBPETokenizer` with train / encode / decode / save / load, `iter_file_lines`).
Backed by the HuggingFace `tokenizers` library; files are the library's own `tokenizer.json`, so a tokenizer trained by
either code base loads in the other.  Special tokens named in the configuration are appended after the learned
vocabulary in the given order."""
import json
import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Iterable, Iterator, List, Optional, Sequence


@dataclass
class NanoChatTokenizerConfig:
    vocab_size: int = 32_000
    special_tokens: Sequence[str] = ("<|unk|>", "<|pad|>", "<|bos|>", "<|eos|>")
    regex_pattern: Optional[str] = None
    add_bos_token: bool = True
    add_eos_token: bool = True


class NanoChatBPETokenizer:
    def __init__(self, tokenizer, config: NanoChatTokenizerConfig):
        self._tokenizer = tokenizer
        self._config = config
        self._bos_id = tokenizer.token_to_id("<|bos|>")
        self._eos_id = tokenizer.token_to_id("<|eos|>")
        ids = (tokenizer.token_to_id(t) for t in config.special_tokens)
        self._special_token_ids = {i for i in ids if i is not None}

    @property
    def tokenizer(self):
        return self._tokenizer

    @property
    def config(self) -> NanoChatTokenizerConfig:
        return self._config

    @property
    def vocab_size(self) -> int:
        return self._tokenizer.get_vocab_size()

    @classmethod
    def train(cls, text_iterator: Iterable[str], *, config: Optional[NanoChatTokenizerConfig] = None):
        from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers
        config = config or NanoChatTokenizerConfig()
        tk = Tokenizer(models.BPE(unk_token="<|unk|>" if "<|unk|>" in config.special_tokens else None))
        byte_level = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=config.regex_pattern is None)
        if config.regex_pattern is None:
            tk.pre_tokenizer = byte_level
        else:
            tk.pre_tokenizer = pre_tokenizers.Sequence(
                [pre_tokenizers.Split(Regex(config.regex_pattern), behavior="isolated"), byte_level])
        tk.decoder = decoders.ByteLevel()
        n_special = len(config.special_tokens)
        trainer = trainers.BpeTrainer(vocab_size=max(config.vocab_size - n_special, 256), special_tokens=[],
                                      initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False)
        tk.train_from_iterator(text_iterator, trainer)
        tk.add_special_tokens(list(config.special_tokens))          # after the learned tokens, in the given order
        return cls(tk, config)

    def _wrap(self, ids, add_special_tokens):
        if add_special_tokens:
            if self._config.add_bos_token and self._bos_id is not None:
                ids = [self._bos_id] + ids
            if self._config.add_eos_token and self._eos_id is not None:
                ids = ids + [self._eos_id]
        return ids

    def encode(self, text: str, *, add_special_tokens: bool = True) -> List[int]:
        return self._wrap(self._tokenizer.encode(text, add_special_tokens=False).ids, add_special_tokens)

    def encode_batch(self, texts: Sequence[str], *, add_special_tokens: bool = True) -> List[List[int]]:
        encs = self._tokenizer.encode_batch(list(texts), add_special_tokens=False)
        return [self._wrap(e.ids, add_special_tokens) for e in encs]

    def decode(self, ids: Sequence[int], *, skip_special_tokens: bool = True) -> str:
        ids = [int(i) for i in ids if not (skip_special_tokens and int(i) in self._special_token_ids)]
        return self._tokenizer.decode(ids, skip_special_tokens=False)

    def decode_batch(self, batch_ids: Sequence[Sequence[int]], *, skip_special_tokens: bool = True) -> List[str]:
        return [self.decode(ids, skip_special_tokens=skip_special_tokens) for ids in batch_ids]

    def save(self, output_dir: Path, filename: str = "tokenizer.json") -> Path:
        output_dir = Path(output_dir)
        output_dir.mkdir(parents=True, exist_ok=True)
        path = output_dir / filename
        self._tokenizer.save(str(path))
        meta = {"vocab_size": self._config.vocab_size, "special_tokens": list(self._config.special_tokens),
                "regex_pattern": self._config.regex_pattern, "add_bos_token": self._config.add_bos_token,
                "add_eos_token": self._config.add_eos_token}
        with open(str(path) + ".config", "w", encoding="utf-8") as f:
            json.dump(meta, f)
        return path

    @classmethod
    def load(cls, tokenizer_path: Path):
        from tokenizers import Tokenizer
        tokenizer_path = Path(tokenizer_path)
        tk = Tokenizer.from_file(str(tokenizer_path))
        cfg = NanoChatTokenizerConfig(vocab_size=tk.get_vocab_size())
        side = str(tokenizer_path) + ".config"
        if os.path.exists(side):
            with open(side, encoding="utf-8") as f:
                meta = json.load(f)
            cfg = NanoChatTokenizerConfig(**{**meta, "special_tokens": tuple(meta["special_tokens"])})
        return cls(tk, cfg)


def iter_file_lines(files: Sequence[Path]) -> Iterator[str]:
    """Non-empty lines of a collection of text files."""
    for p in files:
        with Path(p).open("r", encoding="utf-8") as f:
            for line in f:
                line = line.strip()
                if line:
                    yield line
