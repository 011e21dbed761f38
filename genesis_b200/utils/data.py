"""Minimal dataset / loader. Parity: reference `genesis/utils/data.py:5-54`."""
import random


class Dataset:
    def __getitem__(self, idx):
        raise NotImplementedError

    def __len__(self):
        raise NotImplementedError


class IterableDataset:
    def __iter__(self):
        raise NotImplementedError


class DataLoader:
    """Batches of `batch_size` items as lists; optional shuffling of map-style datasets."""

    def __init__(self, dataset, batch_size=1, shuffle=False, drop_last=False):
        self.dataset, self.batch_size, self.shuffle, self.drop_last = dataset, batch_size, shuffle, drop_last

    def __iter__(self):
        if isinstance(self.dataset, IterableDataset) or not hasattr(self.dataset, "__getitem__"):
            batch = []
            for item in self.dataset:
                batch.append(item)
                if len(batch) == self.batch_size:
                    yield batch
                    batch = []
            if batch and not self.drop_last:
                yield batch
            return
        idx = list(range(len(self.dataset)))
        if self.shuffle:
            random.shuffle(idx)
        for i in range(0, len(idx), self.batch_size):
            chunk = idx[i:i + self.batch_size]
            if len(chunk) < self.batch_size and self.drop_last:
                break
            yield [self.dataset[j] for j in chunk]

    def __len__(self):
        n = len(self.dataset)
        return n // self.batch_size if self.drop_last else (n + self.batch_size - 1) // self.batch_size
