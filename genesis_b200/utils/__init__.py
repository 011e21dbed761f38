from .profile import profile
from . import data
from .data import Dataset, IterableDataset, DataLoader
from . import metrics
