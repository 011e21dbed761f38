"""`genesis.backends.base` of the reference."""
from . import Storage  # noqa: F401
