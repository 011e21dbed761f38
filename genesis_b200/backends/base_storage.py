"""`genesis.backends.base_storage` of the reference."""
from . import Storage  # noqa: F401
