"""`genesis.backends.cpu` of the reference."""
from . import CPUStorage  # noqa: F401
