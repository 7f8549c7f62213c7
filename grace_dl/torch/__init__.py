"""``grace_dl.torch`` compatibility namespace."""
from grace_b200.core import Communicator, Compressor, Memory  # noqa: F401
