"""``grace_from_params`` with the key set of ``grace_dl/tensorflow/helper.py:1-107`` (adds ``adaq``,
``inceptionn`` with ``error_bound``, ``sketch`` with ``quantiles``, ``u8bit``); builds PyTorch objects."""
from grace_b200.helper import grace_from_params  # noqa: F401
