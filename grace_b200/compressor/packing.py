"""2-bit x 4 -> byte packing helpers.
Reference: ``grace_dl/tensorflow/compressor/packing.py:4-29``."""
from .inceptionn import pack2 as encode_byte, unpack2 as decode_byte  # noqa: F401
