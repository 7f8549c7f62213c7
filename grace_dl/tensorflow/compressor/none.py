from grace_b200.compressor.none import NoneCompressor  # noqa: F401
