from grace_b200.compressor.onebit import OneBitCompressor  # noqa: F401
