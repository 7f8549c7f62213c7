from grace_b200.compressor.qsgd import QSGDCompressor  # noqa: F401
