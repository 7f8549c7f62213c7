from grace_b200.compressor.signsgd import SignSGDCompressor  # noqa: F401
