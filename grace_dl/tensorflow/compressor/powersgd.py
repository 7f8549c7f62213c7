from grace_b200.compressor.powersgd import PowerSGDCompressor  # noqa: F401
