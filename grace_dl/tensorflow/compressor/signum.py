from grace_b200.compressor.signum import SignumCompressor  # noqa: F401
