from grace_b200.compressor.randomk import RandomKCompressor  # noqa: F401
