from grace_b200.compressor.threshold import ThresholdCompressor  # noqa: F401
