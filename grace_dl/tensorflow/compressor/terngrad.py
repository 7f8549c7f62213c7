from grace_b200.compressor.terngrad import TernGradCompressor  # noqa: F401
