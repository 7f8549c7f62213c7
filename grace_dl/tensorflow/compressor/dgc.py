from grace_b200.compressor.dgc import DgcCompressor  # noqa: F401
