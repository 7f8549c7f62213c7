from grace_b200.compressor.inceptionn import INCEPTIONNCompressor  # noqa: F401
