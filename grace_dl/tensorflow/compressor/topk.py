from grace_b200.compressor.topk import TopKCompressor  # noqa: F401
