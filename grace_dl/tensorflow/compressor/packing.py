from grace_b200.compressor.packing import *  # noqa: F401,F403
