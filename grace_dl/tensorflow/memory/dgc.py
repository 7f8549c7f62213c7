from grace_b200.memory.dgc import DgcMemory  # noqa: F401
