from grace_b200.memory.none import NoneMemory  # noqa: F401
