from grace_b200.memory.powersgd import PowerSGDMemory  # noqa: F401
