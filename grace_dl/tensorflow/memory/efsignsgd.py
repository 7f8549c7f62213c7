from grace_b200.memory.efsignsgd import EFSignSGDMemory  # noqa: F401
