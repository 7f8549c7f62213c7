from grace_b200.memory.residual import ResidualMemory  # noqa: F401
