from grace_b200.parallel.optimizer import DistributedOptimizer  # noqa: F401
