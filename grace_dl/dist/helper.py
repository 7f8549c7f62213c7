from grace_b200.helper import grace_from_params  # noqa: F401
