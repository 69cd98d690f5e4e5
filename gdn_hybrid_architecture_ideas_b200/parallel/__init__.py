from .data_parallel import DataParallel, from_environment  # noqa: F401
