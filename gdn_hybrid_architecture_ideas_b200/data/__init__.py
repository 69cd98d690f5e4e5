from .synthetic import Batch, SyntheticPackedData, UniformTokens, counter_generator, make_data  # noqa: F401
