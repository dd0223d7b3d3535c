from .options import SamplingOptions  # noqa: F401
