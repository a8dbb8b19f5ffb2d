"""inference/config.py of the reference's GPU package."""
from polarquant_kv.inference.config import PolarQuantConfig  # noqa: F401
