"""hf_integration.py of the reference's GPU package."""
from polarquant_kv.hf_integration import *  # noqa: F401,F403
