"""utils.py of the reference's GPU package."""
from polarquant_kv.utils import *  # noqa: F401,F403
from polarquant_kv.utils import check_memory_warning, cosine_similarity, estimate_memory_bytes  # noqa: F401
