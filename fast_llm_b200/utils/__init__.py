from fast_llm_b200.utils.assertions import Assert  # noqa: F401
from fast_llm_b200.utils.misc import (  # noqa: F401
    Interrupter,
    InvalidObject,
    Registry,
    compare_nested,
    div,
    get_and_reset_memory_usage_mib,
    get_unique,
    padded_cumsum,
    safe_merge_dicts,
    set_global_variables,
    try_decorate,
)
