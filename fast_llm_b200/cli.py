"""`fast-llm <train|convert|evaluate|prepare> <model> [-c config.yaml] [key=value ...]` (parity: `fast_llm/cli.py`)."""

import logging
import sys
import traceback

logger = logging.getLogger(__name__)


def fast_llm_main(args: list[str] | None = None):
    from fast_llm_b200.config import ValidationError
    from fast_llm_b200.config.runnable import RunnableConfig
    from fast_llm_b200.utils import set_global_variables

    set_global_variables()
    import fast_llm_b200.models.auto  # noqa: F401  (fills the registries)

    try:
        return RunnableConfig.parse_and_run(args)
    except ValidationError:
        logger.error("Config validation failed")
        raise
    except Exception:
        logger.critical(traceback.format_exc())
        raise


if __name__ == "__main__":
    fast_llm_main(sys.argv[1:])
