"""Package logger.  ``OMNI_LOGGING_PREFIX`` (or the reference's ``VLLM_LOGGING_PREFIX``,
vllm_omni/entrypoints/omni_stage.py:447-449) tags every record with the stage name."""
import logging
import os
import sys

_FMT = "%(levelname)s %(asctime)s [%(name)s] %(prefix)s%(message)s"


class _Prefix(logging.Filter):
    def filter(self, record):
        record.prefix = os.environ.get("OMNI_LOGGING_PREFIX", os.environ.get("VLLM_LOGGING_PREFIX", ""))
        return True


def init_logger(name: str) -> logging.Logger:
    root = logging.getLogger("vllm_omni_b200")
    if not root.handlers:
        h = logging.StreamHandler(sys.stderr)
        h.setFormatter(logging.Formatter(_FMT, datefmt="%m-%d %H:%M:%S"))
        h.addFilter(_Prefix())
        root.addHandler(h)
        root.setLevel(os.environ.get("OMNI_LOG_LEVEL", "WARNING").upper())
        root.propagate = False
    return logging.getLogger(name if name.startswith("vllm_omni_b200") else f"vllm_omni_b200.{name}")
