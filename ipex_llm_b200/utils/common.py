"""Error convention of the reference (ipex_llm/utils/common/log4Error.py:22-32):
``invalidInputError(cond, msg, fix)`` logs a banner and raises ``RuntimeError(msg)``."""
import logging

logger = logging.getLogger("ipex_llm_b200")


def invalidInputError(condition, errMsg, fixMsg=None):
    if not condition:
        logger.error("\n\n****************************Usage Error************************\n" + errMsg)
        if fixMsg:
            logger.error("\n\n**************************How to fix***********************\n" + fixMsg)
        raise RuntimeError(errMsg)


def invalidOperationError(condition, errMsg, fixMsg=None, cause=None):
    if not condition:
        logger.error("\n\n****************************Usage Error************************\n" + errMsg)
        if cause:
            raise cause
        raise RuntimeError(errMsg)


class LazyModule:
    """A module that is imported at its first attribute access.  The ctypes bindings load (and need) their shared
    library when they are imported; a module that merely names one of them -- the cache classes, say, of which only some
    call that library -- binds it through this and stays importable without it."""

    def __init__(self, name):
        self.__dict__["_name"], self.__dict__["_mod"] = name, None

    def __getattr__(self, attr):
        if self.__dict__["_mod"] is None:
            import importlib
            self.__dict__["_mod"] = importlib.import_module(self.__dict__["_name"])
        return getattr(self.__dict__["_mod"], attr)
