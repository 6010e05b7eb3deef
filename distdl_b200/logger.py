"""Package logger.  Level from ``DISTDL_LOGLEVEL`` (default ERROR); messages go
to stdout at the chosen level and, when ``DISTDL_LOGFILE`` names a path, to
that file at DEBUG (the reference always writes ``distdl.log`` into the
working directory, ``src/distdl/logger.py:23-33``; here that is opt-in so
that importing the package never litters the CWD)."""
import logging
import os
import sys

logger = logging.getLogger("DistDL-Logger")
_level = getattr(logging, os.environ.get("DISTDL_LOGLEVEL", "ERROR").upper(), logging.ERROR)
logger.setLevel(min(_level, logging.DEBUG) if os.environ.get("DISTDL_LOGFILE") else _level)
_fmt = logging.Formatter("%(asctime)s [pid %(process)d] %(levelname)s %(pathname)s:%(lineno)d: %(message)s")
if not logger.handlers:
    _h = logging.StreamHandler(sys.stdout)
    _h.setLevel(_level)
    _h.setFormatter(_fmt)
    logger.addHandler(_h)
    if os.environ.get("DISTDL_LOGFILE"):
        _f = logging.FileHandler(os.environ["DISTDL_LOGFILE"])
        _f.setLevel(logging.DEBUG)
        _f.setFormatter(_fmt)
        logger.addHandler(_f)
logger.propagate = False
