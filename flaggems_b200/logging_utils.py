"""Operator-call log (mirror of ``src/flag_gems/logging_utils.py:18-39``).

``enable(record=True, path=..., once=...)`` attaches a file handler to the logger
``flag_gems``; every operator wrapper emits one ``GEMS ...`` debug record per call.
"""
import logging
from pathlib import Path


class LogOncePerLocationFilter(logging.Filter):
    """Let each (file, line) call site through only once."""

    def __init__(self):
        super().__init__()
        self.logged_locations = set()

    def filter(self, record):
        key = (record.pathname, record.lineno)
        if key in self.logged_locations:
            return False
        self.logged_locations.add(key)
        return True


def setup_flaggems_logging(path=None, record=True, once=False):
    if not record:
        return
    filename = Path(path or Path.home() / ".flaggems/oplist.log")
    filename.parent.mkdir(parents=True, exist_ok=True)
    handler = logging.FileHandler(filename, mode="w")
    if once:
        handler.addFilter(LogOncePerLocationFilter())
    handler.setFormatter(logging.Formatter("[%(levelname)s] %(name)s: %(message)s"))
    logger = logging.getLogger("flag_gems")
    logger.setLevel(logging.DEBUG)
    if not any(isinstance(h, logging.FileHandler) for h in logger.handlers):
        logger.addHandler(handler)
    logger.propagate = False


def teardown_flaggems_logging():
    logger = logging.getLogger("flag_gems")
    for h in list(logger.handlers):
        if isinstance(h, logging.FileHandler):
            h.close()
            logger.removeHandler(h)
