"""Package logger (dlblas/utils/logger.py:32-39 of the reference): INFO level, one stream handler."""
import logging

_FMT = "%(asctime)s %(name)s [%(levelname)s] %(message)s"


def get_logger(name: str = "dlblas_b200", level: int = logging.INFO) -> logging.Logger:
    logger = logging.getLogger(name)
    if not logger.handlers:
        h = logging.StreamHandler()
        h.setFormatter(logging.Formatter(_FMT))
        logger.addHandler(h)
        logger.propagate = False
    logger.setLevel(level)
    return logger
