"""Package logger. Console output is always on; the file handler is attached lazily by
`setup_file_logging` (the reference creates `output/logs/pipeline.log` in the working directory at
import time, src/nanoplm/utils/logger.py:6-28 — here importing the package has no side effects)."""
from __future__ import annotations

import logging
import sys
from pathlib import Path

logger = logging.getLogger("nanoplm_b200")
if not logger.handlers:
    _h = logging.StreamHandler(sys.stdout)
    _h.setFormatter(logging.Formatter("%(message)s"))
    logger.addHandler(_h)
    logger.setLevel(logging.INFO)
    logger.propagate = False


def setup_file_logging(log_dir: str | Path = "output/logs", filename: str = "pipeline.log") -> Path:
    d = Path(log_dir)
    d.mkdir(parents=True, exist_ok=True)
    path = d / filename
    for h in logger.handlers:
        if isinstance(h, logging.FileHandler) and Path(h.baseFilename) == path.resolve():
            return path
    fh = logging.FileHandler(path)
    fh.setFormatter(logging.Formatter("%(asctime)s - %(levelname)s - %(message)s"))
    logger.addHandler(fh)
    return path


def log_stage(name: str) -> None:
    logger.info("=" * 60)
    logger.info(f"  {name}")
    logger.info("=" * 60)
