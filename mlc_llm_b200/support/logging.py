"""Logging set-up shared by the command-line tools (reference: ``python/mlc_llm/support/logging.py``)."""
import logging


def enable_logging(level: int = logging.INFO) -> None:
    logging.basicConfig(level=level, style="{", datefmt="%Y-%m-%d %H:%M:%S",
                        format="[{asctime}] {levelname} {filename}:{lineno}: {message}")


def getLogger(name: str) -> logging.Logger:  # pylint: disable=invalid-name
    return logging.getLogger(name)
