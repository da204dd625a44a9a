"""Rank-0 console logger and scalar loggers (reference: ironcore/logger.py:34-210)."""

from ironcore_b200.utils.logging import *  # noqa: F401,F403
