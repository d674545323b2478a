"""Executors: how the engine core reaches its workers."""
from .base import Executor, make_executor  # noqa: F401
