from .cache import CacheManager
from .decode import DecodeManager
from .prefill import PrefillAdder, PrefillManager
from .scheduler import RequestAllFinished, Scheduler
from .table import TableManager

__all__ = ["CacheManager", "DecodeManager", "PrefillAdder", "PrefillManager", "RequestAllFinished",
           "Scheduler", "TableManager"]
