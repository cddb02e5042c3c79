from .pages import CacheBooks, CacheError, ContextFull, OutOfPages, PagePool, TooManyRequests

__all__ = ["CacheBooks", "CacheError", "ContextFull", "OutOfPages", "PagePool", "TooManyRequests"]
