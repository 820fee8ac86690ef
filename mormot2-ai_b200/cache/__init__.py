"""The cache: host bookkeeping of slots and pages (``pages``), device storage (``storage``)."""
from .pages import PAGE, CacheBook, FreeList, GroupPlan, pages_for, plan_groups

__all__ = ["PAGE", "CacheBook", "FreeList", "GroupPlan", "pages_for", "plan_groups"]
