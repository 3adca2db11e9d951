from .pool import CacheFull, CacheMisuse, FreeList  # noqa: F401
from .paged import PAGE_SIZE, GroupLayout, PagedCache, SlotBook, plan_groups  # noqa: F401
