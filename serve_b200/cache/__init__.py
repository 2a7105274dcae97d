from .manager import CacheManager, CacheView, NoFreeSlot  # noqa: F401
from .pages import OutOfPages, PagePool  # noqa: F401
