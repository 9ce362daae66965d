from .paged_cache import PagedCache, host_runtime
from .specs import PagedKVBinding, PagedKVSpec, SlotStateBinding, SlotStateSpec

__all__ = ["PagedCache", "host_runtime", "PagedKVBinding", "PagedKVSpec", "SlotStateBinding", "SlotStateSpec"]
