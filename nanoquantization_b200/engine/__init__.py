from .engine import BlockManager, LLMEngine, PagedKVCache, Scheduler, Sequence  # noqa: F401
