from .loader import load_model, save_model, shard_slices  # noqa: F401
