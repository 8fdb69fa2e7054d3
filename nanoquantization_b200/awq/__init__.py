from .search import best_clip, best_scales, pseudo_quantize  # noqa: F401
