from .keys import as_signed, draw_key, uniform_from_key

__all__ = ["as_signed", "draw_key", "uniform_from_key"]
