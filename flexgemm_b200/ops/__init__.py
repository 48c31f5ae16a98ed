from . import spconv, utils  # noqa: F401
