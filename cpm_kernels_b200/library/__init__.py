from . import base, cpmk  # noqa: F401
