import refshim  # noqa: F401
