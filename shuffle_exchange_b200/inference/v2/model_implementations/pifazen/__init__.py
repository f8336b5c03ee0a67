from .policy import PifazenPolicy  # noqa: F401
