from .policy import RidazenPolicy  # noqa: F401
