from .naive_router import NaiveRouter  # noqa: F401
