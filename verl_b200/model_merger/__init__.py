from .merger import merge_checkpoint, test_merged  # noqa: F401
