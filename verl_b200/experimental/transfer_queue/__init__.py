from .queue import BatchMeta, TransferQueue, get_transfer_queue, set_transfer_queue, tqbridge  # noqa: F401
