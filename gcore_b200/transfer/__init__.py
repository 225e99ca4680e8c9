from .tq_connector import SimpleStorage, TransferQueue, make_key  # noqa: F401
