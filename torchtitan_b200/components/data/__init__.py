from .loader import BaseDataLoader, DataloaderExhaustedError, PrefetchIterator, SyntheticDataLoader

__all__ = ["BaseDataLoader", "DataloaderExhaustedError", "PrefetchIterator", "SyntheticDataLoader"]
