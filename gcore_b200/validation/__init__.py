"""In-training validation of the text-to-image trainers (the reference's ``gpatch_v4/validation`` package)."""
from .runner import EmbeddingMetrics, ValidationRunner, restore_modes, snapshot_modes

__all__ = ["EmbeddingMetrics", "ValidationRunner", "restore_modes", "snapshot_modes"]
