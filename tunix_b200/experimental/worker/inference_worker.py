"""`InferenceWorker` (tunix/experimental/worker/inference_worker.py); defined beside the other workers."""
from .rollout_worker import InferenceWorker  # noqa: F401
