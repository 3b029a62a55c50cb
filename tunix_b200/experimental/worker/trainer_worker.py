"""`TrainerWorker` (tunix/experimental/worker/trainer_worker.py); defined beside the other workers."""
from .rollout_worker import TrainerWorker  # noqa: F401
