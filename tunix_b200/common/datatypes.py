"""Shared enums (tunix/common/datatypes.py:20-37)."""
import enum


class Mode(str, enum.Enum):
    TRAIN = "train"
    EVAL = "eval"

    def __str__(self):
        return self.value


class Role(str, enum.Enum):
    ACTOR = "actor"
    CRITIC = "critic"
    REFERENCE = "reference"
    REWARD = "reward"
    ROLLOUT = "rollout"

    def __str__(self):
        return self.value
