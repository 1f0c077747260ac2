"""Trainer life-cycle interface (primus/core/trainer/base_trainer.py:28-141 in the reference)."""
from __future__ import annotations

import abc
import os


class BaseTrainer(abc.ABC):
    def __init__(self, params: dict, experiment=None, runtime_state=None):
        self.params = params
        self.experiment = experiment
        self.runtime_state = runtime_state
        self.rank = int(os.environ.get("RANK", 0))
        self.world_size = int(os.environ.get("WORLD_SIZE", 1))
        self.local_rank = int(os.environ.get("LOCAL_RANK", 0))

    def setup(self):
        """Process-level set-up (distributed init, devices)."""

    @abc.abstractmethod
    def init(self):
        """Build model, optimizer, data."""

    @abc.abstractmethod
    def train(self):
        ...

    def cleanup(self):
        """Tear-down (barriers, artifact upload, process-group destruction)."""
