"""A prompt dataset that grows during training (verl/experimental/dynamic_dataset/dynamicgen_dataset.py:38-113).

``data.datagen.{path,name}`` names an :class:`AbstractDataGenerator`; after each training batch the trainer calls
``dataset.on_batch_end(batch)`` and the generator's new rows are appended (over-long prompts filtered as usual)."""

from __future__ import annotations

import copy
import logging
from abc import ABC, abstractmethod
from typing import Optional

from ...utils.dataset.rl_dataset import RLHFDataset
from ...utils.py_functional import load_extern_object

logger = logging.getLogger(__name__)


class AbstractDataGenerator(ABC):
    def __init__(self, config=None):
        self.config = config

    @abstractmethod
    def generate(self, dataset: RLHFDataset) -> list[dict]:
        """Return new rows (same columns as the dataset's rows)."""


class MockDataGenerator(AbstractDataGenerator):
    """Re-adds the first row: enough to exercise the plumbing."""

    def generate(self, dataset: RLHFDataset) -> list[dict]:
        return [copy.deepcopy(dataset.rows[0])] if dataset.rows else []


class DynamicGenDataset(RLHFDataset):
    def __init__(self, data_files, tokenizer, config, processor=None, max_samples: int = -1):
        super().__init__(data_files, tokenizer, config, processor, max_samples)
        dg = config.get("datagen") if hasattr(config, "get") else None
        if not dg or not dg.get("path"):
            raise AssertionError(f"datagen path is not set in config: {config}")
        cls = load_extern_object(dg["path"], dg["name"])
        if not (isinstance(cls, type) and issubclass(cls, AbstractDataGenerator)):
            raise TypeError(f"The custom datagen class '{dg['name']}' from '{dg['path']}' must inherit from "
                            f"{AbstractDataGenerator}")
        self.data_generator = cls(dg)
        self.on_batch_end()

    def append_dataframe(self, new_rows: list[dict]) -> None:
        if self.filter_overlong_prompts:
            new_rows = [r for r in new_rows if len(self._tokenize(r[self.prompt_key])) <= self.max_prompt_length]
        self.rows.extend(new_rows)
        logger.info("new dataset len: %d", len(self.rows))

    def on_batch_end(self, batch: Optional[object] = None) -> None:
        self.append_dataframe(list(self.data_generator.generate(self)))
