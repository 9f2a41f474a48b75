from .dynamicgen_dataset import AbstractDataGenerator, DynamicGenDataset, MockDataGenerator  # noqa: F401
