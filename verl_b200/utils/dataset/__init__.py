from .rl_dataset import RLHFDataset, SyntheticPromptDataset, collate_fn

__all__ = ["RLHFDataset", "SyntheticPromptDataset", "collate_fn"]
