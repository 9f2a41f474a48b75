from .losses import ppo_loss, sft_loss, value_loss  # noqa: F401
from .padding import left_right_2_no_padding, no_padding_2_padding  # noqa: F401
