from .reward_loop import RewardLoopManager, RewardLoopWorker  # noqa: F401
from .reward_manager import (AsyncTokenBucket, DAPORewardManager, NaiveRewardManager, RateLimitedRewardManager,  # noqa: F401
                             RemoteRewardManager, get_reward_manager_cls, register)
from .reward_model import RewardModelManager  # noqa: F401
