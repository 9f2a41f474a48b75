from .env_loop import EnvLoop, EnvWorker, NaiveRolloutRob  # noqa: F401
from .envs.synthetic_env import SyntheticReachEnv  # noqa: F401
