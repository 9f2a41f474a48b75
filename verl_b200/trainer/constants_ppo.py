"""Environment injected into every worker process (role of verl/trainer/constants_ppo.py:1-59). The vLLM entries
of the reference have no counterpart; the NCCL ones matter for the plumbing collectives."""

import os

PPO_RAY_RUNTIME_ENV = {
    "env_vars": {
        "TOKENIZERS_PARALLELISM": "true",
        "NCCL_DEBUG": "WARN",
        "CUDA_DEVICE_MAX_CONNECTIONS": "1",
        "NCCL_CUMEM_ENABLE": "0",
    },
}


def get_ppo_ray_runtime_env() -> dict:
    """A copy without the variables the user already set (those win)."""
    env = {k: v for k, v in PPO_RAY_RUNTIME_ENV["env_vars"].items() if k not in os.environ}
    return {"env_vars": env}
