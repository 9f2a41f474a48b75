from .ray_trainer import OneStepOffRayTrainer  # noqa: F401
