from .sampler import AbstractCurriculumSampler, AbstractSampler, DifficultyCurriculumSampler  # noqa: F401
