from .fully_async import FullyAsyncRollouter, FullyAsyncTrainer, MetricsAggregator, run_fully_async  # noqa: F401
from .message_queue import MessageQueue, QueueSample  # noqa: F401
from .param_sync import ParameterSynchronizer  # noqa: F401
