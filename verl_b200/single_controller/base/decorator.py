"""``@register`` and the dispatch / collect functions that move data between the controller and
SPMD workers. Same public names as verl/single_controller/base/decorator.py (Dispatch, Execute,
register, make_nd_compute_dataproto_dispatch_fn, register_dispatch_mode ...).

A dispatch function turns the controller-side call arguments into one argument tuple per worker;
a collect function merges the per-worker results. Data-parallel modes split ``DataProto`` (or
``DataProtoFuture``) arguments evenly and concatenate the results.
"""

from __future__ import annotations

import inspect
from enum import Enum
from functools import partial, wraps

from ...protocol import DataProto, DataProtoFuture, _PAD_KEY, pad_dataproto_to_divisor, unpad_dataproto

MAGIC_ATTR = "attrs_3141562937"


class DynamicEnumMeta(type):
    def __iter__(cls):
        return iter(cls._registry.values())

    def __contains__(cls, item):
        if isinstance(item, str):
            return item in cls._registry
        return item in cls._registry.values()

    def __getitem__(cls, name):
        return cls._registry[name]

    def __getattr__(cls, name):
        reg = cls.__dict__.get("_registry", {})
        if name in reg:
            return reg[name]
        raise AttributeError(name)


class DynamicEnum(metaclass=DynamicEnumMeta):
    _registry: dict = {}
    _next_value = 0

    def __init__(self, name: str, value: int):
        self.name, self.value = name, value

    def __repr__(self):
        return f"<{self.__class__.__name__}.{self.name}: {self.value}>"

    def __reduce__(self):
        return (getattr, (self.__class__, self.name))

    @classmethod
    def register(cls, name: str):
        key = name.upper()
        if key in cls._registry:
            raise ValueError(f"{key} already registered")
        val = cls(key, cls._next_value)
        cls._registry[key] = val
        cls._next_value += 1
        return val

    @classmethod
    def remove(cls, name: str):
        return cls._registry.pop(name.upper())

    @classmethod
    def from_name(cls, name: str):
        return cls._registry.get(name.upper())


class Dispatch(DynamicEnum):
    _registry = {}
    _next_value = 0


for _n in ("RANK_ZERO", "ONE_TO_ALL", "ALL_TO_ALL", "DP_COMPUTE", "DP_COMPUTE_PROTO", "DP_COMPUTE_PROTO_WITH_FUNC",
           "DP_COMPUTE_METRIC", "DIRECT_ROLLOUT_METHOD"):
    Dispatch.register(_n)


def init_predefined_dispatch_mode():
    """(Re-)register the built-in dispatch modes (after a test removed or shadowed one)."""
    for n in ("RANK_ZERO", "ONE_TO_ALL", "ALL_TO_ALL", "DP_COMPUTE", "DP_COMPUTE_PROTO", "DP_COMPUTE_PROTO_WITH_FUNC",
              "DP_COMPUTE_METRIC", "DIRECT_ROLLOUT_METHOD"):
        if Dispatch.from_name(n) is None:
            Dispatch.register(n)


def init_predefined_execute_mode():
    for n in ("ALL", "RANK_ZERO"):
        if Execute.from_name(n) is None:
            Execute.register(n)


class Execute(DynamicEnum):
    _registry = {}
    _next_value = 0


for _n in ("ALL", "RANK_ZERO"):
    Execute.register(_n)


# ------------------------------------------------------------------- split helpers
def _is_tensordict(x) -> bool:
    from ...utils.tensordict_lite import TensorDict

    return isinstance(x, TensorDict)


def _chunk(x, chunks: int):
    """Equal shares of a DataProto / future / TensorDict (the no-padding batches of the engine workers)."""
    if _is_tensordict(x):
        from ...utils.tensordict_utils import chunk_tensordict

        return chunk_tensordict(x, chunks)
    assert isinstance(x, (DataProto, DataProtoFuture)), f"cannot split argument of type {type(x)}"
    return x.chunk(chunks=chunks)


def _split_args_kwargs_data_proto(chunks: int, *args, **kwargs):
    return [_chunk(a, chunks) for a in args], {k: _chunk(v, chunks) for k, v in kwargs.items()}


def _split_args_kwargs_data_proto_with_auto_padding(chunks: int, *args, **kwargs):
    """Pad every DataProto to a multiple of ``chunks`` first; the pad size is remembered in ``kwargs``
    under the auto-padding key so the collect side can strip it."""
    pad_size = None

    def prep(x):
        nonlocal pad_size
        if _is_tensordict(x):
            return _chunk(x, chunks)
        assert isinstance(x, (DataProto, DataProtoFuture))
        if isinstance(x, DataProto) and x.is_padding_enabled():
            if pad_size is None:
                pad_size = (chunks - len(x) % chunks) % chunks
            x = x[:]  # shallow view; padding must not touch the caller's object
            x.padding(padding_size=pad_size) if pad_size else None
        return x.chunk(chunks=chunks)

    s_args = [prep(a) for a in args]
    s_kwargs = {k: prep(v) for k, v in kwargs.items()}
    if pad_size is not None:
        s_kwargs[_PAD_KEY] = pad_size
    return s_args, s_kwargs


def _concat_data_proto_or_future(outputs: list):
    for o in outputs:
        assert type(o) is type(outputs[0])
    o = outputs[0]
    if isinstance(o, DataProto):
        return DataProto.concat(outputs)
    if isinstance(o, DataProtoFuture) or hasattr(o, "result"):
        # resolved later: the workers' results may be DataProtos or TensorDicts
        return DataProtoFuture(collect_fn=_concat_data_proto_or_future, futures=outputs)
    if _is_tensordict(o):
        from ...utils.tensordict_lite import TensorDict

        return TensorDict.cat(outputs, dim=0)
    raise NotImplementedError(type(o))


# ------------------------------------------------------------------ dispatch modes
def dispatch_one_to_all(worker_group, *args, **kwargs):
    n = worker_group.world_size
    return tuple([a] * n for a in args), {k: [v] * n for k, v in kwargs.items()}


def dummy_direct_rollout_call(worker_group, *args, **kwargs):
    raise NotImplementedError("Direct rollout call is forbidden.")


def dispatch_all_to_all(worker_group, *args, **kwargs):
    return args, kwargs


def collect_all_to_all(worker_group, output):
    return output


def dispatch_dp_compute(worker_group, *args, **kwargs):
    for a in args:
        assert isinstance(a, (tuple, list)) and len(a) == worker_group.world_size
    for v in kwargs.values():
        assert isinstance(v, (tuple, list)) and len(v) == worker_group.world_size
    return args, kwargs


def collect_dp_compute(worker_group, output):
    assert len(output) == worker_group.world_size
    return output


def dispatch_dp_compute_data_proto(worker_group, *args, **kwargs):
    return _split_args_kwargs_data_proto_with_auto_padding(worker_group.world_size, *args, **kwargs)


def dispatch_dp_compute_data_proto_with_func(worker_group, *args, **kwargs):
    assert callable(args[0])
    s_args, s_kwargs = _split_args_kwargs_data_proto(worker_group.world_size, *args[1:], **kwargs)
    return [[args[0]] * worker_group.world_size] + s_args, s_kwargs


def collect_dp_compute_data_proto(worker_group, output):
    for o in output:
        assert isinstance(o, (DataProto, DataProtoFuture)) or hasattr(o, "result"), f"expecting DataProto, got {type(o)}"
    return _concat_data_proto_or_future(collect_dp_compute(worker_group, output))


# ------------------------------------------------- n-d (mesh-aware) compute dispatch
def dispatch_nd_compute(dp_rank_mapping: list[int], dp_size: int, worker_group, *args, **kwargs):
    """Arguments arrive already split into ``dp_size`` pieces; worker i receives piece
    ``dp_rank_mapping[i]`` (workers in the same TP/SP/PP group share a piece)."""
    for a in args:
        assert isinstance(a, (tuple, list)) and len(a) == dp_size
    for v in kwargs.values():
        assert isinstance(v, (tuple, list)) and len(v) == dp_size
    n = worker_group.world_size
    out_args = [[a[dp_rank_mapping[i]] for i in range(n)] for a in args]
    out_kwargs = {k: [v[dp_rank_mapping[i]] for i in range(n)] for k, v in kwargs.items()}
    return out_args, out_kwargs


def collect_nd_compute(collect_mask: list[bool], worker_group, output):
    assert len(output) == worker_group.world_size
    return [o for o, keep in zip(output, collect_mask) if keep]


def dispatch_nd_compute_dataproto(dp_rank_mapping, dp_size, worker_group, *args, **kwargs):
    s_args, s_kwargs = _split_args_kwargs_data_proto(dp_size, *args, **kwargs)
    return dispatch_nd_compute(dp_rank_mapping, dp_size, worker_group, *s_args, **s_kwargs)


def collect_nd_compute_dataproto(collect_mask, worker_group, output):
    output = collect_nd_compute(collect_mask, worker_group, output)
    return _concat_data_proto_or_future(output)


def dispatch_lazy_compute_data_proto(mesh_name: str, worker_group, *args, **kwargs):
    """Mesh-based DP dispatch: the (dp_rank, is_collect) table of ``mesh_name`` is queried from the
    workers on first use and cached on the worker group."""
    if mesh_name not in worker_group._dispatch_info:
        worker_group._dispatch_info[mesh_name] = worker_group._query_dispatch_info(mesh_name)
        assert len(worker_group._dispatch_info[mesh_name]) == worker_group.world_size
    mapping = worker_group._dispatch_info[mesh_name]
    dp_size = max(mapping) + 1
    return dispatch_nd_compute_dataproto(mapping, dp_size, worker_group, *args, **kwargs)


def collect_lazy_compute_data_proto(mesh_name: str, worker_group, *args, **kwargs):
    if mesh_name not in worker_group._collect_info:
        worker_group._collect_info[mesh_name] = worker_group._query_collect_info(mesh_name)
        assert len(worker_group._collect_info[mesh_name]) == worker_group.world_size
    return collect_nd_compute_dataproto(worker_group._collect_info[mesh_name], worker_group, *args, **kwargs)


def make_nd_compute_dataproto_dispatch_fn(mesh_name: str) -> dict:
    return {"dispatch_fn": partial(dispatch_lazy_compute_data_proto, mesh_name),
            "collect_fn": partial(collect_lazy_compute_data_proto, mesh_name)}


DISPATCH_MODE_FN_REGISTRY = {
    Dispatch.ONE_TO_ALL: {"dispatch_fn": dispatch_one_to_all, "collect_fn": collect_all_to_all},
    Dispatch.ALL_TO_ALL: {"dispatch_fn": dispatch_all_to_all, "collect_fn": collect_all_to_all},
    Dispatch.DP_COMPUTE: {"dispatch_fn": dispatch_dp_compute, "collect_fn": collect_dp_compute},
    Dispatch.DP_COMPUTE_PROTO: {"dispatch_fn": dispatch_dp_compute_data_proto,
                                "collect_fn": collect_dp_compute_data_proto},
    Dispatch.DP_COMPUTE_PROTO_WITH_FUNC: {"dispatch_fn": dispatch_dp_compute_data_proto_with_func,
                                          "collect_fn": collect_dp_compute_data_proto},
    Dispatch.DP_COMPUTE_METRIC: {"dispatch_fn": dispatch_dp_compute_data_proto, "collect_fn": collect_dp_compute},
    Dispatch.DIRECT_ROLLOUT_METHOD: {"dispatch_fn": dummy_direct_rollout_call,
                                     "collect_fn": dummy_direct_rollout_call},
}


def get_predefined_dispatch_fn(dispatch_mode):
    return DISPATCH_MODE_FN_REGISTRY[dispatch_mode]


def register_dispatch_mode(dispatch_mode_name: str, dispatch_fn, collect_fn):
    mode = Dispatch.register(dispatch_mode_name)
    assert mode not in DISPATCH_MODE_FN_REGISTRY, f"dispatch_mode_name {dispatch_mode_name} already exists"
    DISPATCH_MODE_FN_REGISTRY[mode] = {"dispatch_fn": dispatch_fn, "collect_fn": collect_fn}


def update_dispatch_mode(dispatch_mode, dispatch_fn, collect_fn):
    assert dispatch_mode in DISPATCH_MODE_FN_REGISTRY
    DISPATCH_MODE_FN_REGISTRY[dispatch_mode] = {"dispatch_fn": dispatch_fn, "collect_fn": collect_fn}


def get_predefined_execute_fn(execute_mode):
    return {Execute.ALL: {"execute_fn_name": "execute_all"},
            Execute.RANK_ZERO: {"execute_fn_name": "execute_rank_zero"}}[execute_mode]


def _check_dispatch_mode(dispatch_mode):
    assert isinstance(dispatch_mode, (Dispatch, dict)), f"dispatch_mode must be a Dispatch or a Dict. Got {dispatch_mode}"
    if isinstance(dispatch_mode, dict):
        for key in ("dispatch_fn", "collect_fn"):
            assert key in dispatch_mode, f"key {key} should be in dispatch_mode if it is a dictionary"


def _check_execute_mode(execute_mode):
    assert isinstance(execute_mode, Execute), f"execute_mode must be a Execute. Got {execute_mode}"


def _materialize_futures(*args, **kwargs):
    args = tuple(a.get() if isinstance(a, DataProtoFuture) else a for a in args)
    kwargs = {k: (v.get() if isinstance(v, DataProtoFuture) else v) for k, v in kwargs.items()}
    return args, kwargs


def register(dispatch_mode=Dispatch.ALL_TO_ALL, execute_mode=Execute.ALL, blocking=True, materialize_futures=True):
    """Mark a worker method as remotely callable and attach how its arguments are distributed.
    The worker-side wrapper strips auto-padding bookkeeping and resolves lazy inputs."""
    _check_dispatch_mode(dispatch_mode)
    _check_execute_mode(execute_mode)

    def decorator(func):
        if inspect.iscoroutinefunction(func):
            @wraps(func)
            async def inner(*args, **kwargs):
                if materialize_futures:
                    args, kwargs = _materialize_futures(*args, **kwargs)
                kwargs.pop(_PAD_KEY, None)
                return await func(*args, **kwargs)
        else:
            @wraps(func)
            def inner(*args, **kwargs):
                if materialize_futures:
                    args, kwargs = _materialize_futures(*args, **kwargs)
                kwargs.pop(_PAD_KEY, None)
                return func(*args, **kwargs)

        setattr(inner, MAGIC_ATTR, {"dispatch_mode": dispatch_mode, "execute_mode": execute_mode, "blocking": blocking})
        return inner

    return decorator
